"""Corpus preparation on a synthetic shard (counterpart of the reference's tests/test_data.py)."""
import json
import shutil
import subprocess
import sys

import numpy as np
import pytest

from q38.data import DEFAULT_TOKENIZER, ROOT, load_tokenizer, open_tokens, tokenizer_sha256


def test_corpus_counts_cache_reuse_and_rejection(tmp_path):
    data = tmp_path / "source"
    data.mkdir()
    (data / "dolma3_mix_50B-00000.jsonl").write_text(
        "".join(json.dumps({"text": f"Example document {i}: test English and 中文训练数据。"}) + "\n" for i in range(100)))
    out = tmp_path / "tokens"
    cmd = [sys.executable, "-m", "q38.data", "corpus", "--tokenizer", str(DEFAULT_TOKENIZER), "--data_dir", str(data),
           "--out", str(out), "--every", "2", "--sub", "2", "--workers", "2", "--val_tokens", "64"]
    subprocess.run(cmd, check=True, capture_output=True, cwd=ROOT)
    meta = json.loads((out / "meta.json").read_text())
    assert meta["docs"] == 50 and meta["dtype"] == "<u4"
    assert (out / "val.bin").stat().st_size == 64 * 4
    assert (out / "train.bin").stat().st_size // 4 + 64 == meta["tokens"]
    tok = load_tokenizer(DEFAULT_TOKENIZER)
    ids = np.concatenate([np.fromfile(out / "train.bin", dtype="<u4"), np.fromfile(out / "val.bin", dtype="<u4")])
    assert ids.max() < len(tok) and np.count_nonzero(ids == tok.eos_token_id) == 50
    before = (out / "train.bin").read_bytes()
    subprocess.run(cmd, check=True, capture_output=True, cwd=ROOT)
    assert (out / "train.bin").read_bytes() == before
    changed = list(cmd)
    changed[changed.index("--every") + 1] = "3"
    failed = subprocess.run(changed, capture_output=True, text=True, cwd=ROOT)
    assert failed.returncode != 0 and "Part cache mismatch" in failed.stderr
    other = tmp_path / "other_tok"
    shutil.copytree(DEFAULT_TOKENIZER, other)
    with (other / "tokenizer.json").open("a") as f:
        f.write("\n")
    changed = list(cmd)
    changed[changed.index("--tokenizer") + 1] = str(other)
    failed = subprocess.run(changed, capture_output=True, text=True, cwd=ROOT)
    assert failed.returncode != 0 and "Part cache mismatch" in failed.stderr
    assert len(open_tokens(out / "train.bin", tokenizer_sha256(DEFAULT_TOKENIZER))) == meta["tokens"] - 64
    with pytest.raises(ValueError, match="tokenizer mismatch"):
        open_tokens(out / "train.bin", tokenizer_sha256(other))


@pytest.mark.parametrize("layout", ["plain", "spec"])
def test_llm_pt_manifest_tokenizer_check(tmp_path, layout):
    sha = tokenizer_sha256(DEFAULT_TOKENIZER)
    block = {"tokenizer": {"files": {"tokenizer.json": sha}}}
    np.arange(16, dtype="<u4").tofile(tmp_path / "valid.bin")
    (tmp_path / "manifest.json").write_text(json.dumps(block if layout == "plain" else {"spec": block}))
    assert len(open_tokens(tmp_path / "valid.bin", sha)) == 16
    with pytest.raises(ValueError, match="tokenizer mismatch"):
        open_tokens(tmp_path / "valid.bin", "0" * 64)


def test_synthetic_stream(tmp_path):
    from q38.data import main
    main(["synthetic", "--out", str(tmp_path / "s" / "train.bin"), "--tokens", "20000", "--mean_doc", "100"])
    ids = np.fromfile(tmp_path / "s" / "train.bin", dtype="<u4")
    assert len(ids) == 20000 and ids.max() < 10112 and 100 < np.count_nonzero(ids == 53) < 400
    assert (tmp_path / "s" / "train.bin").stat().st_size % 4 == 0


def test_evaluator_packing(tmp_path):
    """JSONL -> packed token / text-mask files -> fixed-length batches whose labels skip document separators and padding
    (q38.evaluate; reference: q38/evaluate.py:26-71)."""
    import json
    import numpy as np
    from transformers import PreTrainedTokenizerFast
    from q38.data import DEFAULT_TOKENIZER
    from q38.evaluate import pack_jsonl, packed_batch
    tok = PreTrainedTokenizerFast.from_pretrained(str(DEFAULT_TOKENIZER), local_files_only=True)
    texts = ["hello world, this is a test.", "second document", "third one is a little longer than the others"]
    path = tmp_path / "eval.jsonl"
    path.write_text("".join(json.dumps({"text": t}) + "\n" for t in texts) + "\n")
    meta = pack_jsonl(path, tok, tmp_path)
    tokens = np.fromfile(tmp_path / "tokens.bin", dtype=np.int32)
    is_text = np.fromfile(tmp_path / "is_text.bin", dtype=np.bool_)
    assert meta["total_bytes"] == sum(len(t.encode()) for t in texts)
    assert len(tokens) == len(is_text) == meta["total_tokens"] + len(texts)
    assert int((~is_text).sum()) == len(texts) and tokens[0] == tok.eos_token_id and not is_text[0]
    seq = 8
    n_seq = -(-(len(tokens) - 1) // seq)
    x, y = packed_batch(tokens, is_text, 0, n_seq, seq, meta["pad_token_id"])
    assert x.shape == y.shape == (n_seq, seq)
    flat_x, flat_y = x.reshape(-1), y.reshape(-1)
    n = len(tokens) - 1
    assert np.array_equal(flat_x[:n], tokens[:n]) and (flat_x[n:] == meta["pad_token_id"]).all() and (flat_y[n:] == -100).all()
    scored = flat_y[:n] != -100
    assert np.array_equal(scored, is_text[1:n + 1]) and np.array_equal(flat_y[:n][scored], tokens[1:n + 1][scored])
    assert int(scored.sum()) == meta["total_tokens"]                   # every text token is a label exactly once
