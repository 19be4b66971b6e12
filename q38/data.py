"""Token corpora: flat little-endian uint32 files, one EOS after every document.

  python -m q38.data corpus --out DIR [--data_dir D --every 12 --sub 6 --workers 8 --val_tokens N]
      Sample 1/every of the documents of each ``dolma3_mix_50B-*.jsonl[.zst]`` shard, tokenise them in
      ``sub`` interleaved sub-tasks per shard (each sub-task streams into its own part file, finished
      parts are reused on a rerun), concatenate the parts in a seeded random order into ``train.bin``
      and cut ``val.bin`` from the head of the first part.
  python -m q38.data sample --out FILE [--source S --tokens N]
      A small token file from the head of one JSONL shard, for smoke runs.
  python -m q38.data synthetic --out FILE --tokens N [--mean_doc 1024 --zipf 0]
      A synthetic packed stream (uniform or Zipf ids, EOS at geometric document boundaries).

`open_tokens` memory-maps a token file and refuses it when a neighbouring ``meta.json`` /
``parts_manifest.json`` / ``manifest.json`` records a different ``tokenizer.json`` sha256.
File formats and checks follow the reference (q38/data.py:25-165).
"""
import argparse
import hashlib
import json
import os
import random
import subprocess
import time
from multiprocessing import Pool
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[1]
TOKEN_DTYPE = np.dtype("<u4")
DEFAULT_TOKENIZER = ROOT / "tokenizer/gzy_10k"
SHARED_CACHE = Path("/home/shared/qwen35_moe_sparse/cache/isoflops-gzy10k-16b-v1")
DEFAULT_DATA = SHARED_CACHE / "train.bin"
DEFAULT_VAL_DATA = SHARED_CACHE / "valid.bin"
MAX_CHARS_PER_CALL = 100_000          # very long documents are tokenised in slices of this many characters
CHUNK_CHARS = MAX_CHARS_PER_CALL      # the reference's name for the same constant (q38/data.py:30)
DOCS_PER_CALL = 512
METADATA_FILES = ("meta.json", "parts_manifest.json", "manifest.json")


def load_tokenizer(path):
    """`tokenizer.json` loaded verbatim (AutoTokenizer would substitute a model-type specific pre-tokenizer)."""
    from transformers import PreTrainedTokenizerFast
    return PreTrainedTokenizerFast.from_pretrained(str(path), local_files_only=True)


def tokenizer_sha256(path):
    return hashlib.sha256((Path(path) / "tokenizer.json").read_bytes()).hexdigest()


def recorded_tokenizer_sha(meta):
    """The tokenizer.json digest a metadata file records: ``tokenizer_sha256`` (this framework) or
    ``[spec.]tokenizer.files["tokenizer.json"]`` (llm_pt manifests)."""
    if "tokenizer_sha256" in meta:
        return meta["tokenizer_sha256"]
    block = meta.get("tokenizer")
    if not isinstance(block, dict):
        block = meta.get("spec", {}).get("tokenizer", {})
    return block.get("files", {}).get("tokenizer.json")


def open_tokens(path, tokenizer_sha=None):
    path = Path(path)
    if tokenizer_sha:
        for name in METADATA_FILES:
            meta = path.parent / name
            if meta.exists() and recorded_tokenizer_sha(json.loads(meta.read_text())) not in (None, tokenizer_sha):
                raise ValueError("Corpus tokenizer mismatch: prepare fresh data for this tokenizer")
    if path.stat().st_size % TOKEN_DTYPE.itemsize:
        raise ValueError("Misaligned binary token file")
    return np.memmap(path, dtype=TOKEN_DTYPE, mode="r")


def _slices(text):
    return [text[i:i + MAX_CHARS_PER_CALL] for i in range(0, max(1, len(text)), MAX_CHARS_PER_CALL)]


_WORKER_TOKENIZER = None


def _worker_init(tokenizer_path):
    global _WORKER_TOKENIZER
    _WORKER_TOKENIZER = load_tokenizer(tokenizer_path)


def _tokenize_part(task):
    """One sub-task: every `stride`-th line (phase `phase`) of a shard -> part file + ``.ok`` marker."""
    shard, stride, phase, part = task
    marker = part + ".ok"
    if os.path.exists(marker) and os.path.exists(part):
        return part, 0, 0
    reader = subprocess.Popen(["zstd", "-dc", shard] if shard.endswith(".zst") else ["cat", shard], stdout=subprocess.PIPE)
    tok, eos = _WORKER_TOKENIZER, _WORKER_TOKENIZER.eos_token_id
    docs = tokens = 0
    pending = []
    with open(part, "wb") as sink:
        def drain():
            nonlocal docs, tokens
            for ids in tok(pending, add_special_tokens=False)["input_ids"]:
                np.asarray(ids + [eos], dtype=TOKEN_DTYPE).tofile(sink)
                docs += 1
                tokens += len(ids) + 1
            pending.clear()

        for line_no, line in enumerate(reader.stdout):
            if (line_no + phase) % stride:
                continue
            for piece in _slices(json.loads(line)["text"]):
                pending.append(piece)
                if len(pending) >= DOCS_PER_CALL:
                    drain()
        if pending:
            drain()
    status = reader.wait()
    if status:
        raise RuntimeError(f"Failed reading {shard}: exit {status}")
    Path(marker).write_text(f"{docs} {tokens}")
    return part, docs, tokens


def prepare_corpus(tokenizer, out, data_dir, every=12, sub=6, workers=8, val_tokens=30_000_000, seed=0):
    started = time.time()
    out = Path(out)
    parts_dir = out / "parts"
    parts_dir.mkdir(parents=True, exist_ok=True)
    # A part cache is only reusable under the same tokenizer and sampling rule.
    manifest = dict(every=every, sub=sub, data_dir=os.path.realpath(data_dir), tokenizer_sha256=tokenizer_sha256(tokenizer))
    manifest_path = out / "parts_manifest.json"
    if manifest_path.exists():
        if json.loads(manifest_path.read_text()) != manifest:
            raise ValueError("Part cache mismatch: choose a fresh --out directory")
    elif any(parts_dir.iterdir()):
        raise ValueError("Unverified existing parts: choose a fresh --out directory")
    else:
        manifest_path.write_text(json.dumps(manifest, indent=2))
    shards = sorted(name for name in os.listdir(data_dir)
                    if name.startswith("dolma3_mix_50B-") and name.endswith((".jsonl.zst", ".jsonl")))
    if not shards:
        raise ValueError("No dolma3_mix_50B JSONL shards found")
    tasks = [(os.path.join(data_dir, shard), every * sub, phase, str(parts_dir / f"{shard.split('.jsonl')[0]}_{phase}.bin"))
             for shard in shards for phase in range(sub)]
    with Pool(min(workers, len(tasks)), initializer=_worker_init, initargs=(str(tokenizer),)) as pool:
        for done, (part, docs, tokens) in enumerate(pool.imap_unordered(_tokenize_part, tasks), 1):
            print(f"part {done}/{len(tasks)} {os.path.basename(part)}: {docs} docs, {tokens / 1e6:.1f}M tokens, "
                  f"{time.time() - started:.0f}s", flush=True)
    parts = [task[3] for task in tasks]
    random.Random(seed).shuffle(parts)
    stats = [tuple(map(int, Path(part + ".ok").read_text().split())) for part in parts]
    n_docs, n_tokens = sum(s[0] for s in stats), sum(s[1] for s in stats)
    if n_tokens <= val_tokens:
        raise ValueError("Corpus is smaller than val_tokens")
    if os.path.getsize(parts[0]) // TOKEN_DTYPE.itemsize < val_tokens:
        raise ValueError("First shuffled part must contain val_tokens; reduce --val_tokens")
    with open(out / "val.bin", "wb") as val, open(out / "train.bin", "wb") as train:
        head = np.fromfile(parts[0], dtype=TOKEN_DTYPE)
        head[:val_tokens].tofile(val)
        head[val_tokens:].tofile(train)
        for part in parts[1:]:
            with open(part, "rb") as source:
                while block := source.read(1 << 26):
                    train.write(block)
    meta = dict(shards=shards, every=every, sub=sub, docs=n_docs, tokens=n_tokens, val_tokens=val_tokens,
                tokenizer=str(tokenizer), tokenizer_sha256=manifest["tokenizer_sha256"], dtype=TOKEN_DTYPE.str,
                part_order=[os.path.basename(part) for part in parts])
    (out / "meta.json").write_text(json.dumps(meta, indent=1))
    print(f"{n_docs} docs, {n_tokens / 1e9:.3f}B tokens; train.bin {os.path.getsize(out / 'train.bin') / 1e9:.2f} GB, "
          f"val.bin {os.path.getsize(out / 'val.bin') / 1e6:.0f} MB, {time.time() - started:.0f}s", flush=True)


def prepare_sample(tokenizer, out, source, tokens=262144):
    tok = load_tokenizer(tokenizer)
    out = Path(out)
    out.parent.mkdir(parents=True, exist_ok=True)
    written = 0
    with open(source) as lines, out.open("wb") as sink:
        for line in lines:
            for piece in _slices(json.loads(line)["text"]):
                ids = tok.encode(piece, add_special_tokens=False) + [tok.eos_token_id]
                np.asarray(ids, dtype=TOKEN_DTYPE).tofile(sink)
                written += len(ids)
                if written >= tokens:
                    break
            if written >= tokens:
                break
    if written < tokens:
        raise ValueError(f"Source exhausted: {written} < {tokens}")
    meta = dict(source=str(source), tokens=written, path=str(out), dtype=TOKEN_DTYPE.str, tokenizer=str(tokenizer),
                tokenizer_sha256=tokenizer_sha256(tokenizer))
    (out.parent / "meta.json").write_text(json.dumps(meta, indent=2) + "\n")
    print(json.dumps(meta))
    return meta


def prepare_synthetic(tokenizer, out, tokens, mean_doc=1024, zipf=0.0, seed=0):
    from .utils.synthetic import packed_stream
    out = Path(out)
    out.parent.mkdir(parents=True, exist_ok=True)
    tok = load_tokenizer(tokenizer)
    stream = packed_stream(tokens, len(tok), tok.eos_token_id, mean_doc=mean_doc, zipf=zipf, seed=seed)
    stream.astype(TOKEN_DTYPE).tofile(out)
    meta = dict(source="synthetic", tokens=int(tokens), path=str(out), dtype=TOKEN_DTYPE.str, mean_doc=mean_doc, zipf=zipf,
                seed=seed, tokenizer=str(tokenizer), tokenizer_sha256=tokenizer_sha256(tokenizer))
    (out.parent / "meta.json").write_text(json.dumps(meta, indent=2) + "\n")
    print(json.dumps(meta))
    return meta


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    commands = ap.add_subparsers(dest="cmd", required=True)
    corpus = commands.add_parser("corpus", help="sampled training corpus -> train.bin / val.bin")
    corpus.add_argument("--out", required=True)
    corpus.add_argument("--tokenizer", default=str(DEFAULT_TOKENIZER))
    corpus.add_argument("--data_dir", default="/home/shared/data")
    for name, default in (("every", 12), ("sub", 6), ("workers", 8), ("val_tokens", 30_000_000), ("seed", 0)):
        corpus.add_argument(f"--{name}", type=int, default=default)
    sample = commands.add_parser("sample", help="small token sample for smoke tests")
    sample.add_argument("--out", required=True)
    sample.add_argument("--tokenizer", default=str(DEFAULT_TOKENIZER))
    sample.add_argument("--source", default="/home/shared/data/dolma3_mix_50B-00000.jsonl")
    sample.add_argument("--tokens", type=int, default=262144)
    synth = commands.add_parser("synthetic", help="synthetic packed stream")
    synth.add_argument("--out", required=True)
    synth.add_argument("--tokenizer", default=str(DEFAULT_TOKENIZER))
    synth.add_argument("--tokens", type=int, required=True)
    synth.add_argument("--mean_doc", type=int, default=1024)
    synth.add_argument("--zipf", type=float, default=0.0)
    synth.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    if a.cmd == "corpus":
        if min(a.every, a.sub, a.workers, a.val_tokens) < 1:
            ap.error("sampling, workers and val_tokens must be positive")
        prepare_corpus(a.tokenizer, a.out, a.data_dir, a.every, a.sub, a.workers, a.val_tokens, a.seed)
    elif a.cmd == "sample":
        prepare_sample(a.tokenizer, a.out, a.source, a.tokens)
    else:
        prepare_synthetic(a.tokenizer, a.out, a.tokens, a.mean_doc, a.zipf, a.seed)


if __name__ == "__main__":
    main()
