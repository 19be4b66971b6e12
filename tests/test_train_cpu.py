"""End-to-end trainer on CPU: CLI run on a synthetic corpus, checkpoint layout, resume, HF export, and a
two-rank gloo run that must produce the same weights as the single-rank run of the same global batch."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from q38.data import DEFAULT_TOKENIZER, ROOT

TINY = ["--layers", "4", "--hidden", "32", "--heads", "2", "--kv_heads", "1", "--lin_k_heads", "1", "--lin_v_heads", "2",
        "--experts", "8", "--topk", "2", "--moe_ffn", "8", "--shared_ffn", "8", "--ngram_rows", "64", "--qsa_blocks", "2",
        "--mhc_iters", "3"]


def corpus(tmp_path, tokens=40000):
    from q38.data import prepare_synthetic
    path = tmp_path / "corpus" / "train.bin"
    prepare_synthetic(DEFAULT_TOKENIZER, path, tokens, mean_doc=96, seed=3)
    return path


def train_args(run_dir, data, steps, extra=()):
    return ["--run_dir", str(run_dir), "--data", str(data), "--val_data", "", "--tokenizer", str(DEFAULT_TOKENIZER),
            "--seq", "128", "--tokens", str(steps * 512), "--batch_tokens", "512", "--micro_bs", "2", "--eval_tokens", "1024",
            "--warmup", "2", "--log_every", "1", "--ckpt_every", "2", "--tensorboard", "0", "--device", "cpu",
            "--data_sampling", "shuffled_blocks", "--lr", "0.01", *TINY, *extra]


def test_cli_run_checkpoint_resume_and_export(tmp_path):
    from q38.train import main, parse_args, prepare_inputs
    data = corpus(tmp_path)
    run = tmp_path / "run"
    plan = main(train_args(run, data, 4) + ["--dry-run"])
    assert plan["steps"] == 4 and plan["accumulation"] == 2 and not run.exists()
    main(train_args(run, data, 4, ["--max_steps", "3"]))
    ck = torch.load(run / "ckpt.pt", map_location="cpu", weights_only=False)
    assert set(ck) == {"model", "opt", "step", "tok_seen", "rng", "rank_rng", "world"}
    assert ck["step"] == 2 and ck["tok_seen"] == 3 * 512 and ck["world"] == 1
    assert set(ck["opt"]) == {"adam", "muon"} and set(ck["rank_rng"][0]) == {"numpy", "torch", "cuda"}
    adam_state = ck["opt"]["adam"]["state"]
    assert set(adam_state[0]) == {"step", "exp_avg", "exp_avg_sq"} and float(adam_state[0]["step"]) == 3.0
    assert set(ck["opt"]["muon"]["state"][0]) == {"buf"}
    rows = (run / "training_metrics.csv").read_text().strip().splitlines()
    assert rows[0].split(",")[:4] == ["step", "tokens", "loss", "aux"] and len(rows) == 4
    for name in ("run_config.json", "summary.json", "flops.json", "hf/config.json", "hf/model.safetensors",
                 "hf/modeling_qwen3_8_moe.py", "hf/tokenizer.json"):
        assert (run / name).exists(), name
    # resume continues to step 3 and must refuse changed hyper-parameters
    main(train_args(run, data, 4))
    ck2 = torch.load(run / "ckpt.pt", map_location="cpu", weights_only=False)
    assert ck2["step"] == 3 and ck2["tok_seen"] == 4 * 512
    assert len((run / "training_metrics.csv").read_text().strip().splitlines()) == 5
    with pytest.raises(ValueError, match="Unsafe resume: lr changed"):
        main(train_args(run, data, 4, ["--lr", "0.02"]))
    # an uninterrupted 4-step run gives the same weights as 3 steps + resume
    straight = tmp_path / "straight"
    main(train_args(straight, data, 4))
    ck3 = torch.load(straight / "ckpt.pt", map_location="cpu", weights_only=False)
    for key in ck3["model"]:
        torch.testing.assert_close(ck2["model"][key], ck3["model"][key], rtol=0, atol=0, msg=key)


def test_unknown_preset_fields_are_rejected(tmp_path):
    from q38.train import parse_args
    bad = tmp_path / "config.json"
    bad.write_text(json.dumps(dict(compute=1e15, model=dict(hidden=32, bogus=1), train=dict(run_dir=str(tmp_path)))))
    with pytest.raises(SystemExit):
        parse_args(["--config", str(bad)])


def test_two_rank_gloo_matches_single_rank(tmp_path):
    data = corpus(tmp_path)
    single, double = tmp_path / "w1", tmp_path / "w2"
    env = {**os.environ, "PYTHONPATH": str(ROOT), "OMP_NUM_THREADS": "2"}
    base = [sys.executable, "-m", "q38.train"]
    subprocess.run(base + train_args(single, data, 2, ["--export_hf", "0"]), check=True, env=env, cwd=ROOT, capture_output=True)
    launch = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
              "--master-port", "29611", "-m", "q38.train"]
    done = subprocess.run(launch + train_args(double, data, 2, ["--export_hf", "0"]), env=env, cwd=ROOT, capture_output=True, text=True)
    assert done.returncode == 0, done.stderr[-3000:]
    a = torch.load(single / "ckpt.pt", map_location="cpu", weights_only=False)
    b = torch.load(double / "ckpt.pt", map_location="cpu", weights_only=False)
    assert b["world"] == 2 and len(b["rank_rng"]) == 2
    for key in a["model"]:
        torch.testing.assert_close(b["model"][key], a["model"][key], rtol=2e-4, atol=2e-6, msg=key)
    for index, entry in a["opt"]["adam"]["state"].items():
        torch.testing.assert_close(b["opt"]["adam"]["state"][index]["exp_avg"], entry["exp_avg"], rtol=2e-3, atol=1e-7)
    ma, mb = a["opt"]["muon"]["state"], b["opt"]["muon"]["state"]
    assert set(ma) == set(mb)
    for index in ma:
        torch.testing.assert_close(mb[index]["buf"], ma[index]["buf"], rtol=2e-3, atol=1e-7)
    rows_a = (single / "training_metrics.csv").read_text().strip().splitlines()
    rows_b = (double / "training_metrics.csv").read_text().strip().splitlines()
    for ra, rb in zip(rows_a[1:], rows_b[1:]):
        assert abs(float(ra.split(",")[2]) - float(rb.split(",")[2])) < 1e-4


def test_arena_ownership_is_balanced_and_complete(tiny_config):
    from q38.models import Q38ForCausalLM
    from q38.parallel import ParamArena
    model = Q38ForCausalLM(tiny_config)
    reference = {n: p.detach().clone() for n, p in model.named_parameters()}
    arena = ParamArena(model, "cpu", world=4)
    assert sorted(u.name for u in arena.units) == sorted(reference)
    for name, p in model.named_parameters():
        torch.testing.assert_close(p.detach(), reference[name], rtol=0, atol=0)
        assert p.data_ptr() >= arena.params.data_ptr() and p.grad.data_ptr() >= arena.grads.data_ptr()
    spans = sorted((u.offset, u.offset + u.numel) for u in arena.units)
    assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))
    for owner, (s, e) in enumerate(arena.segments):
        assert all(s <= u.offset and u.offset + u.numel <= e for u in arena.owned(owner))
    assert max(arena.load) <= 1.6 * (sum(arena.load) / 4)
    assert model.lm_head.weight.data_ptr() == model.model.embed_tokens.weight.data_ptr()
