"""Host-side failure handling, on CPU with gloo ranks (no GPU is faulted, trapped or hung anywhere):

* a rank that leaves between two steps makes the remaining rank raise within the process-group timeout instead of waiting
  forever (the reference relies on NCCL's collective timeout for the same event, q38/train.py:472-479);
* a checkpoint write that fails half-way never replaces ``ckpt.pt``, and a truncated ``ckpt.pt.tmp`` left behind by a killed
  process is ignored by the next resume (q38/train.py:540-541 of the reference writes tmp + rename for the same reason);
* a run resumed with a different world size keeps the deterministic shuffled-block stream (q38/train.py:518-524).
"""
import os
import subprocess
import sys
import textwrap

import pytest
import torch

from q38.data import DEFAULT_TOKENIZER, ROOT
from test_train_cpu import corpus, train_args

LEAVER = textwrap.dedent('''
    import datetime, os, sys, time
    from types import SimpleNamespace
    import torch, torch.distributed as dist
    sys.path.insert(0, os.environ["Q38_ROOT"])
    from q38.presets import model_config
    from q38.train import TRAIN_DEFAULTS, Trainer
    rank = int(os.environ["RANK"])
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=8))
    cfg = model_config(dict(layers=4, hidden=32, heads=2, kv_heads=1, lin_k_heads=1, lin_v_heads=2, experts=8, topk=2, moe_ffn=8, shared_ffn=8,
                            ngram_rows=64, qsa_blocks=2, mhc_iters=3), 128, 128, eos_token_id=0)
    torch.manual_seed(0)
    args = SimpleNamespace(**{**TRAIN_DEFAULTS, "aux_coef": 0.001, "lr": 1e-2, "grad_sync": "collective", "micro_bs": 1, "seq": 128})
    trainer = Trainer(cfg, args, torch.device("cpu"), rank, 2)
    x = torch.randint(1, 128, (1, 128)); y = x.roll(-1, 1)
    trainer.read_step(trainer.train_step([(x, y)], lr=1e-2))
    dist.barrier()
    if rank == 1:
        os._exit(0)                      # leaves between steps: none of its collectives is in flight
    started = time.time()
    try:
        trainer.read_step(trainer.train_step([(x, y)], lr=1e-2))
    except Exception as exc:             # gloo reports the closed connection or the timeout as a RuntimeError
        print(f"PEER_LOST_DETECTED after {time.time() - started:.1f}s: {type(exc).__name__}", flush=True)
        os._exit(0)
    print("STEP_COMPLETED_WITHOUT_PEER", flush=True)
    os._exit(3)
''')


def test_rank_that_leaves_between_steps_is_detected(tmp_path):
    script = tmp_path / "leaver.py"
    script.write_text(LEAVER)
    env = {**os.environ, "Q38_ROOT": str(ROOT), "OMP_NUM_THREADS": "2"}
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29621", str(script)]
    done = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert "PEER_LOST_DETECTED" in done.stdout and "STEP_COMPLETED_WITHOUT_PEER" not in done.stdout, done.stdout[-1500:] + done.stderr[-3000:]


def test_failed_checkpoint_write_keeps_the_previous_checkpoint(tmp_path, monkeypatch):
    from q38 import train
    path = tmp_path / "ckpt.pt"
    train.write_checkpoint({"step": 1, "payload": torch.arange(10)}, str(path))
    good = path.read_bytes()

    def failing_save(state, target):
        with open(target, "wb") as f:
            f.write(b"truncated")
        raise OSError("disk full")

    monkeypatch.setattr(train.torch, "save", failing_save)
    with pytest.raises(OSError):
        train.write_checkpoint({"step": 2}, str(path))
    assert path.read_bytes() == good and not (tmp_path / "ckpt.pt.tmp").exists()
    assert torch.load(path, weights_only=False)["step"] == 1


def test_resume_ignores_a_truncated_temporary_checkpoint(tmp_path):
    from q38.train import main
    data = corpus(tmp_path)
    run = tmp_path / "run"
    main(train_args(run, data, 4, ["--max_steps", "2", "--export_hf", "0"]))
    (run / "ckpt.pt.tmp").write_bytes(b"\x80\x02 this is what a killed writer leaves behind")
    main(train_args(run, data, 4, ["--export_hf", "0"]))
    ck = torch.load(run / "ckpt.pt", map_location="cpu", weights_only=False)
    assert ck["step"] == 3 and ck["tok_seen"] == 4 * 512


def test_resume_with_another_world_size_keeps_the_shuffled_stream(tmp_path):
    data = corpus(tmp_path)
    straight, resumed = tmp_path / "straight", tmp_path / "resumed"
    env = {**os.environ, "PYTHONPATH": str(ROOT), "OMP_NUM_THREADS": "2"}
    base = [sys.executable, "-m", "q38.train"]
    subprocess.run(base + train_args(straight, data, 4, ["--export_hf", "0"]), check=True, env=env, cwd=ROOT, capture_output=True)
    subprocess.run(base + train_args(resumed, data, 4, ["--export_hf", "0", "--max_steps", "2"]), check=True, env=env, cwd=ROOT, capture_output=True)
    launch = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29623",
              "-m", "q38.train"]
    done = subprocess.run(launch + train_args(resumed, data, 4, ["--export_hf", "0"]), env=env, cwd=ROOT, capture_output=True, text=True)
    assert done.returncode == 0 and "World size changed" in done.stdout, done.stdout[-1500:] + done.stderr[-3000:]
    a = torch.load(straight / "ckpt.pt", map_location="cpu", weights_only=False)
    b = torch.load(resumed / "ckpt.pt", map_location="cpu", weights_only=False)
    assert a["step"] == b["step"] == 3 and b["world"] == 2 and a["tok_seen"] == b["tok_seen"]
    for key in a["model"]:
        torch.testing.assert_close(b["model"][key], a["model"][key], rtol=2e-4, atol=2e-6, msg=key)
