"""Multi-GPU checks (need at least two GPUs on the box; skipped otherwise): the peer-memory gradient path against the
library-collective path, replica bit-identity, and the bounded wait of the cross-GPU barrier kernel."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def test_barrier_wait_is_bounded_and_reports():
    """A flag that nothing sets: the kernel gives up after its clock budget, records an error and the context stays usable."""
    from q38 import ops
    lib = ops.load()
    dev = torch.device("cuda", 0)
    flags = lib.p2p_alloc(256, 0).view(torch.int64)
    err = ops.error_flag(dev)
    err.zero_()
    lib.p2p_barrier(flags, [flags.data_ptr(), flags.data_ptr()], 0, 5, 0.05, err)     # slot 1 never reaches epoch 5
    torch.cuda.synchronize()
    assert int(err.item()) == 4
    with pytest.raises(RuntimeError, match="peer flag"):
        ops.check_errors()
    assert int(flags[0].item()) == 5 and torch.ones(4, device=dev).sum().item() == 4.0        # the device still works


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_memory_gradient_path_matches_collectives():
    world = min(torch.cuda.device_count(), 8)
    env = {**os.environ, "NCCL_NVLS_ENABLE": "0"}
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", "29655", str(ROOT / "tests" / "multi_gpu_worker.py")]
    done = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=900)
    assert done.returncode == 0 and "MULTI_GPU_OK" in done.stdout, done.stdout[-2000:] + done.stderr[-4000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_late_rank_aborts_the_step_cleanly():
    """A rank that stalls on the host for longer than the bounded barrier wait: every rank raises, nothing is updated."""
    world = min(torch.cuda.device_count(), 4)
    # plain peer loads and IPC allocations: a failure test must not run with memory bound to an NVLink multicast object
    env = {**os.environ, "NCCL_NVLS_ENABLE": "0", "Q38_PEER_WAIT_SECONDS": "1", "Q38_PEER_ALLOC": "ipc", "Q38_RS_ALGO": "pull"}
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", "29657", str(ROOT / "tests" / "late_rank_worker.py")]
    done = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0 and "LATE_RANK_OK" in done.stdout, done.stdout[-2000:] + done.stderr[-4000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_expert_parallel_training_run_reaches_validation_checkpoint_and_export(tmp_path):
    """`python -m q38.train --expert_parallel 1` on two GPUs: validation on every rank (replicated expert path on gathered
    experts), periodic and final checkpoint, final evaluation and the HF export."""
    from q38.data import DEFAULT_TOKENIZER, prepare_synthetic
    data, val = tmp_path / "corpus" / "train.bin", tmp_path / "corpus" / "valid.bin"
    prepare_synthetic(DEFAULT_TOKENIZER, data, 60000, mean_doc=96, seed=3)
    prepare_synthetic(DEFAULT_TOKENIZER, val, 6000, mean_doc=96, seed=4)
    run = tmp_path / "run"
    args = ["--run_dir", str(run), "--data", str(data), "--val_data", str(val), "--tokenizer", str(DEFAULT_TOKENIZER), "--seq", "256",
            "--tokens", str(4 * 2048), "--batch_tokens", "2048", "--micro_bs", "2", "--eval_tokens", "1024", "--final_eval_tokens", "1500",
            "--eval_sampling", "sequential", "--warmup", "1", "--log_every", "1", "--eval_every", "2", "--ckpt_every", "2", "--tensorboard", "0",
            "--lr", "0.003", "--expert_parallel", "1", "--layers", "4", "--hidden", "128", "--heads", "4", "--kv_heads", "2", "--lin_k_heads", "2",
            "--lin_v_heads", "6", "--experts", "8", "--topk", "2", "--moe_ffn", "32", "--shared_ffn", "32", "--ngram_rows", "1024", "--qsa_blocks", "2",
            "--mhc_iters", "3"]
    env = {**os.environ, "NCCL_NVLS_ENABLE": "0", "PYTHONPATH": str(ROOT)}
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29659",
           "-m", "q38.train", *args]
    done = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=900)
    assert done.returncode == 0 and "DONE" in done.stdout, done.stdout[-2000:] + done.stderr[-4000:]
    rows = (run / "training_metrics.csv").read_text().strip().splitlines()
    assert len(rows) == 5 and rows[-1].split(",")[8] != "" and rows[3].split(",")[8] != ""       # validation at step 2 and at the last step
    for name in ("ckpt.pt", "final_eval.json", "summary.json", "hf/model.safetensors"):
        assert (run / name).exists(), name
    first, last = float(rows[1].split(",")[2]), float(rows[-1].split(",")[2])
    assert last < first
