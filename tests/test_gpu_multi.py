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
