"""Python side of the hand-written sm_100a kernels.

`install()` loads the in-tree shared object (`q38/ops/_C.so`, built by ``__graft_entry__.build()``), runs a
short numerical self-check of the tensor-core GEMM layouts and installs the kernel backend into the model
file.  It raises when the extension is missing or the device is not a CUDA device: there is no silent
PyTorch fallback for a GPU run.  The individual wrappers below are what the optimizer and the gradient
engine call directly.
"""
import os
from pathlib import Path

import torch

_LIB = Path(__file__).resolve().parent / "_C.so"
# bf16 products go to the persistent kernel (one CTA per SM, epilogue overlapped with the next tile's MMAs);
# Q38_GEMM_PERSISTENT=0 selects the one-tile-per-CTA kernel.
PERSISTENT_GEMM = os.environ.get("Q38_GEMM_PERSISTENT", "1") != "0"
_loaded = False
_error_flags = {}


def loaded_library():
    return str(_LIB) if _loaded else None


def load():
    global _loaded
    if not _loaded:
        if not _LIB.exists():
            raise RuntimeError(f"q38.ops: {_LIB} is missing; build it with `python __graft_entry__.py` (nvcc, sm_100a)")
        torch.ops.load_library(str(_LIB))
        _loaded = True
    return torch.ops.q38


def error_flag(device=None):
    """Per-device int32 word into which kernels record a bounded-wait timeout or a failed self-check."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = device.index
    if key not in _error_flags:
        _error_flags[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_flags[key]


ERROR_NAMES = {1: "TMA stage never arrived", 2: "tensor core never released a stage", 3: "accumulator never became ready",
               4: "peer flag never arrived", 5: "index self-check failed"}


def check_errors():
    """Synchronise and raise if any kernel reported an error since the last check."""
    for flag in _error_flags.values():
        code = int(flag.item())
        if code:
            flag.zero_()
            raise RuntimeError(f"q38 kernel error {code}: {ERROR_NAMES.get(code, 'unknown')}")


def install(self_check=True):
    if not torch.cuda.is_available():
        raise RuntimeError("q38.ops.install: no CUDA device")
    load()
    from .backend import Backend
    from ..models import modeling
    backend = modeling.get_backend()
    if backend is None:
        backend = Backend(self_check=self_check)
        modeling.set_backend(backend)
    return backend.describe()


# ---- thin wrappers used outside the model ------------------------------------------------------------------
def gemm(a, b, out=None, a_mn_major=False, b_mn_major=False, alpha=1.0, accumulate=False, out_dtype=torch.bfloat16, splits=-1,
         addend=None, beta=0.0):
    """``out[b] (+)= alpha * A[b] @ B[b]^T (+ beta * addend[b])`` on the tcgen05 tensor cores.

    a: ``[batch, M, K]`` (K-major) or ``[batch, K, M]`` (``a_mn_major``); b likewise with N.  2-D inputs are treated as batch 1.
    ``splits`` (only with ``accumulate`` into fp32): -1 no split-K, 0 automatic, n > 0 that many K slices whose partial
    sums are added atomically (the summation order, hence the last bits, then vary from run to run)."""
    ops = load()
    squeeze = a.dim() == 2
    if squeeze:
        a, b = a.unsqueeze(0), b.unsqueeze(0)
    M = a.shape[2] if a_mn_major else a.shape[1]
    N = b.shape[2] if b_mn_major else b.shape[1]
    if out is None:
        out3 = torch.empty(a.shape[0], M, N, dtype=out_dtype, device=a.device)
    else:
        out3 = out.unsqueeze(0) if out.dim() == 2 else out
    if PERSISTENT_GEMM:
        if addend is not None and addend.dim() == 2:
            addend = addend.unsqueeze(0)
        ops.gemm_bf16_persistent(a, b, out3, a_mn_major, b_mn_major, float(alpha), bool(accumulate), error_flag(a.device), int(splits), addend, float(beta))
    else:
        if addend is not None:
            raise ValueError("the addend epilogue exists in the persistent kernel only")
        ops.gemm_bf16(a, b, out3, a_mn_major, b_mn_major, float(alpha), bool(accumulate), error_flag(a.device), int(splits))
    return out3[0] if squeeze else out3


def sum_squares(x):
    return load().sum_squares(x)


def adamw_flat(p, g, m, v, step, lr, wd, beta1, beta2, eps, grad_scale=None, shadow=None, hyper=None, err=None):
    """`hyper`: optional CUDA fp32 tensor {lr, 1/(1-b1^t), 1/sqrt(1-b2^t)} that overrides the step-dependent scalars, so that a
    captured launch can be replayed with new values.  `err`: device error word; when it is non-zero the kernel writes nothing."""
    if grad_scale is not None:
        grad_scale = grad_scale.reshape(1).float()
    load().adamw_flat(p, g, m, v, shadow, grad_scale, int(step), float(lr), float(wd), float(beta1), float(beta2), float(eps), hyper, err)


def muon_batched_step(views, per_call, lr, momentum, weight_decay, ns_steps, scale, grad_scale=None):
    """`lr` is a float or a 0-dim CUDA tensor (replayable step)."""
    from .muon_gpu import batched_step
    batched_step(views, per_call, lr, momentum, weight_decay, ns_steps, scale, grad_scale)


def launch_count():
    """Kernels launched by this library since it was loaded."""
    return int(load().launch_count())
