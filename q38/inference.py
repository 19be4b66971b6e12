"""Inference entry point with the reference's name:  ``from q38.inference import optimize_for_inference``.

The reference patches a loaded model in place with its inference fast paths (Triton expert kernels, an FLA prefill path for the
Gated DeltaNet layers, fused mHC kernels, compiled norms; q38/inference.py:333-356) and returns counts for logging.  Here the
fast paths are not patches of a model but one process-wide kernel backend that the model file calls through named hooks whenever
its tensors are on a GPU, so this function installs that backend, puts the model in evaluation mode and reports what it covers in
the reference's vocabulary.  On a CPU model it changes nothing and says so.  `q38.evaluate` and the HF export
(`trust_remote_code` model file) use the same hooks.
"""
import torch


def compile_inference_norms(model):
    """Number of norm modules served by the kernel backend (the reference compiles them one by one; here they need no compilation)."""
    from .models import modeling
    kinds = tuple(getattr(modeling, name) for name in ("Qwen3_8MoeRMSNorm", "Qwen3_8MoeRMSNormGated") if hasattr(modeling, name))
    return sum(isinstance(m, kinds) for m in model.modules()) if kinds else 0


def optimize_for_inference(model):
    """Install the kernel backend for `model` (in place) and return what it serves:
    ``dict(experts=..., gated_deltanet=<layers>, mhc=<modules>, norms=<modules>, backend=<description or None>)``."""
    from .models import modeling
    model.eval()
    first = next(model.parameters())
    count = lambda name: sum(type(m).__name__ == name for m in model.modules())
    info = dict(experts="reference (PyTorch)", gated_deltanet=count("Qwen3_8MoeGatedDeltaNet"), mhc=count("MHC"),
                norms=compile_inference_norms(model), backend=None)
    if not first.is_cuda:
        return info
    from . import ops
    info["backend"] = ops.install()
    info["experts"] = "grouped tcgen05 kernels"
    inner = getattr(model, "model", None)
    if inner is not None and getattr(inner, "compute_dtype", None) is None and first.dtype == torch.float32:
        inner.compute_dtype = torch.bfloat16        # fp32 master weights: activations and tensor-core operands in bf16, as in training
    return info
