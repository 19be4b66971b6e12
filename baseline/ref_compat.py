"""Environment shims that let the UNMODIFIED reference tree (a byte-for-byte copy under ``baseline/_ref``) import
on the transformers release of this image.

The reference vendors a model file written against transformers 5.19; this image ships 5.5.  Four names are missing or
have a different signature.  They are added to *transformers* here; no file of the reference is touched.

1. ``transformers.integrations.use_kernel_func_from_hub_with_fallback(name, package)`` – decorator factory.  When
   ``package`` is importable and exports ``name`` the decorated function dispatches CUDA inputs to that package's
   kernel and everything else to the decorated PyTorch fallback (the reference's trainer checks that fla's kernel
   sits in the closure, q38/train.py ``gdn_kernel``).
2. ``transformers.integrations.accelerate.force_accelerate_hooks(attr)`` – decorator factory that returns the
   function unchanged (no accelerate offloading hooks are used here).
3. ``transformers.masking_utils.create_recurrent_attention_mask`` – imported by the model file, never called by the
   Q38 trunk; a stub that raises if it ever is.
4. ``PreTrainedModel._initialize_weights`` – accept the ``is_custom_code=`` keyword the reference passes and forward
   it as this release's ``is_remote_code``.

5. torch 2.11's Inductor picks ``FlexBwDConfig(64, 128, 128, 64)`` as the only flex-attention backward candidate on
   sm_100 and then drops it because the reference's sparse block size (64) is not a multiple of 128, so the stock QSA
   backward fails to compile ("NoValidChoicesError: No choices exist for backend", target flex_attention_backward).
   The candidate list gets the (64, 64, 64, 64, stages 2, warps 4) entry that the same table uses on sm_8x, where the
   reference was developed; the block sizes actually compiled are the ones the reference passes in ``kernel_options``.

``activate()`` applies the shims once and puts ``baseline/_ref`` first on ``sys.path`` so that ``import q38`` is the
reference's package.  It must run in a process that never imports this repository's own ``q38``.
"""
import functools
import importlib
import inspect
import os
import sys
from pathlib import Path

REF_ROOT = Path(__file__).resolve().parent / "_ref"
_DONE = False


def available():
    return (REF_ROOT / "q38" / "train.py").is_file()


def _first_tensor_is_cuda(args, kwargs):
    import torch
    for v in list(args) + list(kwargs.values()):
        if isinstance(v, torch.Tensor):
            return v.is_cuda
    return False


def _kernel_or_fallback(name, package):
    locations = {"fla": ("fla.ops.gated_delta_rule",), "causal_conv1d": ("causal_conv1d",)}

    def decorate(fallback):
        kernel = None
        for module_name in locations.get(package, (package,)):
            try:
                kernel = getattr(importlib.import_module(module_name), name)
                break
            except Exception:
                kernel = None
        if kernel is None:
            return fallback

        @functools.wraps(fallback)
        def dispatch(*args, **kwargs):
            if _first_tensor_is_cuda(args, kwargs):
                return kernel(*args, **kwargs)
            return fallback(*args, **kwargs)
        return dispatch
    return decorate


def _identity_decorator_factory(*_args, **_kwargs):
    def decorate(fn):
        return fn
    return decorate


def _missing_mask(*_args, **_kwargs):
    raise NotImplementedError("create_recurrent_attention_mask is not part of this transformers release")


def _add_flex_backward_candidate():
    try:
        from torch._inductor.template_heuristics import triton as heuristics
    except Exception:
        return
    cls = getattr(heuristics, "CUDAConfigHeuristic", None)
    if cls is None or getattr(cls, "_q38_ref_patch", False):
        return
    original = cls.get_flex_attn_bwd_configs

    def get_flex_attn_bwd_configs(self, head_dim, dtype):
        configs = list(original(self, head_dim, dtype))
        extra = heuristics.FlexBwDConfig(64, 64, 64, 64, 2, 4)
        if extra not in configs:
            configs.append(extra)
        return configs

    cls.get_flex_attn_bwd_configs = get_flex_attn_bwd_configs
    cls._q38_ref_patch = True


def activate():
    global _DONE
    if _DONE:
        return
    if not available():
        raise FileNotFoundError(f"reference tree not found under {REF_ROOT}")
    if "q38" in sys.modules and not str(getattr(sys.modules["q38"], "__file__", "")).startswith(str(REF_ROOT)):
        raise RuntimeError("another q38 package is already imported in this process")
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
    import transformers.integrations as integrations
    import transformers.integrations.accelerate as accelerate_integration
    import transformers.masking_utils as masking_utils
    from transformers.modeling_utils import PreTrainedModel
    if not hasattr(integrations, "use_kernel_func_from_hub_with_fallback"):
        integrations.use_kernel_func_from_hub_with_fallback = _kernel_or_fallback
    if not hasattr(accelerate_integration, "force_accelerate_hooks"):
        accelerate_integration.force_accelerate_hooks = _identity_decorator_factory
    if not hasattr(masking_utils, "create_recurrent_attention_mask"):
        masking_utils.create_recurrent_attention_mask = _missing_mask
    original = PreTrainedModel._initialize_weights
    if "is_custom_code" not in inspect.signature(original).parameters:
        def _initialize_weights(self, module, is_remote_code=False, is_custom_code=None):
            return original(self, module, is_remote_code=bool(is_custom_code) if is_custom_code is not None else is_remote_code)
        PreTrainedModel._initialize_weights = _initialize_weights
    _add_flex_backward_candidate()
    sys.path.insert(0, str(REF_ROOT))
    _DONE = True
