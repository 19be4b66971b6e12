"""Model package: the Q38 module tree lives in ``hf_export/modeling_qwen3_8_moe.py`` so that the very
same file can be shipped inside HF exports; this package re-exports it for in-repo use."""
import hashlib
from pathlib import Path

from .hf_export import modeling_qwen3_8_moe as modeling
from .hf_export.configuration_qwen3_8_moe import Qwen3_8MoeTextConfig
from .hf_export.modeling_qwen3_8_moe import Q38ForCausalLM, RouterStats, set_backend, get_backend

EXPORT_FILES = ("modeling_qwen3_8_moe.py", "configuration_qwen3_8_moe.py")


def source_info():
    """sha256 of the model source files, recorded in ``run_config.json`` (reference:
    q38/models/qwen3_8_moe/__init__.py:15-22)."""
    root = Path(__file__).resolve().parent / "hf_export"
    return {"module": Q38ForCausalLM.__module__,
            "files": {name: hashlib.sha256((root / name).read_bytes()).hexdigest() for name in EXPORT_FILES}}


def hf_model_class():
    """The ``PreTrainedModel`` front end (imports transformers lazily)."""
    return modeling.Qwen3_8MoeForCausalLM


__all__ = ["Qwen3_8MoeTextConfig", "Q38ForCausalLM", "RouterStats", "set_backend", "get_backend",
           "source_info", "hf_model_class", "modeling"]
