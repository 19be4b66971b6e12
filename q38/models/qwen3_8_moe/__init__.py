"""Import path of the reference kept for its users:  ``from q38.models.qwen3_8_moe import Qwen3_8MoeForCausalLM, Qwen3_8MoeTextConfig``.

The model source lives in ``q38/models/hf_export`` (the same two files are copied into every HF export); this package re-exports
the transformers front end, the config class and ``source_info`` from there (reference: q38/models/qwen3_8_moe/__init__.py:1-25).
The model class is resolved on first access because it imports transformers."""
from .. import source_info
from ..hf_export.configuration_qwen3_8_moe import Qwen3_8MoeTextConfig

__all__ = ["Qwen3_8MoeTextConfig", "Qwen3_8MoeForCausalLM", "source_info"]


def __getattr__(name):
    if name == "Qwen3_8MoeForCausalLM":
        from .. import hf_model_class
        return hf_model_class()
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
