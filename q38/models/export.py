"""HF export / import of a trained model.

`save_hf` writes a directory that `AutoModelForCausalLM.from_pretrained(dir, trust_remote_code=True)`
loads without this repository: safetensors weights (``mtp.*`` and the n-gram tables included), a
``config.json`` whose ``auto_map`` points at the two model source files, the files themselves and,
optionally, the tokenizer.  State-dict keys are those of the reference export (q38/train.py:600), so a
directory written by either implementation carries the same tensors under the same names.
"""
import json
import shutil
from pathlib import Path

import torch

from . import EXPORT_FILES, hf_model_class

AUTO_MAP = {"AutoConfig": "configuration_qwen3_8_moe.Qwen3_8MoeTextConfig",
            "AutoModelForCausalLM": "modeling_qwen3_8_moe.Qwen3_8MoeForCausalLM"}


def to_hf(model, dtype=None):
    """Wrap the weights of a `Q38ForCausalLM` in the `PreTrainedModel` front end (weights are copied)."""
    cls = hf_model_class()
    hf = cls(model.config)
    state = {k: v.detach().to("cpu") for k, v in model.state_dict().items()}
    hf.load_state_dict(state)
    hf.tie_weights()
    if dtype is not None:
        hf = hf.to(dtype)
    return hf.eval()


def save_hf(model, out_dir, tokenizer=None, dtype=torch.bfloat16):
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    hf = to_hf(model, dtype)
    hf.config.auto_map = dict(AUTO_MAP)
    hf.config.architectures = ["Qwen3_8MoeForCausalLM"]
    hf.save_pretrained(out)
    source = Path(__file__).resolve().parent / "hf_export"
    for name in EXPORT_FILES:
        shutil.copyfile(source / name, out / name)
    config_path = out / "config.json"
    config = json.loads(config_path.read_text())
    config["auto_map"] = dict(AUTO_MAP)
    config_path.write_text(json.dumps(config, indent=2) + "\n")
    if tokenizer is not None:
        tokenizer.save_pretrained(out)
    return out


def load_hf(path, dtype=torch.bfloat16, device="cpu"):
    """Load an export into the dependency-free `Q38ForCausalLM` (strict on everything except ``mtp.*``)."""
    from safetensors.torch import load_file
    from . import Q38ForCausalLM, Qwen3_8MoeTextConfig
    path = Path(path)
    config = Qwen3_8MoeTextConfig.from_pretrained(path, local_files_only=True)
    model = Q38ForCausalLM(config, init=False)
    state = {}
    for shard in sorted(path.glob("*.safetensors")):
        state.update(load_file(shard))
    if "lm_head.weight" not in state and "model.embed_tokens.weight" in state:
        state["lm_head.weight"] = state["model.embed_tokens.weight"]
    missing, unexpected = model.load_state_dict(state, strict=False)
    missing = [k for k in missing if not k.startswith("mtp.")]
    if missing or unexpected:
        raise RuntimeError(f"Checkpoint did not fully initialize the language model: missing={missing} unexpected={unexpected}")
    model.tie_embeddings()
    return model.to(device=device, dtype=dtype).eval()
