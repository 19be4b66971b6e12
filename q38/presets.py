"""Preset files (``configs/<name>.json``) and construction of the model config from shape fields.

A preset has the sections ``compute`` (FLOP budget), ``model`` (shape), ``train`` (trainer defaults)
and ``accounting``.  Shape fields use the short names of the command line (``hidden``, ``layers`` ...);
`model_config` expands them into the HF-style config.  Scaling rules shared by all presets: every
fourth layer is QSA (the others Gated DeltaNet), 64 experts top-5 plus a shared expert, head_dim 64
with an output gate, partial rotary 0.25 at theta 1e7, tied embeddings.
(Reference behaviour: q38/presets.py:21-98.)
"""
import json
import os
from pathlib import Path

from .flops import count
from .models import Qwen3_8MoeTextConfig

ROOT = Path(__file__).resolve().parents[1]
PRESET_DIR = ROOT / "configs"
# Run directories of the c1..c4 presets; override with Q38_CKPT_ROOT on machines without that mount.
CKPT_ROOT = Path(os.environ.get("Q38_CKPT_ROOT", "/home/shared/ckpt"))

MODEL_DEFAULTS = dict(
    layers=5, hidden=96, heads=2, kv_heads=1, head_dim=64, lin_k_heads=1, lin_v_heads=2, lin_head_dim=64,
    experts=64, topk=5, moe_ffn=24, shared_ffn=24, layer_types="", aux_coef=0.001, rope_theta=1e7,
    partial_rotary=0.25, experts_impl="eager", n_branch=4, mhc_iters=20, qsa_blocks=8, indexer_heads=4,
    indexer_head_dim=64, ngram_rows=-1, mtp=1)


def preset_names():
    return sorted(path.stem for path in PRESET_DIR.glob("*.json"))


def load_preset(name):
    path = PRESET_DIR / f"{name}.json"
    if not path.is_file():
        raise ValueError(f"Unknown preset {name!r}; available: {', '.join(preset_names())}")
    return json.loads(path.read_text())


def load_training_config(target):
    """Resolve a JSON file (or a directory holding ``config.json``) and check its sections."""
    path = Path(target).expanduser()
    path = path if path.is_absolute() else ROOT / path
    path = (path / "config.json" if path.is_dir() else path).resolve()
    config = json.loads(path.read_text())
    if not isinstance(config, dict) or any(key not in config for key in ("compute", "model", "train")):
        raise ValueError(f"Training config requires compute/model/train sections: {path}")
    if not isinstance(config["model"], dict) or not isinstance(config["train"], dict):
        raise ValueError("model and train must be JSON objects")
    return path, config


def default_layer_types(layers):
    return ["full_attention" if i % 4 == 3 else "linear_attention" for i in range(layers)]


def auto_ngram_rows(config_dict, hidden, seq):
    """Rows per hash table when ``ngram_rows == -1``: 20.5 % of the non-vocabulary parameters of the
    model without tables and MTP, per table row of width ``hidden``, rounded to a multiple of 1024."""
    base = count({**config_dict, "ngram_rows": 0, "mtp": False}, seq)["total_nonvocab_params"]
    return max(1024, round(0.205 * base / hidden / 1024) * 1024)


def model_config(shape, vocab_size, seq, bos_token_id=None, eos_token_id=None, pad_token_id=None):
    s = {**MODEL_DEFAULTS, **shape}
    kinds = s["layer_types"].split(",") if s["layer_types"] else default_layer_types(s["layers"])
    rope = {"rope_type": "default", "rope_theta": s["rope_theta"], "partial_rotary_factor": s["partial_rotary"]}
    cfg = Qwen3_8MoeTextConfig(
        vocab_size=vocab_size, hidden_size=s["hidden"], num_hidden_layers=s["layers"],
        num_attention_heads=s["heads"], num_key_value_heads=s["kv_heads"], head_dim=s["head_dim"],
        linear_num_key_heads=s["lin_k_heads"], linear_num_value_heads=s["lin_v_heads"],
        linear_key_head_dim=s["lin_head_dim"], linear_value_head_dim=s["lin_head_dim"], linear_conv_kernel_dim=4,
        num_experts=s["experts"], num_experts_per_tok=s["topk"], moe_intermediate_size=s["moe_ffn"],
        shared_expert_intermediate_size=s["shared_ffn"], router_aux_loss_coef=s["aux_coef"],
        output_router_logits=False, layer_types=kinds, max_position_embeddings=seq, rms_norm_eps=1e-6,
        rope_parameters=rope, partial_rotary_factor=s["partial_rotary"], tie_word_embeddings=True,
        attention_bias=False, initializer_range=0.02,
        bos_token_id=eos_token_id if bos_token_id is None else bos_token_id, eos_token_id=eos_token_id,
        pad_token_id=eos_token_id if pad_token_id is None else pad_token_id)
    for key in ("n_branch", "mhc_iters", "qsa_blocks", "indexer_heads", "indexer_head_dim"):
        setattr(cfg, key, s[key])
    cfg.mtp = bool(s["mtp"])
    cfg.ngram_rows = auto_ngram_rows(cfg.to_dict(), s["hidden"], seq) if s["ngram_rows"] == -1 else s["ngram_rows"]
    if cfg.indexer_head_dim != cfg.head_dim or cfg.qsa_blocks < 1 or cfg.ngram_rows < 0:
        raise ValueError("Invalid Q38 indexer head dimension, sparse budget or N-gram rows")
    cfg.use_cache = False
    return cfg


def budget_tokens(train_flops_per_token, compute, batch_tokens):
    """Tokens of the largest whole number of global batches that fits into `compute` FLOPs."""
    return int(compute) // (train_flops_per_token * batch_tokens) * batch_tokens


def preset_budget(name, vocab_size, seq=None, batch_tokens=None):
    """Token budget and ledger of a preset for a given vocabulary / sequence length."""
    preset = load_preset(name)
    train = preset["train"]
    seq = train.get("seq", 4096) if seq is None else seq
    batch_tokens = train.get("batch_tokens", 524288) if batch_tokens is None else batch_tokens
    ledger = count(model_config(preset["model"], vocab_size, seq).to_dict(), seq)
    reserve = preset.get("accounting", {}).get("compute_reserve_fraction", 0.0)
    usable = int(preset["compute"] * (1 - reserve))
    return budget_tokens(ledger["train_flops_per_token"], usable, batch_tokens), ledger
