"""Configuration of the Q38 sparse MoE text model (HF `model_type = "qwen38_moe_sparse"`).

Field names and defaults follow the reference config
(q38/models/qwen3_8_moe/configuration_qwen3_8_moe.py:25-112) so that a `config.json` written by
either implementation loads in the other.  This file is self-contained: it is copied next to
the weights by the HF export and loaded there with `trust_remote_code=True`.
"""
from huggingface_hub.dataclasses import strict
from transformers.configuration_utils import PreTrainedConfig


@strict
class Qwen3_8MoeTextConfig(PreTrainedConfig):
    """Gated DeltaNet / gated attention / MoE backbone plus the Q38 additions
    (mHC branches, QSA block budget, indexer shape, n-gram rows, MTP switch)."""

    model_type = "qwen38_moe_sparse"
    base_config_key = "text_config"
    keys_to_ignore_at_inference = ["past_key_values"]
    ignore_keys_at_rope_validation = {"mrope_section", "mrope_interleaved"}

    # backbone
    vocab_size: int = 248320
    hidden_size: int = 2048
    num_hidden_layers: int = 40
    num_attention_heads: int = 16
    num_key_value_heads: int = 2
    head_dim: int = 256
    hidden_act: str = "silu"
    max_position_embeddings: int = 32768
    initializer_range: float = 0.02
    rms_norm_eps: float = 1e-6
    use_cache: bool = False
    tie_word_embeddings: bool = True
    rope_parameters: dict | None = None
    attention_bias: bool = False
    attention_dropout: float | int = 0.0
    # Gated DeltaNet
    linear_conv_kernel_dim: int = 4
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 32
    # MoE
    moe_intermediate_size: int = 512
    shared_expert_intermediate_size: int = 512
    num_experts_per_tok: int = 5
    num_experts: int = 256
    output_router_logits: bool = False
    router_aux_loss_coef: float = 0.001
    # Q38 additions
    n_branch: int = 4
    mhc_iters: int = 20
    qsa_blocks: int = 8
    indexer_heads: int = 4
    indexer_head_dim: int = 64
    ngram_rows: int = 0
    mtp: bool = True
    layer_types: list[str] | None = None
    pad_token_id: int | None = None
    bos_token_id: int | None = None
    eos_token_id: int | list[int] | None = None

    def __post_init__(self, **kwargs):
        kwargs.setdefault("partial_rotary_factor", 0.25)
        if self.layer_types is None:
            every = kwargs.pop("full_attention_interval", 4)
            self.layer_types = ["full_attention" if (i + 1) % every == 0 else "linear_attention"
                                for i in range(self.num_hidden_layers)]
        super().__post_init__(**kwargs)


__all__ = ["Qwen3_8MoeTextConfig"]
