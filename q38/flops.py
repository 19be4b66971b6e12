"""Parameter and FLOP ledger for the Q38 model (`python -m q38.flops q38_c2 --seq 4096`).

The ledger reproduces the accounting of the reference (q38/flops.py:14-105): the
backbone terms follow the pinned Megatron convention for Gated DeltaNet / MoE layers, and
the Q38 additions (sparse QSA average, indexer, mHC, n-gram gate, training-only MTP, the
dense distillation target) are layered on top.  MFU numbers printed by the benchmark are
defined against ``count(...)["train_flops_per_token"]``.

The implementation is a term ledger: every entry is produced by one small function of a
``Shape`` record, so the GPU roofline code can ask for a single term (for instance the
expert GEMM FLOPs of one layer) without re-deriving it.
"""
from __future__ import annotations

import argparse
import json
from dataclasses import dataclass

MEGATRON_COMMIT = "b92c3ed70029005fd5769d2cf4c65bc3d061a74b"
BACKBONE_METHOD = "megatron_b92c3ed_plus_router_shared_gate_v1"
ACCOUNTING_METHOD = BACKBONE_METHOD            # the name the reference exports for the backbone convention (q38/flops.py:11)
Q38_METHOD = "q38_sparse_mhc_ngram_mtp_v2"
QSA_BLOCK = 64


@dataclass(frozen=True)
class Shape:
    """The subset of the model config that the ledger needs."""
    layers: int
    hidden: int
    vocab: int
    experts: int
    topk: int
    expert_ffn: int
    shared_ffn: int
    heads: int
    kv_heads: int
    head_dim: int
    lin_k_heads: int
    lin_v_heads: int
    lin_k_dim: int
    lin_v_dim: int
    conv_kernel: int
    layer_types: tuple

    @classmethod
    def from_config(cls, cfg):
        cfg = cfg.get("text_config", cfg)
        n = cfg["num_hidden_layers"]
        return cls(layers=n, hidden=cfg["hidden_size"], vocab=cfg["vocab_size"],
                   experts=cfg["num_experts"], topk=cfg["num_experts_per_tok"],
                   expert_ffn=cfg["moe_intermediate_size"], shared_ffn=cfg["shared_expert_intermediate_size"],
                   heads=cfg["num_attention_heads"], kv_heads=cfg["num_key_value_heads"], head_dim=cfg["head_dim"],
                   lin_k_heads=cfg["linear_num_key_heads"], lin_v_heads=cfg["linear_num_value_heads"],
                   lin_k_dim=cfg["linear_key_head_dim"], lin_v_dim=cfg["linear_value_head_dim"],
                   conv_kernel=cfg["linear_conv_kernel_dim"], layer_types=tuple(cfg["layer_types"][:n]))

    @property
    def n_linear(self):
        return sum(t == "linear_attention" for t in self.layer_types)

    @property
    def n_full(self):
        return sum(t == "full_attention" for t in self.layer_types)

    @property
    def conv_dim(self):
        return 2 * self.lin_k_heads * self.lin_k_dim + self.lin_v_heads * self.lin_v_dim

    @property
    def value_dim(self):
        return self.lin_v_heads * self.lin_v_dim


# ---- parameter terms ---------------------------------------------------------------

def _moe_params(s: Shape, experts_counted: int) -> int:
    router = s.experts * s.hidden
    shared = 3 * s.hidden * s.shared_ffn + s.hidden          # shared expert + its scalar gate
    return router + shared + experts_counted * 3 * s.hidden * s.expert_ffn


def _gdn_params(s: Shape) -> int:
    h, nv = s.hidden, s.lin_v_heads
    projections = h * s.conv_dim + h * s.value_dim + 2 * h * nv      # qkv, z, b, a
    conv = s.conv_dim * s.conv_kernel
    small = 2 * nv + s.lin_v_dim                                        # dt_bias, A_log, gated-norm weight
    return projections + conv + small + s.value_dim * h                # + out_proj


def _attention_params(s: Shape) -> int:
    h, hd = s.hidden, s.head_dim
    return h * 2 * s.heads * hd + 2 * h * s.kv_heads * hd + s.heads * hd * h + 2 * hd


# ---- forward FLOP terms (per token) -------------------------------------------------

def _backbone_terms(s: Shape, seq: int) -> dict:
    h = s.hidden
    return dict(
        full_projections=s.n_full * 2 * h * (3 * s.heads * s.head_dim + 2 * s.kv_heads * s.head_dim),
        gdn_projections=s.n_linear * 2 * h * (2 * s.lin_k_heads * s.lin_k_dim + 3 * s.value_dim + 2 * s.lin_v_heads),
        gdn_conv=s.n_linear * 2 * s.conv_kernel * s.conv_dim,
        # The pinned convention charges dv^2 per value head even when dk != dv.
        gdn_core=s.n_linear * 8 * s.lin_v_heads * s.lin_v_dim ** 2,
        expert_gemm=s.layers * 6 * h * (s.topk * s.expert_ffn + s.shared_ffn),
        router=s.layers * 2 * h * s.experts,
        shared_gate=s.layers * 2 * h,
        attn_score=s.n_full * 2 * seq * s.heads * s.head_dim,
        logits=2 * h * s.vocab,
    )


def _count_backbone(c, seq):
    """Backbone-only ledger (GDN + gated attention + MoE + logits), also used for archived Q35 configs."""
    s = Shape.from_config(c)
    cfg = c.get("text_config", c)
    if seq <= 0 or len(s.layer_types) != s.layers or set(s.layer_types) - {"linear_attention", "full_attention"}:
        raise ValueError("Positive sequence length and one supported layer type per layer are required")
    if cfg.get("attention_bias", False):
        raise ValueError("This accounting supports the bias-free Qwen attention projections")
    mixers = s.n_linear * _gdn_params(s) + s.n_full * _attention_params(s)
    norms = s.layers * 2 * s.hidden + s.hidden
    active = mixers + norms + s.layers * _moe_params(s, s.topk)
    total = mixers + norms + s.layers * _moe_params(s, s.experts)
    terms = _backbone_terms(s, seq)
    fwd = sum(terms.values())
    extra = terms["router"] + terms["shared_gate"]
    return dict(layers=s.layers, hidden=s.hidden, layer_types=list(s.layer_types), vocab=s.vocab, seq=seq,
                experts=s.experts, topk=s.topk, expert_ffn=s.expert_ffn, shared_ffn=s.shared_ffn,
                attn_heads=s.heads, kv_heads=s.kv_heads, head_dim=s.head_dim,
                lin_k_heads=s.lin_k_heads, lin_v_heads=s.lin_v_heads,
                active_nonvocab_params=active, total_nonvocab_params=total, nonvocab_params=active,
                embed_params=s.hidden * s.vocab,
                accounting_method=BACKBONE_METHOD, megatron_commit=MEGATRON_COMMIT,
                fwd_flops_per_token=fwd, train_flops_per_token=3 * fwd,
                megatron_reference_train_flops_per_token=3 * (fwd - extra),
                extra_router_shared_gate_train_flops_per_token=3 * extra,
                breakdown=terms)


def mhc_rank(hidden: int) -> int:
    return max(1, round(hidden / 8))


def sparse_keys_per_query(seq: int, budget: int) -> float:
    """Average number of keys a query attends to under the QSA block budget.

    Query block i sees min(i+1, budget) blocks; all but its own are full 64-key blocks and
    the causal own block contributes 32.5 keys on average.
    """
    blocks = (seq + QSA_BLOCK - 1) // QSA_BLOCK
    return sum(QSA_BLOCK * (min(i + 1, budget) - 1) + 32.5 for i in range(blocks)) / blocks


def count(c, seq):
    """Full Q38 ledger.  Dense warm-up and optimizer work are not counted (as in the reference)."""
    c = c.get("text_config", c)
    out = _count_backbone(c, seq)
    s = Shape.from_config(c)
    h, L, nf = s.hidden, s.layers, s.n_full
    n = c.get("n_branch", 4)
    r = mhc_rank(h)
    ni, di = c.get("indexer_heads", 4), c.get("indexer_head_dim", 64)
    rows, budget = c.get("ngram_rows", 0), c.get("qsa_blocks", 8)
    if rows < 0 or budget < 1 or seq < 1:
        raise ValueError("Invalid Q38 N-gram rows, sparse block budget or sequence length")
    coeffs = 2 * n + n * n                                   # pre, post and the n x n residual mix

    terms = dict(out["breakdown"])
    terms["attn_score"] = round(nf * 4 * s.heads * s.head_dim * sparse_keys_per_query(seq, budget))
    indexer_params = nf * h * (ni * di + di + ni)
    mhc_params = 2 * L * (n * h * r + r * coeffs + coeffs + 3)
    gate_params, table_params = (h * h + 2 * h, 2 * rows * h) if rows else (0, 0)
    terms.update(indexer_projections=2 * indexer_params,
                 indexer_score=nf * 2 * seq * ni * di,
                 mhc_projections=2 * 2 * L * (n * h * r + r * coeffs),
                 mhc_mix=2 * L * 2 * h * coeffs,
                 ngram_gate=2 * h * h if rows else 0)
    mtp_params = mtp_active = 0
    if c.get("mtp", True):
        one = _count_backbone(dict(c, num_hidden_layers=1, layer_types=["linear_attention"]), seq)
        glue = 2 * h * h + 2 * h                              # proj[2h->h] and the two input norms
        mtp_params = one["total_nonvocab_params"] + glue
        mtp_active = one["active_nonvocab_params"] + glue
        terms["mtp"] = one["fwd_flops_per_token"] + 4 * h * h
    distill = nf * 2 * seq * s.heads * s.head_dim             # dense block-mass target, forward only
    active = out["active_nonvocab_params"] + indexer_params + mhc_params + gate_params + (2 * h if rows else 0)
    total = out["total_nonvocab_params"] + indexer_params + mhc_params + gate_params + table_params + mtp_params
    fwd = sum(terms.values())
    # The indexer input is detached, so its projections cost forward + weight gradient only.
    train = 3 * fwd - terms["indexer_projections"] + distill
    out.update(accounting_method=Q38_METHOD, breakdown=terms,
               active_nonvocab_params=active, nonvocab_params=active, total_nonvocab_params=total,
               total_params_all=total + out["embed_params"], ngram_params=table_params, ngram_rows=rows,
               indexer_params=indexer_params, mhc_params=mhc_params, mtp_params=mtp_params,
               mtp_active_params=mtp_active, distill_target_flops=distill,
               fwd_flops_per_token=fwd, main_fwd_flops_per_token=fwd - terms.get("mtp", 0),
               train_flops_per_token=train)
    return out


def validate_resume_accounting(previous, current):
    """A run directory must not mix FLOP conventions across resumes."""
    same_flops = previous.get("flops_per_token") == current["train_flops_per_token"]
    same_method = previous.get("flops_accounting", current["accounting_method"]) == current["accounting_method"]
    if not (same_flops and same_method):
        raise ValueError("Unsafe resume: FLOPs accounting changed; use a new run_dir")


def main(argv=None):
    from .data import DEFAULT_TOKENIZER
    from .presets import preset_budget, preset_names
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("target", help="preset name or a config.json holding a model config")
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--tokens", type=float, default=0)
    ap.add_argument("--batch_tokens", type=int, default=None)
    ap.add_argument("--tokenizer", default=str(DEFAULT_TOKENIZER))
    a = ap.parse_args(argv)
    if a.target in preset_names():
        from tokenizers import Tokenizer
        vocab = Tokenizer.from_file(f"{a.tokenizer}/tokenizer.json").get_vocab_size()
        tokens, res = preset_budget(a.target, vocab, a.seq, a.batch_tokens)
        res["budget_tokens"] = tokens
        a.tokens = a.tokens or tokens
    else:
        with open(a.target) as f:
            res = count(json.load(f), a.seq)
    if a.tokens:
        res["train_tokens"] = a.tokens
        res["train_flops"] = res["train_flops_per_token"] * a.tokens
    print(json.dumps(res, indent=1))
    return res


if __name__ == "__main__":
    main()
