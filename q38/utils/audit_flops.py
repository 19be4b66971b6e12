"""Cross-check of the FLOPs ledger (`q38.flops`) against the instantiated model.

  python -m q38.utils.audit_flops [q38_c1 q38_c2 ...] [--seq 4096]

Three independent checks per preset:
  1. parameters: the model built from the preset (meta device, no memory) has exactly `accounting.total_params` parameters,
     and the ledger's parameter terms add up to the same number;
  2. GEMM FLOPs: every weight matrix of the instantiated model is visited and charged 2 x in x out FLOPs per token it is applied
     to (top-k of the routed experts, every layer's projections, the tied output head once); the sum is compared with the
     ledger's GEMM-shaped forward terms (attention scores, delta-rule products, mHC low-rank and n-gram terms are analytic
     and listed separately);
  3. the train/forward ratio and the token budget `compute / train_flops_per_token` recorded in the preset file.
Exits non-zero if a check fails.

  python -m q38.utils.audit_flops --backbone [--megatron-source training.py]

audits the backbone-only convention (`q38.flops._count_backbone`, the one the archived Q35 IsoFLOPs configs were budgeted
with) the way the reference does in scripts/audit_flops.py:1-297: an independent expansion of the formula of Megatron-LM's
`num_floating_point_operations` at the pinned revision b92c3ed (Transformer branch with Gated DeltaNet layers and the attention
output gate) must equal the ledger's `megatron_reference_train_flops_per_token` for every archived config and every width of
the one-parameter family, and the ledger's total must exceed it by exactly the router and shared-expert-gate projections that
formula leaves out.  With `--megatron-source` pointing at that revision's `megatron/training/training.py` (SHA-256 pinned; the
file is not distributed with this repository) the original function is extracted by AST and evaluated too.  The report also
lists the logical 64x64x64 products per chunk and value head of this repository's delta-rule kernels (counted from
`csrc/gdn.cu`), next to the convention's 8 dv^2 per token - a partial GEMM ledger, not a complete operator count.
"""
import argparse
import ast
import hashlib
import json
import re
import sys
from pathlib import Path
from types import SimpleNamespace

import torch

MEGATRON_COMMIT = "b92c3ed70029005fd5769d2cf4c65bc3d061a74b"
MEGATRON_URL = f"https://raw.githubusercontent.com/NVIDIA/Megatron-LM/{MEGATRON_COMMIT}/megatron/training/training.py"
MEGATRON_SHA256 = "370d7844ccc0b36e60bc7f8238b84671ed488c1d2b5c02b5e2f6c32deef8d177"


def matrix_flops_per_token(model, cfg):
    """2 x in x out per token for every 2-D/3-D weight, grouped by role."""
    groups = {}
    topk, experts = cfg.num_experts_per_tok, cfg.num_experts
    for name, p in model.named_parameters():
        if p.dim() < 2 or "emb2" in name or "emb3" in name or name.endswith("embed_tokens.weight"):
            continue
        if ".mhc" in name or name.startswith("model.mhc") or ".conv1d." in name:
            continue
        flops = 2 * p.numel()
        if ".experts." in name:
            flops = flops // experts * topk
        role = ("mtp" if name.startswith("mtp.") else "indexer" if ".indexer" in name or "indexers" in name else
                "experts" if ".experts." in name else "shared_expert" if "shared_expert" in name else "router" if name.endswith("mlp.gate.weight") else
                "ngram_gate" if "ngram" in name else "mixer")
        groups[role] = groups.get(role, 0) + flops
    groups["lm_head"] = 2 * cfg.vocab_size * cfg.hidden_size
    return groups


def audit(name, seq):
    from ..flops import count
    from ..models import Q38ForCausalLM
    from ..presets import load_preset, model_config
    preset = load_preset(name)
    cfg = model_config(preset["model"], 10112, seq, bos_token_id=1, eos_token_id=53, pad_token_id=0)
    with torch.device("meta"):
        model = Q38ForCausalLM(cfg)
    model.tie_embeddings()
    unique = {id(p): p.numel() for p in model.parameters()}
    params = sum(unique.values())
    ledger = count(cfg.to_dict(), seq)
    acct = preset["accounting"]
    failures = []
    if params != acct["total_params"]:
        failures.append(f"parameter count {params} != accounting.total_params {acct['total_params']}")
    if ledger["train_flops_per_token"] != acct["train_flops_per_token"]:
        failures.append(f"ledger train FLOPs {ledger['train_flops_per_token']} != preset {acct['train_flops_per_token']}")
    groups = matrix_flops_per_token(model, cfg)
    gemm = sum(groups.values())
    report = dict(preset=name, seq=seq, total_params=params, train_flops_per_token=ledger["train_flops_per_token"],
                  fwd_flops_per_token=ledger["fwd_flops_per_token"], weight_gemm_flops_per_token=gemm,
                  weight_gemm_share_of_forward=round(gemm / ledger["fwd_flops_per_token"], 4), gemm_groups=groups,
                  ledger_terms=ledger["breakdown"])
    if not 0.5 < report["weight_gemm_share_of_forward"] <= 1.0:
        failures.append(f"weight GEMMs are {report['weight_gemm_share_of_forward']:.2%} of the ledger's forward FLOPs")
    report["failures"] = failures
    return report


# ---- backbone convention against the pinned Megatron formula -------------------------------------------------------------------

def megatron_forward_terms(c, seq):
    """Forward FLOPs per token by the pinned Megatron formula, expanded by hand for this architecture."""
    h, types = c["hidden_size"], c["layer_types"]
    full, linear = types.count("full_attention"), types.count("linear_attention")
    q_width, kv_width = c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    key_width = c["linear_num_key_heads"] * c["linear_key_head_dim"]
    value_width = c["linear_num_value_heads"] * c["linear_value_head_dim"]
    return {
        "attention_projections_with_output_gate": full * 2 * h * (3 * q_width + 2 * kv_width),     # q, gate, out: 3 q_width; k, v: 2 kv_width
        "attention_causal_core": full * 2 * seq * q_width,                                          # QK^T and PV, halved by causality
        "gdn_projections": linear * 2 * h * (2 * key_width + 3 * value_width + 2 * c["linear_num_value_heads"]),
        "gdn_conv": linear * 2 * c["linear_conv_kernel_dim"] * (2 * key_width + value_width),
        "gdn_recurrent_core": linear * 8 * c["linear_num_value_heads"] * c["linear_value_head_dim"] ** 2,
        "routed_and_shared_swiglu": c["num_hidden_layers"] * 6 * h * (c["num_experts_per_tok"] * c["moe_intermediate_size"] + c["shared_expert_intermediate_size"]),
        "logits": 2 * h * c["vocab_size"],
    }


def megatron_arguments(c, seq):
    """The fields `num_floating_point_operations` reads, filled from a model config."""
    return SimpleNamespace(
        seq_length=seq, hidden_size=c["hidden_size"], num_layers=c["num_hidden_layers"], num_attention_heads=c["num_attention_heads"],
        num_query_groups=c["num_key_value_heads"], kv_channels=c["head_dim"], group_query_attention=True, attention_output_gate=True,
        ffn_hidden_size=c["moe_intermediate_size"], moe_ffn_hidden_size=c["moe_intermediate_size"],
        moe_shared_expert_intermediate_size=c["shared_expert_intermediate_size"], num_experts=c["num_experts"],
        moe_router_topk=c["num_experts_per_tok"], moe_layer_freq=1, moe_latent_size=None, mtp_num_layers=None, swiglu=True,
        multi_latent_attention=False, padded_vocab_size=c["vocab_size"], experimental_attention_variant="gated_delta_net",
        linear_attention_freq=[int(t == "linear_attention") for t in c["layer_types"]],
        linear_key_head_dim=c["linear_key_head_dim"], linear_value_head_dim=c["linear_value_head_dim"],
        linear_num_key_heads=c["linear_num_key_heads"], linear_num_value_heads=c["linear_num_value_heads"],
        linear_conv_kernel_dim=c["linear_conv_kernel_dim"])


def load_megatron_function(path, expected_sha256=MEGATRON_SHA256):
    """`num_floating_point_operations` of the pinned revision, compiled alone (no Megatron import, no GPU, no process group)."""
    raw = Path(path).read_bytes()
    digest = hashlib.sha256(raw).hexdigest()
    if digest != expected_sha256:
        raise ValueError(f"{path}: SHA-256 {digest[:16]}... is not the pinned Megatron revision {MEGATRON_COMMIT[:7]} ({MEGATRON_URL})")
    tree = ast.parse(raw)
    node = next((n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "num_floating_point_operations"), None)
    if node is None:
        raise ValueError(f"{path}: no num_floating_point_operations")
    scope = {"is_hybrid_model": lambda args: False,
             "is_linear_attention_variant": lambda variant: variant == "gated_delta_net",
             "is_gated_delta_net_variant": lambda variant: variant == "gated_delta_net"}
    exec(compile(ast.Module(body=[node], type_ignores=[]), str(path), "exec"), scope)
    return scope["num_floating_point_operations"]


def delta_rule_kernel_products(source=None):
    """64x64x64 tensor-core products per (chunk, value head) issued by each delta-rule kernel, counted from the kernel source."""
    text = Path(source or Path(__file__).resolve().parents[2] / "csrc" / "gdn.cu").read_text()
    kernels = re.split(r"__global__ void[^\n]*?\b(gdn_\w+_kernel)\(", text)
    counts = {}
    for name, body in zip(kernels[1::2], kernels[2::2]):
        code = "\n".join(line.split("//")[0] for line in body.splitlines())
        counts[name] = len(re.findall(r"\bmma64h?<", code))
    return counts


def audit_backbone(c, seq, megatron=None):
    from ..flops import _count_backbone
    ledger, terms = _count_backbone(c, seq), megatron_forward_terms(c, seq)
    by_formula = 3 * sum(terms.values())
    left_out = 6 * c["num_hidden_layers"] * c["hidden_size"] * (c["num_experts"] + 1)            # router and shared-expert gate, forward + backward
    failures = []
    if ledger["megatron_reference_train_flops_per_token"] != by_formula:
        failures.append(f"ledger's Megatron component {ledger['megatron_reference_train_flops_per_token']} != formula {by_formula}")
    if ledger["train_flops_per_token"] != by_formula + left_out:
        failures.append(f"ledger total {ledger['train_flops_per_token']} != formula + router/gate {by_formula + left_out}")
    if ledger["breakdown"]["attn_score"] != terms["attention_causal_core"]:
        failures.append("causal attention term differs")
    original = None
    if megatron is not None:
        original = megatron(megatron_arguments(c, seq), 1) / seq
        if original != by_formula:
            failures.append(f"pinned Megatron function gives {original}, hand expansion {by_formula}")
    return dict(shape=f"h{c['hidden_size']}_L{c['num_hidden_layers']}", train_flops_per_token=ledger["train_flops_per_token"],
                megatron_train_flops_per_token=by_formula, megatron_function_evaluated=original,
                router_and_shared_gate_train_flops_per_token=left_out, over_megatron_fraction=ledger["train_flops_per_token"] / by_formula - 1,
                megatron_forward_terms=terms, failures=failures)


def backbone_report(seq=8192, vocab=10112, megatron_source=None):
    from .. import make_isoflops
    from ..presets import ROOT, model_config
    megatron = load_megatron_function(megatron_source) if megatron_source else None
    archived = []
    for path in sorted((ROOT / "configs/q35_isoflops").glob("*/*/config.json")):
        p = json.loads(path.read_text())
        row = audit_backbone(model_config(p["model"], vocab, p["train"]["seq"]).to_dict(), p["train"]["seq"], megatron)
        if p["accounting"]["train_flops_per_token"] != row["train_flops_per_token"]:
            row["failures"].append(f"stale accounting in {path}")
        tokens = p["accounting"]["train_tokens"]
        row.update(config=str(path.relative_to(ROOT)), compute=p["compute"], train_tokens=tokens,
                   budget_fraction=tokens * row["train_flops_per_token"] / p["compute"] - 1,
                   megatron_reaccounted_budget_fraction=tokens * row["megatron_train_flops_per_token"] / p["compute"] - 1)
        archived.append(row)
    family = [audit_backbone(model_config(make_isoflops.shape_for(hidden), vocab, seq).to_dict(), seq, megatron) for hidden in make_isoflops.WIDTHS]
    products = delta_rule_kernel_products()
    per_token = {name: n * 2 * 64 * 64 * 64 / 64 for name, n in products.items()}
    return dict(reference=dict(commit=MEGATRON_COMMIT, url=MEGATRON_URL, sha256=MEGATRON_SHA256, original_function_evaluated=megatron is not None),
                scope=dict(seq=seq, vocab=vocab, physical_kernel_flops=False),
                archived_configs=archived, canonical_family=family,
                delta_rule_kernels=dict(products_64x64x64_per_chunk_and_value_head=products, gemm_flops_per_token_and_value_head=per_token,
                                        training_total_per_token_and_value_head=sum(per_token.values()),
                                        convention_training_per_token_and_value_head=3 * 8 * 64 * 64,
                                        note="partial ledger: tensor-core products only (the triangular solve, gating, norms and "
                                             "reductions are vector work); the convention charges the recurrent form"),
                failures=[f for row in archived + family for f in row["failures"]])


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("presets", nargs="*", default=["q38_c1", "q38_c2", "q38_c3", "q38_c4"])
    ap.add_argument("--seq", type=int, default=None)
    ap.add_argument("--backbone", action="store_true", help="audit the backbone convention against the pinned Megatron formula instead")
    ap.add_argument("--megatron-source", default="", help="megatron/training/training.py of the pinned revision (SHA-256 checked)")
    ap.add_argument("--output", default="", help="write the backbone report to this JSON file")
    a = ap.parse_args(argv)
    if a.backbone:
        report = backbone_report(a.seq or 8192, megatron_source=a.megatron_source or None)
        if a.output:
            Path(a.output).write_text(json.dumps(report, indent=2) + "\n")
        for row in report["canonical_family"]:
            print(f"{row['shape']:12} ledger={row['train_flops_per_token']:13,d} megatron={row['megatron_train_flops_per_token']:13,d} "
                  f"router/gate={row['over_megatron_fraction']:+.3%}")
        print(f"checked {len(report['archived_configs'])} archived configs and {len(report['canonical_family'])} widths; "
              f"delta-rule kernel products {report['delta_rule_kernels']['products_64x64x64_per_chunk_and_value_head']}; failures: {len(report['failures'])}")
        return 1 if report["failures"] else 0
    a.seq = a.seq or 4096
    bad = 0
    for name in a.presets:
        report = audit(name, a.seq)
        bad += bool(report["failures"])
        print(json.dumps(report))
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
