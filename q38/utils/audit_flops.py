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
Exits non-zero if a check fails.  (Reference: scripts/audit_flops.py:1-297, which audits the same ledger against Megatron's
formula and an FLA GEMM list.)
"""
import argparse
import json
import sys

import torch


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


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("presets", nargs="*", default=["q38_c1", "q38_c2", "q38_c3", "q38_c4"])
    ap.add_argument("--seq", type=int, default=4096)
    a = ap.parse_args(argv)
    bad = 0
    for name in a.presets:
        report = audit(name, a.seq)
        bad += bool(report["failures"])
        print(json.dumps(report))
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
