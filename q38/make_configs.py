"""Generate / verify the ``configs/q38_c{1..4}.json`` presets:  python -m q38.make_configs [--check]

One architecture rule maps a hidden width on the 64-grid to every other dimension; the compute budget
fixes the global batch (DeepSeek-style power law rounded to a power-of-two number of sequences), the
learning rate ``0.3118 * C**-0.125`` and, with 0.5 % of the budget held back, the whole-batch token count.
The width per budget comes from the Q35 IsoFLOPs sweep (``configs/q35_isoflops/results.json``, 19 completed
runs): per sweep budget a parabola of bits-per-byte over log10(active parameters) gives the optimal model and
data size, two power laws in the compute extrapolate them to the four Q38 budgets, and of all widths on the
64-grid the one whose (active parameters, tokens) lies nearest the prediction in log distance is taken -
448 / 576 / 768 / 1024 (the reference does the same in scripts/make_q38_configs.py:46-110; the fitted slopes
0.777 and 0.436 and the chosen widths are checked in tests/test_accounting.py).  The Q35 prior transfers to a
different architecture and, beyond 3e17, extrapolates: it selects a starting point, it predicts no Q38 loss.
"""
import argparse
import json
import math
from functools import lru_cache

import numpy as np

from .flops import count, sparse_keys_per_query
from .presets import CKPT_ROOT, MODEL_DEFAULTS, PRESET_DIR, ROOT, budget_tokens, model_config

SEQ, VOCAB, RESERVE = 4096, 10112, 0.005
BUDGETS = {"c1": 3 * 10 ** 17, "c2": 10 ** 18, "c3": 3 * 10 ** 18, "c4": 10 ** 19}
SWEEP_RESULTS = ROOT / "configs" / "q35_isoflops" / "results.json"
POOL = "/home/shared/qwen35_moe_sparse/cache/isoflops-gzy10k-16b-v1"
# Frozen validation partitions of the shared pool: (offset, targets) of the dev and the final curve split.
DEV_SPLIT, FINAL_SPLIT = (0, 2002535), (2002536, 16001875)


def shape_for(hidden):
    key_heads = max(2, round(0.8 * hidden / 64))
    width = max(8, round(hidden / 4 / 8) * 8)
    return {**MODEL_DEFAULTS, "hidden": hidden, "layers": max(4, round(hidden / 51.2)),
            "heads": 2 * max(1, round(1.2 * hidden / 64)), "kv_heads": 2,
            "lin_k_heads": key_heads, "lin_v_heads": 3 * key_heads, "experts": 64, "topk": 5,
            "moe_ffn": width, "shared_ffn": width, "experts_impl": "grouped_mm", "ngram_rows": -1}


def batch_for(compute):
    return SEQ * max(8, 2 ** round(math.log2(0.2920 * compute ** 0.3271 / SEQ)))


def fit_sweep(rows):
    """Scaling prior from completed IsoFLOPs runs.

    ``rows``: dicts with budget, compute, active_params, train_tokens, bpb.  Per budget (three or more runs) the loss is fitted
    as a parabola in x = log10(active parameters); its vertex is the optimal size, and the tokens at that size are read from a
    polynomial of log10(tokens) over x through the same runs.  Returns (per-budget fits, line of log10 N_opt over log10 C,
    line of log10 D_opt over log10 C, leave-one-budget-out slopes with the size each predicts at 1e19 FLOPs).
    """
    fits = []
    for budget in sorted({r["budget"] for r in rows}, key=float):
        runs = sorted((r for r in rows if r["budget"] == budget), key=lambda r: r["active_params"])
        if len(runs) < 3:
            raise ValueError(f"budget {budget}: a parabola needs three completed runs, found {len(runs)}")
        x, y = np.log10([r["active_params"] for r in runs]), np.array([r["bpb"] for r in runs])
        curve = np.polyfit(x, y, 2)
        if curve[0] <= 0:
            raise ValueError(f"budget {budget}: the fitted parabola has no minimum")
        x_opt = -curve[1] / (2 * curve[0])
        tokens_curve = np.polyfit(x, np.log10([r["train_tokens"] for r in runs]), min(2, len(runs) - 1))
        fits.append(dict(budget=budget, compute=float(np.mean([r["compute"] for r in runs])), parabola=curve.tolist(),
                         active_opt=float(10 ** x_opt), tokens_opt=float(10 ** np.polyval(tokens_curve, x_opt)),
                         bpb_opt=float(np.polyval(curve, x_opt)), inside_grid=bool(x.min() <= x_opt <= x.max()),
                         residual_rmse=float(np.sqrt(np.mean((np.polyval(curve, x) - y) ** 2))),
                         measured_best=min(runs, key=lambda r: r["bpb"])["model"]))
    log_c = np.log10([f["compute"] for f in fits])
    log_n, log_d = np.log10([f["active_opt"] for f in fits]), np.log10([f["tokens_opt"] for f in fits])
    size_law, data_law = np.polyfit(log_c, log_n, 1), np.polyfit(log_c, log_d, 1)
    left_out = []
    for i, f in enumerate(fits):
        keep = [j for j in range(len(fits)) if j != i]
        law = np.polyfit(log_c[keep], log_n[keep], 1)
        left_out.append(dict(omitted_budget=f["budget"], active_exponent=float(law[0]), c4_active_prediction=float(10 ** np.polyval(law, 19))))
    return fits, size_law, data_law, left_out


@lru_cache(maxsize=None)
def sweep_prior():
    return fit_sweep(json.loads(SWEEP_RESULTS.read_text())["runs"])


def ranked_widths(compute, batch):
    """Every admissible width on the 64-grid with its ledger, nearest the prior's (N_opt, D_opt) for `compute` first."""
    _, size_law, data_law, _ = sweep_prior()
    n_target, d_target = 10 ** np.polyval(size_law, math.log10(compute)), 10 ** np.polyval(data_law, math.log10(compute))
    ranked = []
    for hidden in range(128, 1601, 64):
        shape = shape_for(hidden)
        cfg = model_config(shape, VOCAB, SEQ)
        shape["ngram_rows"] = cfg.ngram_rows
        ledger = count(cfg.to_dict(), SEQ)
        tokens = budget_tokens(ledger["train_flops_per_token"], int(compute * (1 - RESERVE)), batch)
        if tokens == 0 or ledger["active_nonvocab_params"] / ledger["total_nonvocab_params"] <= 0.10:
            continue
        distance = math.log(ledger["active_nonvocab_params"] / n_target) ** 2 + math.log(tokens / d_target) ** 2
        ranked.append(dict(distance=distance, hidden=hidden, shape=shape, ledger=ledger, tokens=tokens))
    ranked.sort(key=lambda r: r["distance"])
    return ranked, float(n_target), float(d_target)


def omitted_bounds(shape, ledger, steps, warmup):
    """Upper bounds on work the ledger leaves out: dense warm-up attention and mHC pointwise/Sinkhorn math."""
    h, L, n = shape["hidden"], shape["layers"], shape["n_branch"]
    avg = sparse_keys_per_query(SEQ, shape["qsa_blocks"])
    dense = 3 * (L // 4) * shape["heads"] * shape["head_dim"] * (2 * SEQ - 4 * avg) * warmup / steps
    mhc = 3 * 2 * L * (10 * n * n * shape["mhc_iters"] + 20 * n * h + 200 * n * n)
    per_token = ledger["train_flops_per_token"]
    return dict(dense_warmup_extra_train_flops_per_token=dense, dense_warmup_fraction=dense / per_token,
                mhc_unlisted_pointwise_train_flops_per_token_bound=mhc,
                mhc_unlisted_pointwise_fraction_bound=mhc / per_token,
                combined_fraction_bound=(dense + mhc) / per_token,
                excludes="Does not bound every other unlisted non-GEMM operation; not organizer-reviewed.")


def build(name):
    compute = BUDGETS[name]
    batch = batch_for(compute)
    best = ranked_widths(compute, batch)[0][0]
    shape, ledger, tokens = best["shape"], best["ledger"], best["tokens"]
    steps = tokens // batch
    warmup = min(steps, max(10, round(steps * 0.01)))
    train = dict(run_dir=str(CKPT_ROOT / name), data=f"{POOL}/train.bin", val_data=f"{POOL}/valid.bin",
                 tokenizer=f"{POOL}/tokenizer", seq=SEQ, tokens=tokens, batch_tokens=batch, micro_bs=4,
                 auto_micro_bs=1, probe_mem_frac=0.92, lr=round(0.3118 * compute ** -0.125, 6), min_lr_ratio=0.1,
                 warmup=warmup, warmup_ratio=0.01, warmup_min=10, wd=0.1, clip=1.0, seed=0, data_seed=0,
                 data_sampling="shuffled_blocks", require_ready_pool=1, eval_sampling="sequential",
                 eval_offset=DEV_SPLIT[0], eval_tokens=DEV_SPLIT[1],
                 final_eval_offset=FINAL_SPLIT[0], final_eval_tokens=FINAL_SPLIT[1],
                 log_every=10, eval_every=500, ckpt_every=500, resume=1, max_steps=0, tensorboard=1,
                 mtp_coef=0.3, kl_coef=0.05, muon=1, dense_warmup=1)
    if name == "c4":
        # The reference preset: per-layer activation checkpointing and micro batch 2 (sized for 40 GB GPUs).
        # On 180 GB parts run it with --grad_ckpt 0 --micro_bs 4.
        train.update(grad_ckpt=1, micro_bs=2)
    accounting = dict(
        accounting_method=ledger["accounting_method"], vocab_size=VOCAB, compute_reserve_fraction=RESERVE,
        total_params=ledger["total_params_all"], total_nonvocab_params=ledger["total_nonvocab_params"],
        active_nonvocab_params=ledger["active_nonvocab_params"],
        active_fraction=ledger["active_nonvocab_params"] / ledger["total_nonvocab_params"],
        ngram_params=ledger["ngram_params"], mtp_params=ledger["mtp_params"],
        train_flops_per_token=ledger["train_flops_per_token"], train_tokens=tokens, steps=steps,
        actual_train_flops=tokens * ledger["train_flops_per_token"],
        compute_shortfall_fraction=1 - tokens * ledger["train_flops_per_token"] / compute,
        tokens_per_active_param=tokens / ledger["active_nonvocab_params"], global_batch_sequences=batch // SEQ,
        counted_compute_target=int(compute * (1 - RESERVE)),
        omitted_operation_bounds=omitted_bounds(shape, ledger, steps, warmup))
    return dict(schema_version=2, architecture="q38", compute=compute, model=shape, train=train,
                accounting=accounting, scaling_rule="q38/make_configs.py:shape_for; width grid 128:64:1600")


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--check", action="store_true", help="recompute and compare with the files on disk")
    ap.add_argument("--plan", default="", help="also write the scaling fit behind the widths (per-budget optima, power laws, leave-one-out, targets) to this JSON file")
    a = ap.parse_args(argv)
    if a.plan:
        fits, size_law, data_law, left_out = sweep_prior()
        targets = {}
        for name, compute in BUDGETS.items():
            ranked, n_target, d_target = ranked_widths(compute, batch_for(compute))
            targets[name] = dict(compute=compute, active_target=n_target, tokens_target=d_target,
                                 nearest_widths=[dict(hidden=r["hidden"], log_distance_squared=r["distance"]) for r in ranked[:3]])
        plan = dict(source=str(SWEEP_RESULTS.relative_to(ROOT)), budget_fits=fits,
                    power_laws=dict(active_log10_slope=float(size_law[0]), active_log10_intercept=float(size_law[1]),
                                    tokens_log10_slope=float(data_law[0]), tokens_log10_intercept=float(data_law[1])),
                    leave_one_budget_out=left_out, targets=targets,
                    limitations=["The Q35 sweep is a prior for a different architecture.", "Only c1 lies at a measured budget; c2-c4 extrapolate.",
                                 "No Q38 loss is predicted."])
        with open(a.plan, "w") as f:
            f.write(json.dumps(plan, indent=2) + "\n")
    for name in BUDGETS:
        preset, path = build(name), PRESET_DIR / f"q38_{name}.json"
        if a.check:
            if json.loads(path.read_text()) != preset:
                raise SystemExit(f"Generated preset differs: {path}")
        else:
            path.write_text(json.dumps(preset, indent=2) + "\n")
        acc = preset["accounting"]
        print(f"{name}: h{preset['model']['hidden']} L{preset['model']['layers']} Na={acc['active_nonvocab_params']:,} "
              f"D={acc['train_tokens']:,} steps={acc['steps']:,}")


if __name__ == "__main__":
    main()
