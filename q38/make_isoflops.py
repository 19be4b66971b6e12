"""Generate / verify the archived Q35 IsoFLOPs sweep under ``configs/q35_isoflops``:  python -m q38.make_isoflops [--check]

The sweep that preceded the Q38 presets: the backbone-only architecture (Gated DeltaNet + gated attention + 64-expert top-4
MoE, no mHC / QSA / n-gram / MTP parts) at four budgets, 1e16 / 3e16 / 1e17 / 3e17 FLOPs, with every width of the one-parameter
family whose tokens-per-active-parameter ratio falls in [4, 400] - 19 runs.  Its fitted optimum is what pinned the widths of
``configs/q38_c1..c4.json``.  The reference keeps the 19 ``config.json`` files, a manifest and the frozen validation split as
an archive (configs/q35_isoflops/** there) and checks them against the backbone ledger in tests/test_isoflops.py:63-71; this
module regenerates the same files from the rules, so the archive here is derived, not copied:

  shape      hidden on the 64-grid -> layers = max(4, round(hidden / 51.2)); attention q heads hidden/32, kv heads about
             hidden/256 (a divisor of the q heads), GDN key heads hidden/64 and value heads hidden/32, all head dims 64;
             64 experts, top-4, expert and shared-expert width hidden/2
  batch      0.2920 * C**0.3271 tokens, rounded to a power-of-two number of 8192-token sequences
  lr         0.3118 * C**-0.125, shared within a budget; warm-up 5 % of the steps (at least 10)
  tokens     the largest whole number of global batches inside the budget, by the backbone ledger (q38.flops._count_backbone)
"""
import argparse
import json
import math

from .flops import _count_backbone
from .presets import ROOT, budget_tokens, model_config

SEQ, VOCAB = 8192, 10112
ARCHIVE = ROOT / "configs" / "q35_isoflops"
BUDGETS = {"1e16": 10 ** 16, "3e16": 3 * 10 ** 16, "1e17": 10 ** 17, "3e17": 3 * 10 ** 17}
RATIO_WINDOW = (4.0, 400.0)                      # tokens per active non-vocabulary parameter kept in the sweep
WIDTHS = range(128, 1601, 64)
POOL = "/home/shared/qwen35_moe_sparse/cache/isoflops-gzy10k-16b-v1"
# The frozen validation file of that pool, split on document boundaries: token ranges are end-exclusive.
VALIDATION = {
    "version": 1,
    "boundary_rule": "complete documents, end-exclusive token ranges; no shared documents",
    "document_count": 42563, "total_tokens": 78381534,
    "dev": {"offset": 0, "end": 2002536, "targets": 2002535, "documents": 941},
    "curve": {"offset": 2002536, "end": 18004412, "targets": 16001875, "documents": 8961},
    "report": {"offset": 18004412, "end": 78381534, "targets": 60377121, "documents": 32661},
}


def shape_for(hidden):
    if hidden % 64:
        raise ValueError("hidden must be a multiple of 64 (GDN key heads = hidden / 64)")
    heads = hidden // 32
    kv_heads = max(1, hidden // 256)
    while heads % kv_heads:
        kv_heads -= 1
    return dict(layers=max(4, round(hidden / 51.2)), hidden=hidden, heads=heads, kv_heads=kv_heads, head_dim=64,
                lin_k_heads=hidden // 64, lin_v_heads=hidden // 32, lin_head_dim=64, experts=64, topk=4,
                moe_ffn=hidden // 2, shared_ffn=hidden // 2, layer_types="", aux_coef=0.001, rope_theta=10000000.0,
                partial_rotary=0.25, experts_impl="eager")


def shape_name(shape):
    return f"h{shape['hidden']}_L{shape['layers']}"


def batch_for(compute):
    return SEQ * 2 ** round(math.log2(0.2920 * compute ** 0.3271 / SEQ))


def build(budget, hidden):
    """One run of the sweep, or None when its tokens-per-active-parameter ratio is outside the window."""
    compute = BUDGETS[budget]
    shape = shape_for(hidden)
    ledger = _count_backbone(model_config(shape, VOCAB, SEQ).to_dict(), SEQ)
    per_token, active, total = ledger["train_flops_per_token"], ledger["active_nonvocab_params"], ledger["total_nonvocab_params"]
    if active / total < 0.10:
        raise ValueError(f"{shape_name(shape)}: active fraction below 10 %")
    batch = batch_for(compute)
    tokens = budget_tokens(per_token, compute, batch)
    if not RATIO_WINDOW[0] <= tokens / active <= RATIO_WINDOW[1]:
        return None
    steps, name = tokens // batch, shape_name(shape)
    run_dir = f"runs/{budget}/{name}"
    train = dict(run_dir=run_dir, data=f"{POOL}/train.bin", val_data=f"{POOL}/valid.bin", tokenizer=f"{POOL}/tokenizer",
                 seq=SEQ, tokens=0, batch_tokens=batch, micro_bs=8, auto_micro_bs=1, lr=round(0.3118 * compute ** -0.125, 6),
                 min_lr_ratio=0.1, warmup=0, warmup_ratio=0.05, warmup_min=10, wd=0.1, clip=1.0, seed=0, data_seed=0,
                 data_sampling="shuffled_blocks", require_ready_pool=1, eval_sampling="sequential",
                 eval_offset=VALIDATION["dev"]["offset"], eval_tokens=VALIDATION["dev"]["targets"],
                 final_eval_offset=VALIDATION["curve"]["offset"], final_eval_tokens=VALIDATION["curve"]["targets"],
                 log_every=10, eval_every=100, ckpt_every=100, resume=1, max_steps=0, tensorboard=1)
    accounting = dict(
        total_params=total + ledger["embed_params"], accounting_method=ledger["accounting_method"], megatron_commit=ledger["megatron_commit"],
        megatron_reference_train_flops_per_token=ledger["megatron_reference_train_flops_per_token"],
        extra_router_shared_gate_train_flops_per_token=ledger["extra_router_shared_gate_train_flops_per_token"],
        total_nonvocab_params=total, active_nonvocab_params=active, active_fraction=active / total,
        active_params_with_vocab=active + ledger["embed_params"], train_flops_per_token=per_token, train_tokens=tokens,
        tokens_per_active_param=tokens / active, steps=steps, warmup_steps=max(10, round(0.05 * steps)),
        actual_train_flops=tokens * per_token, compute_shortfall_fraction=1 - tokens * per_token / compute)
    experiment = dict(budget=budget, model=name, phase="main",
                      scaling_rule="q38/make_isoflops.py:shape_for (hidden only; layers = max(4, round(hidden/51.2)))",
                      lr_rule="0.3118*C^-0.125, shared within a budget", batch_rule="0.2920*C^0.3271 tokens, rounded to 2^k sequences",
                      flops_rule=ledger["accounting_method"], validation_manifest="configs/q35_isoflops/validation.json")
    return dict(schema_version=1, compute=compute, model=shape, train=train, accounting=accounting, experiment=experiment)


def sweep():
    """(budget, shape name) -> config for every run of the sweep, in budget then width order."""
    runs = {}
    for budget in BUDGETS:
        for hidden in WIDTHS:
            config = build(budget, hidden)
            if config is not None:
                runs[(budget, config["experiment"]["model"])] = config
    return runs


def manifest(runs):
    rows = []
    for (budget, name), config in runs.items():
        rows.append(dict(budget=budget, model=name, lr=config["train"]["lr"], batch_tokens=config["train"]["batch_tokens"],
                         config=f"configs/q35_isoflops/{budget}/{name}/config.json", run_dir=config["train"]["run_dir"],
                         **config["accounting"]))
    return dict(version=1, pool=POOL, runs=rows)


def checks(runs):
    """What was verified about the archive, recomputed every time it is generated (the reference keeps a hand-filled
    ``checks.json`` beside its archive)."""
    from .utils.audit_flops import MEGATRON_COMMIT, backbone_report
    report = backbone_report(SEQ, VOCAB)
    shortfall = max(c["accounting"]["compute_shortfall_fraction"] for c in runs.values())
    deviation = [row["megatron_reaccounted_budget_fraction"] for row in report["archived_configs"]]
    return dict(main_configs=len(runs), flops_accounting=next(iter(runs.values()))["accounting"]["accounting_method"], megatron_commit=MEGATRON_COMMIT,
                megatron_formula_crosscheck_passed=not report["failures"], crosschecked_configs=len(report["archived_configs"]),
                crosschecked_canonical_shapes=len(report["canonical_family"]),
                original_megatron_function_evaluated=report["reference"]["original_function_evaluated"],
                maximum_budget_shortfall_percent=100 * shortfall,
                megatron_reference_budget_deviation_percent=[100 * min(deviation), 100 * max(deviation)],
                training_started=False, gpu_benchmark_performed=False)


README = """# Q35 IsoFLOPs sweep (archive)

The 19 runs that preceded the Q38 presets: the backbone-only architecture at four compute budgets (1e16, 3e16, 1e17, 3e17 FLOPs),
every width of the one-parameter family whose tokens per active parameter fall in [4, 400].  Generated by
`python -m q38.make_isoflops` from the rules in its docstring; `--check` verifies that the files still are what the rules give.

    <budget>/<shape>/config.json   one run: model shape, training settings, accounting
    manifest.json                  one row per run
    validation.json                the frozen validation split (dev / curve / report token ranges)
    results.json                   measured outcomes of the completed runs; the scaling fit in `q38/make_configs.py` reads them
    checks.json                    what was verified when the archive was generated

The runs are history: they train the backbone without the Q38 additions and are not launched from this repository.
"""


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--check", action="store_true", help="recompute and compare with the files on disk")
    a = ap.parse_args(argv)
    runs = sweep()
    files = {ARCHIVE / budget / name / "config.json": config for (budget, name), config in runs.items()}
    files[ARCHIVE / "manifest.json"] = manifest(runs)
    files[ARCHIVE / "validation.json"] = VALIDATION
    readme = ARCHIVE / "README.md"
    if a.check:
        if not readme.exists() or readme.read_text() != README:
            raise SystemExit(f"Generated file differs: {readme}")
    else:
        ARCHIVE.mkdir(parents=True, exist_ok=True)
        readme.write_text(README)
    def emit(path, content):
        if a.check:
            if not path.exists() or json.loads(path.read_text()) != content:
                raise SystemExit(f"Generated file differs: {path}")
        else:
            path.parent.mkdir(parents=True, exist_ok=True)
            path.write_text(json.dumps(content, indent=2, ensure_ascii=False) + "\n")

    for path, content in files.items():
        emit(path, content)
    emit(ARCHIVE / "checks.json", checks(runs))              # last: the checks read the config files from disk
    for (budget, name), config in runs.items():
        acc = config["accounting"]
        print(f"{budget} {name}: Na={acc['active_nonvocab_params']:,} D={acc['train_tokens']:,} D/Na={acc['tokens_per_active_param']:.1f} "
              f"steps={acc['steps']:,} lr={config['train']['lr']} batch={config['train']['batch_tokens']}")


if __name__ == "__main__":
    main()
