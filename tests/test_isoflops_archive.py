"""The archived Q35 IsoFLOPs sweep (configs/q35_isoflops): every stored run is what the generator derives from its rules, agrees
with the backbone FLOPs ledger, and reproduces figures published with the reference's archive (tests/test_isoflops.py:63-71 and
configs/q35_isoflops/manifest.json of the reference)."""
import json

from q38 import make_isoflops
from q38.flops import _count_backbone
from q38.presets import ROOT, budget_tokens, load_training_config, model_config

# (budget, shape) -> (train FLOPs per token, train tokens, steps, warm-up steps, total parameters), read from the reference's manifest
PUBLISHED = {
    ("1e16", "h128_L4"): (27780096, 359923712, 5492, 275, 8235992),
    ("1e16", "h192_L4"): (46107648, 216858624, 3309, 165, 17517092),
    ("3e17", "h512_L10"): (386562048, 775946240, 5920, 296, 281494016),
}


def test_archive_is_what_the_generator_derives():
    make_isoflops.main(["--check"])
    runs = make_isoflops.sweep()
    assert len(runs) == 19
    assert [name for (budget, name) in runs if budget == "1e17"] == ["h256_L5", "h320_L6", "h384_L8", "h448_L9", "h512_L10"]


def test_archived_configs_match_the_backbone_ledger_and_the_budget():
    paths = sorted((ROOT / "configs/q35_isoflops").glob("*/*/config.json"))
    assert len(paths) == 19
    for path in paths:
        _, p = load_training_config(path)
        ledger = _count_backbone(model_config(p["model"], 10112, 8192).to_dict(), 8192)
        acc = p["accounting"]
        assert ledger["train_flops_per_token"] == acc["train_flops_per_token"], path
        assert budget_tokens(ledger["train_flops_per_token"], p["compute"], p["train"]["batch_tokens"]) == acc["train_tokens"], path
        assert acc["train_tokens"] * acc["train_flops_per_token"] <= p["compute"] and acc["compute_shortfall_fraction"] < 1e-3
        assert 0.10 <= acc["active_fraction"] < 0.16 and 4 <= acc["tokens_per_active_param"] <= 400


def test_published_figures_of_the_sweep_are_reproduced():
    manifest = json.loads((ROOT / "configs/q35_isoflops/manifest.json").read_text())
    rows = {(r["budget"], r["model"]): r for r in manifest["runs"]}
    for key, (per_token, tokens, steps, warmup, params) in PUBLISHED.items():
        row = rows[key]
        assert (row["train_flops_per_token"], row["train_tokens"], row["steps"], row["warmup_steps"], row["total_params"]) == (per_token, tokens, steps, warmup, params)


def test_recomputed_checks_reproduce_the_published_ones():
    """`checks.json` is recomputed from the FLOPs audit; its budget figures equal the ones published with the reference's
    archive (configs/q35_isoflops/checks.json there)."""
    checks = json.loads((ROOT / "configs/q35_isoflops/checks.json").read_text())
    assert checks["main_configs"] == checks["crosschecked_configs"] == 19 and checks["crosschecked_canonical_shapes"] == 24
    assert checks["megatron_formula_crosscheck_passed"] is True
    assert abs(checks["maximum_budget_shortfall_percent"] - 0.0652218892287948) < 1e-12
    low, high = checks["megatron_reference_budget_deviation_percent"]
    assert abs(low + 0.7315429477580793) < 1e-9 and abs(high + 0.45544902819839583) < 1e-9
