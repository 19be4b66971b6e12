"""Ledger and preset checks (behavioural counterparts of the reference's tests/test_presets.py and
tests/test_flops_audit.py)."""
import copy
import json

import pytest

from q38.flops import _count_backbone, count, validate_resume_accounting
from q38.presets import ROOT, budget_tokens, load_preset, model_config, preset_budget, preset_names

EXPECTED_TRAIN_FLOPS = {"q38_c1": 291_721_216, "q38_c2": 486_353_152, "q38_c3": 1_057_826_304, "q38_c4": 2_284_543_232}
EXPECTED_PARAMS = {"q38_c1": 167_752_070, "q38_c2": 326_609_782, "q38_c3": 778_030_326, "q38_c4": 1_804_657_560}


def small():
    return dict(hidden_size=128, num_hidden_layers=4, vocab_size=10112, num_experts=64, num_experts_per_tok=4,
                moe_intermediate_size=64, shared_expert_intermediate_size=64, num_attention_heads=4,
                num_key_value_heads=1, head_dim=64, linear_num_key_heads=2, linear_num_value_heads=4,
                linear_key_head_dim=64, linear_value_head_dim=64, linear_conv_kernel_dim=4,
                layer_types=["linear_attention"] * 3 + ["full_attention"])


def test_presets_match_published_accounting():
    assert set(EXPECTED_TRAIN_FLOPS) <= set(preset_names())
    for name in EXPECTED_TRAIN_FLOPS:
        p = load_preset(name)
        cfg = model_config(p["model"], 10112, 4096)
        assert (cfg.num_experts, cfg.num_experts_per_tok) == (64, 5) and cfg.ngram_rows > 0 and cfg.mtp
        tokens, fc = preset_budget(name, 10112, 4096)
        assert fc["train_flops_per_token"] == EXPECTED_TRAIN_FLOPS[name] == p["accounting"]["train_flops_per_token"]
        assert fc["total_params_all"] == EXPECTED_PARAMS[name]
        assert tokens == p["train"]["tokens"]
        assert fc["accounting_method"] == p["accounting"]["accounting_method"]
        target = p["compute"] * (1 - p["accounting"]["compute_reserve_fraction"])
        assert tokens * fc["train_flops_per_token"] <= target < (tokens + p["train"]["batch_tokens"]) * fc["train_flops_per_token"]
        assert fc["active_nonvocab_params"] / fc["total_nonvocab_params"] > 0.10


def test_preset_generator_reproduces_files():
    from q38 import make_configs
    for name in make_configs.BUDGETS:
        assert json.loads((ROOT / f"configs/q38_{name}.json").read_text()) == make_configs.build(name)


def test_widths_come_from_the_isoflops_fit(tmp_path):
    """The scaling fit over the 19 completed Q35 runs: slopes and per-budget optima as published with the reference
    (audits/q38_config_plan.json there), and the nearest width per Q38 budget."""
    import json
    from q38 import make_configs
    fits, size_law, data_law, left_out = make_configs.sweep_prior()
    assert [f["budget"] for f in fits] == ["1e16", "3e16", "1e17", "3e17"] and all(f["inside_grid"] for f in fits)
    assert abs(size_law[0] - 0.7767049) < 1e-6 and abs(data_law[0] - 0.4360745) < 1e-6
    assert abs(fits[0]["active_opt"] - 1651930.3) < 1.0 and abs(fits[3]["tokens_opt"] - 1235554175.5) < 1e3
    assert abs(left_out[3]["active_exponent"] - 0.8093009) < 1e-6
    chosen = {name: make_configs.ranked_widths(c, make_configs.batch_for(c))[0][0]["hidden"] for name, c in make_configs.BUDGETS.items()}
    assert chosen == {"c1": 448, "c2": 576, "c3": 768, "c4": 1024}
    with pytest.raises(ValueError, match="three completed runs"):
        make_configs.fit_sweep([dict(budget="1e16", compute=1e16, active_params=1e6 * (i + 1), train_tokens=1e8, bpb=1.4) for i in range(2)])
    make_configs.main(["--check", "--plan", str(tmp_path / "plan.json")])
    plan = json.loads((tmp_path / "plan.json").read_text())
    assert plan["targets"]["c2"]["nearest_widths"][0]["hidden"] == 576


def test_backbone_terms():
    c = small()
    r = _count_backbone(c, 8192)
    assert r["breakdown"]["attn_score"] == 2 * 8192 * 4 * 64                 # two causal matmuls at half density
    assert _count_backbone(c, 4096)["breakdown"]["attn_score"] == 8192 * 4 * 64
    q, kv, h = 4 * 64, 64, 128
    assert r["breakdown"]["full_projections"] == 2 * h * (q + kv + kv + q) + 2 * h * q   # q, k, v, gate, o
    assert r["breakdown"]["gdn_core"] == 3 * 4 * 8 * 64 ** 2
    assert r["train_flops_per_token"] == 27_780_096
    assert r["fwd_flops_per_token"] == sum(r["breakdown"].values())
    assert r["extra_router_shared_gate_train_flops_per_token"] == 6 * 4 * 128 * (64 + 1)
    d = copy.deepcopy(c)
    d["linear_num_value_heads"] = 8
    assert _count_backbone(d, 8192)["breakdown"]["gdn_core"] == 2 * r["breakdown"]["gdn_core"]


def test_indexer_projection_is_charged_twice_not_three_times():
    for mtp in (False, True):
        r = count(dict(small(), mtp=mtp), 64)
        proj = r["breakdown"]["indexer_projections"]
        assert r["train_flops_per_token"] == 3 * (r["fwd_flops_per_token"] - proj) + 2 * proj + r["distill_target_flops"]
        assert r["breakdown"]["gdn_core"] == _count_backbone(small(), 64)["breakdown"]["gdn_core"]


def test_resume_rejects_changed_accounting():
    now = count(small(), 4096)
    validate_resume_accounting(dict(flops_accounting=now["accounting_method"], flops_per_token=now["train_flops_per_token"]), now)
    with pytest.raises(ValueError, match="FLOPs accounting changed"):
        validate_resume_accounting(dict(flops_accounting="q38_sparse_mhc_ngram_mtp_v1",
                                        flops_per_token=now["train_flops_per_token"]), now)
    with pytest.raises(ValueError, match="FLOPs accounting changed"):
        validate_resume_accounting(dict(flops_per_token=now["train_flops_per_token"] + 1), now)


def test_budget_is_whole_batches():
    assert budget_tokens(100, 1e9, 4096) % 4096 == 0
    assert budget_tokens(100, 1e9, 4096) * 100 <= 1e9


def test_flops_audit_agrees_with_instantiated_models():
    """Parameter counts of the models built from the presets equal the presets' accounting, and the ledger reproduces
    the recorded train FLOPs per token (q38.utils.audit_flops)."""
    from q38.utils.audit_flops import audit
    for name in ("q38_c1", "q38_c2"):
        report = audit(name, 4096)
        assert report["failures"] == [], report["failures"]
        assert report["weight_gemm_flops_per_token"] < report["fwd_flops_per_token"]


def test_backbone_ledger_equals_the_pinned_megatron_formula(tmp_path):
    """Counterpart of the reference's tests/test_flops_audit.py: the hand expansion of the pinned Megatron formula equals the
    ledger's Megatron component for the 19 archived configs and the 24 widths of the family; a source file with another hash
    is refused; a stand-in function is extracted by AST and compared."""
    import hashlib
    from q38.utils import audit_flops
    report = audit_flops.backbone_report()
    assert report["failures"] == [] and len(report["archived_configs"]) == 19 and len(report["canonical_family"]) == 24
    first = report["archived_configs"][0]
    assert (first["shape"], first["megatron_train_flops_per_token"], first["router_and_shared_gate_train_flops_per_token"]) == ("h128_L4", 27580416, 199680)
    assert report["delta_rule_kernels"]["products_64x64x64_per_chunk_and_value_head"] == {
        "gdn_scan_fwd_kernel": 4, "gdn_scan_bwd_kernel": 8, "gdn_prep_fwd_kernel": 4, "gdn_prep_bwd_kernel": 12}
    fake = tmp_path / "training.py"
    fake.write_text("import os\n\ndef num_floating_point_operations(args, batch_size):\n"
                    "    assert is_gated_delta_net_variant(args.experimental_attention_variant) and not is_hybrid_model(args)\n"
                    "    return 123 * batch_size * args.seq_length\n")
    with pytest.raises(ValueError, match="not the pinned Megatron revision"):
        audit_flops.load_megatron_function(fake)
    function = audit_flops.load_megatron_function(fake, hashlib.sha256(fake.read_bytes()).hexdigest())
    row = audit_flops.audit_backbone(small(), 8192, function)
    assert row["megatron_function_evaluated"] == 123 and any("pinned Megatron function gives" in f for f in row["failures"])
    assert audit_flops.main(["--backbone", "--output", str(tmp_path / "audit.json")]) == 0


def test_launcher_builds_loopback_torchrun_command():
    from q38.launch import command
    single = command("q38.train", 1, 29500, ["--preset", "q38_c1"])
    multi = command("q38.train", 8, 29511, ["--preset", "q38_c2"])
    assert single[1:3] == ["-m", "q38.train"]
    assert "--nproc-per-node=8" in multi and multi[multi.index("--master-addr") + 1] == "127.0.0.1" and multi[-2:] == ["--preset", "q38_c2"]


def test_owner_assignment_balances_segments_and_newton_schulz_work():
    """Owner-computes layout of q38_c2 on 8 ranks (shapes only, meta device): no rank's segment is more than 1.35 x the mean and no
    rank's Newton-Schulz work more than 1.3 x the mean; balancing the Newton-Schulz FLOPs alone left both n-gram tables on two
    ranks with segments of twice the mean."""
    import torch
    from q38.models import Q38ForCausalLM
    from q38.optim.hybrid import split_parameters
    from q38.parallel.arena import GROUPS, Unit, assign_owners, newton_schulz_flops
    cfg = model_config(load_preset("q38_c2")["model"], 10112, 4096)
    with torch.device("meta"):
        model = Q38ForCausalLM(cfg)
    groups = split_parameters(model, True)
    for world in (2, 4, 8):
        units = [Unit(n, p, g, i) for g, items in zip(GROUPS, groups) for i, (n, p) in enumerate(items)]
        load = assign_owners(units, world)
        sizes = [sum(u.numel for u in units if u.owner == r) for r in range(world)]
        work = [sum(newton_schulz_flops(tuple(u.param.shape)) for u in units if u.owner == r and u.group == "muon") for r in range(world)]
        assert max(sizes) <= 1.35 * sum(sizes) / world, (world, sizes)
        assert max(work) <= 1.3 * sum(work) / world, (world, work)
        assert max(load) <= 1.05 * sum(load) / world
        assert {u.owner for u in units} == set(range(world))


def test_committed_audit_files_are_what_the_tools_generate(tmp_path):
    from q38 import make_configs
    from q38.utils import audit_flops
    assert audit_flops.main(["--backbone", "--output", str(tmp_path / "flops_audit.json")]) == 0
    make_configs.main(["--check", "--plan", str(tmp_path / "q38_config_plan.json")])
    for name in ("flops_audit.json", "q38_config_plan.json"):
        assert json.loads((tmp_path / name).read_text()) == json.loads((ROOT / "audits" / name).read_text()), name
