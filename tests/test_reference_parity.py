"""Parity against the UNMODIFIED reference (a copy under ``baseline/_ref``), on CPU in fp32.

The reference's package is also called ``q38``, so its side runs in a child process (``baseline/ref_oracle.py``) that
writes golden vectors to a temporary file; this process loads them and compares this repository's model, losses,
optimizer and op specifications.  Skipped when ``baseline/_ref`` is absent (the copy is not part of the history).

Counterpart of the reference's tiny CPU workload: one forward/backward and one Muon+AdamW step, loss and gradient
parity (q38/train.py:215-264, q38/muon.py:122-152).
"""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch
import torch.nn.functional as F

ROOT = Path(__file__).resolve().parents[1]
ORACLE = ROOT / "baseline" / "ref_oracle.py"
pytestmark = pytest.mark.skipif(not (ROOT / "baseline" / "_ref" / "q38" / "train.py").is_file(),
                                reason="baseline/_ref (copy of the reference) is absent")

TINY = {"layers": 4, "hidden": 128, "heads": 4, "kv_heads": 2, "head_dim": 32, "lin_k_heads": 2, "lin_v_heads": 6, "experts": 8,
        "topk": 2, "moe_ffn": 32, "shared_ffn": 32, "n_branch": 4, "mhc_iters": 3, "qsa_blocks": 8, "indexer_heads": 4,
        "indexer_head_dim": 32, "ngram_rows": 1024, "mtp": 1}
# seq 256 has four 64-token blocks, fewer than the budget of 8: every causal block is selected.  The second case has
# 8 blocks and a budget of 2, so the indexer's selection decides what the attention sees.
CASES = {"budget_covers_all": dict(shape=TINY, vocab=10112, seq=256, batch=2, seed=0, mean_doc=96),
         "budget_selects": dict(shape={**TINY, "qsa_blocks": 2}, vocab=10112, seq=512, batch=1, seed=3, mean_doc=96)}


def run_oracle(mode, out, spec=None):
    cmd = [sys.executable, str(ORACLE), mode, str(out)] + ([json.dumps(spec)] if spec is not None else [])
    done = subprocess.run(cmd, cwd="/tmp", capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr[-3000:]
    return out


class PlainCE(torch.nn.Module):
    def forward(self, weight, hidden, labels):
        return F.cross_entropy(F.linear(hidden, weight), labels)


@pytest.fixture(scope="module")
def ops_golden(tmp_path_factory):
    return torch.load(run_oracle("ops", tmp_path_factory.mktemp("ref") / "ops.pt"), weights_only=False)


@pytest.mark.parametrize("case", list(CASES))
def test_losses_gradients_and_optimizer_step_match_reference(case, tmp_path):
    from q38.losses import LossModel
    from q38.models import Q38ForCausalLM
    from q38.muon import HybridOptimizer
    from q38.presets import model_config
    spec = CASES[case]
    gold = torch.load(run_oracle("model", tmp_path / "model.pt", spec), weights_only=False)
    cfg = model_config(dict(spec["shape"]), spec["vocab"], spec["seq"], eos_token_id=53, pad_token_id=0)
    model = Q38ForCausalLM(cfg).train()
    own = model.state_dict()
    assert list(own) == list(gold["state"]), "state-dict keys or their order differ from the reference"
    model.load_state_dict(gold["state"])
    wrapped = LossModel(model, spec["shape"]["experts"], spec["shape"]["topk"], ce=PlainCE())
    x, y = gold["x"], gold["y"]
    for phase in ("dense", "sparse"):
        model.zero_grad(set_to_none=True)
        model.model.qsa_dense = phase == "dense"
        parts = wrapped(x, y)
        (parts[0] + 0.001 * parts[1] + 0.3 * parts[2] + 0.05 * parts[3]).backward()
        ref = gold["phases"][phase]
        for name, ours, theirs in zip(("ce", "aux", "mtp", "kl"), parts, ref["losses"]):
            assert abs(float(ours.detach()) - theirs) <= 1e-5 * max(1.0, abs(theirs)), (phase, name, float(ours), theirs)
        largest = max(float(g.norm()) for g in ref["grads"].values())
        for name, p in model.named_parameters():
            theirs = ref["grads"][name]
            norm = float(theirs.norm())
            if norm < 1e-8 * largest:           # analytically zero in the reference: ours must be (near) zero too
                assert p.grad is None or float(p.grad.norm()) < 1e-6 * largest, (phase, name)
                continue
            assert p.grad is not None, (phase, name)
            # 1e-3 of the gradient's own norm; gradients below a millionth of the largest one are sums with heavy
            # cancellation in fp32, so they also get an absolute allowance of 1e-9 of the largest norm.
            error = float((p.grad - theirs).norm())
            assert error <= 1e-3 * norm + 1e-9 * largest, (phase, name, error / norm)
    # Optimizer parity is checked from the reference's own gradients: Newton-Schulz runs in bf16, where a last-bit
    # difference of an input flips roundings, so the step is compared on identical inputs and must then agree closely.
    for name, p in model.named_parameters():
        p.grad = gold["phases"]["sparse"]["grads"][name].clone()
    opt = HybridOptimizer(model, lr=1e-3, weight_decay=0.1)
    opt.step()
    for name, p in model.named_parameters():
        step_ref = gold["after_step"][name] - gold["state"][name]
        step_own = p.detach() - gold["state"][name]
        scale = float(step_ref.abs().max()) + 1e-12
        assert float((step_own - step_ref).abs().max()) <= 1e-3 * scale + 1e-9, name


def test_gated_delta_rule_specifications_match_reference(ops_golden):
    from q38.models import modeling
    g = ops_golden["gdn"]
    chunked = modeling.gated_delta_rule_chunked(g["q"], g["k"], g["v"], g["g"], g["beta"])
    recurrent = modeling.gated_delta_rule_recurrent(g["q"], g["k"], g["v"], g["g"], g["beta"])
    chunked = chunked[0] if isinstance(chunked, tuple) else chunked
    recurrent = recurrent[0] if isinstance(recurrent, tuple) else recurrent
    torch.testing.assert_close(chunked, g["chunk"].to(chunked.dtype), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(recurrent, g["recurrent"].to(recurrent.dtype), rtol=1e-4, atol=1e-5)


def test_sinkhorn_block_mass_and_selection_match_reference(ops_golden):
    from q38.models import modeling
    s = ops_golden["sinkhorn"]
    torch.testing.assert_close(modeling.sinkhorn(s["logits"], 3), s["out3"], rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(modeling.sinkhorn(s["logits"], 20), s["out20"], rtol=1e-5, atol=1e-6)
    b = ops_golden["block_mass"]
    torch.testing.assert_close(modeling.block_mass(b["q"], b["k"], b["scale"]), b["out"], rtol=1e-5, atol=1e-6)
    sel = ops_golden["select"]
    nb = sel["lp_blk"].shape[-1]
    for budget, (num, idx) in sel["out"].items():
        count, index = modeling.select_blocks(sel["lp_blk"], budget)
        k = min(budget, nb)
        assert torch.equal(count.reshape(num.shape[0], -1).long(), num.reshape(num.shape[0], -1).long()), budget
        ref_idx = idx[:, 0, :, :k].long()
        own_idx = index.reshape(ref_idx.shape[0], ref_idx.shape[1], -1)[..., :k].long()
        for qb in range(nb):               # only the first `count` entries are read; compare them as sets
            n = int(num.reshape(num.shape[0], -1)[0, qb])
            for batch in range(ref_idx.shape[0]):
                assert set(own_idx[batch, qb, :n].tolist()) == set(ref_idx[batch, qb, :n].tolist()), (budget, batch, qb)


def test_aux_loss_and_newton_schulz_match_reference(ops_golden):
    from q38.models import RouterStats
    from q38.muon import newton_schulz
    a = ops_golden["aux"]
    stats = RouterStats(8)
    for logits in a["router"]:
        probs = torch.softmax(logits.float(), -1)
        top = probs.topk(2, -1).indices
        counts = torch.zeros(8).index_add_(0, top.reshape(-1), torch.ones(top.numel()))
        stats.add(counts, probs.sum(0), probs.shape[0])
    torch.testing.assert_close(stats.loss(), a["loss"], rtol=1e-5, atol=1e-6)
    n = ops_golden["ns"]
    torch.testing.assert_close(newton_schulz(n["mats"]).float(), n["out"], rtol=0, atol=2e-2)
    torch.testing.assert_close(newton_schulz(n["tall"]).float(), n["tall_out"], rtol=0, atol=2e-2)
