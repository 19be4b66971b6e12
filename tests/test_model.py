"""Tiny-model checks on CPU: parameter ledger, losses, optimizer step, HF export, checkpointing
(counterpart of the reference's tests/test_model.py) plus oracle cross-checks of the op specifications."""
import torch
import torch.nn.functional as F

from q38.flops import count
from q38.losses import LossModel
from q38.models import Q38ForCausalLM, modeling
from q38.muon import HybridOptimizer, Muon, newton_schulz


class CE(torch.nn.Module):
    def forward(self, weight, hidden, labels):
        return F.cross_entropy(F.linear(hidden, weight), labels)


def total_loss(parts):
    ce, aux, mtp, kl = parts
    return ce + 0.001 * aux + 0.3 * mtp + 0.05 * kl


def test_smoke_forward_backward_step_and_export(tiny_config, tmp_path):
    from transformers import AutoModelForCausalLM
    from q38.models.export import save_hf
    torch.manual_seed(0)
    model = Q38ForCausalLM(tiny_config)
    assert sum(p.numel() for p in model.parameters()) == count(tiny_config.to_dict(), 128)["total_params_all"]
    ids = torch.randint(1, 128, (1, 128))
    wrapped = LossModel(model, 8, 2, ce=CE())
    loss = total_loss(wrapped(ids, ids.roll(-1, 1)))
    assert torch.isfinite(loss)
    loss.backward()
    for name, p in model.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad).all(), name
    opt = HybridOptimizer(model, lr=1e-3, weight_decay=0.1)
    opt.step()
    opt.zero_grad()
    assert opt.state_dict()["muon"] is not None
    model.eval()
    with torch.no_grad():
        expected = model(input_ids=ids, use_cache=False).logits
    save_hf(model, tmp_path / "hf", dtype=None)
    loaded = AutoModelForCausalLM.from_pretrained(tmp_path / "hf", trust_remote_code=True, local_files_only=True).eval()
    with torch.no_grad():
        actual = loaded(input_ids=ids, use_cache=False).logits
    torch.testing.assert_close(actual, expected, rtol=0, atol=0)
    assert loaded.config.model_type == "qwen38_moe_sparse"
    assert any(k.startswith("mtp.") for k in loaded.state_dict())


def test_gradient_checkpointing_matches(tiny_config):
    torch.manual_seed(0)
    model = Q38ForCausalLM(tiny_config).train()
    wrapped = LossModel(model, 8, 2, ce=CE())
    ids = torch.randint(1, 128, (1, 128))
    runs = []
    for ckpt in (False, True):
        model.model.gradient_checkpointing = ckpt
        parts = wrapped(ids, ids.roll(-1, 1))
        total_loss(parts).backward()
        assert all(block.stats_sink is None for block in model.moe_blocks())
        assert len(wrapped.last_stats.counts) == tiny_config.num_hidden_layers + 1      # L routers + the MTP block's
        runs.append(([p.detach() for p in parts], {n: p.grad.clone() for n, p in model.named_parameters()}))
        model.zero_grad(set_to_none=True)
    (plain, plain_grads), (ck, ck_grads) = runs
    for a, b in zip(plain, ck):
        torch.testing.assert_close(b, a, rtol=0, atol=0)
    for name in plain_grads:
        torch.testing.assert_close(ck_grads[name], plain_grads[name], rtol=1e-5, atol=1e-6, msg=name)


def test_state_dict_layout(tiny_config):
    model = Q38ForCausalLM(tiny_config)
    keys = list(model.state_dict())
    assert keys[0] == "model.embed_tokens.weight"
    gdn = [k.split("linear_attn.")[1] for k in keys if k.startswith("model.layers.0.linear_attn.")]
    assert gdn == ["dt_bias", "A_log", "conv1d.weight", "norm.weight", "out_proj.weight", "in_proj_qkv.weight",
                   "in_proj_z.weight", "in_proj_b.weight", "in_proj_a.weight"]
    mhc = [k.split("mhc.0.")[1] for k in keys if k.startswith("model.mhc.0.")]
    assert mhc == ["b_pre", "b_post", "b_res", "alphas", "A.weight", "B.weight"]
    assert [k for k in keys if k.startswith("model.indexers.")] == [f"model.indexers.3.{w}.weight" for w in ("wq", "wk", "ww")]
    assert [k for k in keys if k.startswith("model.ngram.")] == [f"model.ngram.{s}" for s in
                                                                   ("emb2.weight", "emb3.weight", "norm.weight", "gate.weight", "gate.bias")]
    assert "lm_head.weight" in keys and model.lm_head.weight is model.model.embed_tokens.weight
    assert {k.split(".")[1] for k in keys if k.startswith("mtp.")} == {"enorm", "hnorm", "proj", "block", "norm"}
    top = [k.split(".")[1] for k in keys if k.startswith("model.") and k.count(".") >= 2]
    order = [t for i, t in enumerate(top) if t not in top[:i]]
    assert order == ["embed_tokens", "layers", "norm", "mhc", "indexers", "ngram"]
    assert model.model.embed_tokens.weight[tiny_config.pad_token_id].abs().sum() == 0


def test_optimizer_split_counts(tiny_config):
    model = Q38ForCausalLM(tiny_config)
    opt = HybridOptimizer(model, lr=1e-3, weight_decay=0.1)
    names = opt.names
    assert "model.layers.0.linear_attn.conv1d.weight" in names["muon"]          # C matrices of 1 x 4
    assert "model.ngram.gate.weight" in names["muon"] and "model.indexers.3.ww.weight" in names["muon"]
    assert "mtp.proj.weight" in names["muon"] and "model.mhc.0.A.weight" in names["muon"]
    assert "model.embed_tokens.weight" in names["decay"] and "model.layers.0.mlp.gate.weight" in names["decay"]
    assert "model.layers.0.linear_attn.in_proj_a.weight" in names["decay"]
    assert "model.ngram.emb2.weight" in names["no_decay"] and "model.mhc.0.b_res" in names["no_decay"]
    assert "model.layers.0.linear_attn.A_log" in names["no_decay"] and "model.ngram.gate.bias" in names["no_decay"]
    assert sum(len(v) for v in names.values()) == len(list(model.parameters()))


def test_chunked_delta_rule_matches_recurrence():
    torch.manual_seed(1)
    q, k = torch.randn(2, 150, 2, 16), torch.randn(2, 150, 2, 16)
    v, g, beta = torch.randn(2, 150, 6, 16), -torch.rand(2, 150, 6), torch.rand(2, 150, 6)
    a = modeling.gated_delta_rule_chunked(q, k, v, g, beta)
    b = modeling.gated_delta_rule_recurrent(q, k, v, g, beta)
    torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5)


def test_ngram_hash_is_wrapping_int64_and_respects_eos():
    ng = modeling.NGramEmbedding(8, 128, 64, eos_id=0)
    ids = torch.tensor([[5, 9, 0, 7, 3, 11]])
    i2, i3 = ng.indices(ids)
    M = 1 << 64

    def wrap(x):
        x %= M
        return x - M if x >= (1 << 63) else x

    def mix(x):
        return wrap((x ^ (x >> 17)) * 2654435761)

    # The context window starts at the latest EOS (inclusive): the EOS token itself sees only placeholders,
    # the tokens after it may see the EOS but nothing before it.
    prev = [128, 5, 128, 0, 7, 3]
    prev2 = [128, 128, 128, 128, 0, 7]
    for t in range(6):
        a, b, c = prev[t], int(ids[0, t]), prev2[t]
        assert int(i2[0, t]) == mix(wrap(a * 1000003) ^ wrap(b * 998244353)) % 64
        assert int(i3[0, t]) == mix(wrap(c * 1000033) ^ wrap(a * 998244353) ^ wrap(b * 1000000007)) % 64
    assert i2.min() >= 0 and i3.min() >= 0


def test_select_blocks_rules():
    torch.manual_seed(0)
    lp = torch.randn(2, 8 * 64, 8).log_softmax(-1)
    count, index = modeling.select_blocks(lp, 3)
    assert count.tolist() == [[1, 2, 3, 3, 3, 3, 3, 3]] * 2
    for b in range(2):
        for j in range(8):
            chosen = index[b, j, :count[b, j]].tolist()
            assert j in chosen and all(c <= j for c in chosen) and len(set(chosen)) == len(chosen)
    first = lp.view(2, 8, 64, 8)[:, :, 0]
    c2, i2 = modeling.select_blocks(first, 3)
    assert torch.equal(c2, count) and torch.equal(i2, index)              # only the first query of a block matters
    mask = modeling.block_sparse_mask(count, index, 512)
    assert mask[0, 200, 200] and not mask[0, 200, 201] and mask.sum(-1).min() >= 1


def test_qsa_recall_statistic(tiny_config):
    """QSA_STAT["on"] records, per QSA layer and training forward of the sparse phase, the share of the dense attention mass that
    lies in the selected blocks: within (0, 1] for a budget of one block, exactly 1 when the budget covers every causal block
    (reference: modeling_qwen3_8_moe.py:1114,1136-1142)."""
    torch.manual_seed(0)
    ids = torch.randint(1, 128, (1, 128))
    recalls = {}
    for budget in (1, 2):
        tiny_config.qsa_blocks = budget
        model = Q38ForCausalLM(tiny_config).train()
        model.model.qsa_dense = False
        modeling.QSA_STAT.clear()
        modeling.QSA_STAT["on"] = True
        try:
            LossModel(model, 8, 2, ce=CE())(ids, ids.roll(-1, 1))
            recalls[budget] = list(modeling.QSA_STAT["recall"])
        finally:
            modeling.QSA_STAT.clear()
    assert len(recalls[1]) == 1 and 0.0 < recalls[1][0] < 1.0                       # one QSA layer in four; 128 tokens = two blocks
    assert abs(recalls[2][0] - 1.0) < 1e-5
    model.eval()
    with torch.no_grad():
        model(input_ids=ids, use_cache=False)
    assert "recall" not in modeling.QSA_STAT                                        # off: nothing recorded


def test_mhc_initialisation_is_a_residual_connection():
    torch.manual_seed(0)
    mhc = modeling.MHC(32, 4, 4, slot=1, iters=20)
    X = torch.randn(2, 5, 1, 32).expand(-1, -1, 4, -1).contiguous()
    xin, state = mhc.pre(X)
    torch.testing.assert_close(xin, X[:, :, 0], rtol=1e-5, atol=1e-5)         # pre sums to 1 over identical branches
    y = torch.randn(2, 5, 32)
    out = mhc.post(y, state)
    torch.testing.assert_close(out.mean(2), X[:, :, 0] + y, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(state[2].sum(-1), torch.ones(2, 5, 4), rtol=1e-3, atol=1e-3)


def test_muon_orthogonalises_and_batches():
    torch.manual_seed(0)
    g = torch.randn(3, 24, 48)
    o = newton_schulz(g).float()
    s = torch.linalg.svdvals(o)
    assert s.min() > 0.3 and s.max() < 1.4
    p = torch.nn.Parameter(torch.randn(3, 48, 24))
    p.grad = torch.randn_like(p)
    before = p.detach().clone()
    Muon([p], lr=0.01).step()
    step = (p.detach() - before * (1 - 0.01 * 0.1)).norm() / before.numel() ** 0.5
    assert abs(step.item() / (0.01 * 0.2) - 1) < 0.4          # RMS of a semi-orthogonal update is 1/sqrt(max dim): step RMS ~ 0.2 lr


def test_reference_import_paths_and_inference_entry_point(tiny_config):
    """The import paths a user of the reference has in their scripts resolve here: the model package, the optimizer module and
    `optimize_for_inference`, which on a CPU model only switches to evaluation mode and reports the module counts."""
    from q38.inference import compile_inference_norms, optimize_for_inference
    from q38.models.qwen3_8_moe import Qwen3_8MoeForCausalLM, Qwen3_8MoeTextConfig, source_info
    from q38.muon import HybridOptimizer as FromOldPath, MUON_MAX_CHUNK_ELEMENTS
    from q38.train import LossModel as FromTrain, gdn_kernel, install_fast_paths
    from q38.flops import ACCOUNTING_METHOD
    from q38.data import CHUNK_CHARS
    assert (MUON_MAX_CHUNK_ELEMENTS, CHUNK_CHARS, ACCOUNTING_METHOD) == (64 * 1024 * 1024, 100_000, "megatron_b92c3ed_plus_router_shared_gate_v1")
    assert FromTrain is LossModel and callable(gdn_kernel)
    assert install_fast_paths(Q38ForCausalLM(tiny_config))["experts"] == "reference (PyTorch)"
    assert FromOldPath is HybridOptimizer and Qwen3_8MoeTextConfig is type(tiny_config)
    assert Qwen3_8MoeForCausalLM.__name__ == "Qwen3_8MoeForCausalLM" and set(source_info()["files"]) == {"modeling_qwen3_8_moe.py", "configuration_qwen3_8_moe.py"}
    model = Q38ForCausalLM(tiny_config).train()
    info = optimize_for_inference(model)
    assert not model.training and info["backend"] is None and info["mhc"] == 2 * tiny_config.num_hidden_layers
    assert info["norms"] == compile_inference_norms(model) > 0 and info["gated_deltanet"] >= 3
