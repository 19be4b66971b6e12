"""Golden vectors from the UNMODIFIED reference (``baseline/_ref``), computed on CPU in fp32.

Run as a separate process (the reference's package is also called ``q38``):

    python baseline/ref_oracle.py model  <out.pt> '<json: shape, vocab, seq, batch, seed, mean_doc, lr, wd>'
    python baseline/ref_oracle.py ops    <out.pt>
    python baseline/ref_oracle.py curve  <out.json> '<json: shape, vocab, seq, batch, steps, lr, ...>'

``model``  builds ``Qwen3_8MoeForCausalLM`` with the given shape, records the initial ``state_dict``, then for the dense
           and the sparse QSA phase runs the reference's ``LossModel`` forward/backward (q38/train.py:215-264) and records
           the four loss terms and every parameter gradient; finally one ``HybridOptimizer.step()`` (q38/muon.py:122-152)
           on the sparse-phase gradients and the resulting parameters.
``ops``    evaluates the reference's pure functions on seeded random inputs: the chunked and the recurrent gated delta
           rule, Sinkhorn, ``select_blocks``, ``load_balancing_loss_func``, ``newton_schulz``.
``curve``  trains the reference for N optimizer steps on a seeded synthetic stream and writes the loss curve.
"""
import json
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import ref_compat  # noqa: E402

ref_compat.activate()
import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.nn.functional as F  # noqa: E402
from q38.models.qwen3_8_moe import Qwen3_8MoeForCausalLM, modeling_qwen3_8_moe as M  # noqa: E402
from q38.muon import HybridOptimizer, newton_schulz  # noqa: E402
from q38.presets import model_config  # noqa: E402
from q38.train import LossModel  # noqa: E402


class PlainCE(torch.nn.Module):
    def forward(self, weight, hidden, labels):
        return F.cross_entropy(F.linear(hidden, weight), labels)


def synthetic_tokens(vocab, eos, batch, seq, mean_doc, seed):
    rng = np.random.default_rng(seed)
    ids = rng.integers(1, vocab, (batch, seq + 1), dtype=np.int64)
    flat = ids.reshape(-1)
    position = -1
    while True:
        position += int(rng.geometric(1.0 / mean_doc))
        if position >= flat.size:
            break
        flat[position] = eos
    ids = torch.from_numpy(ids)
    return ids[:, :-1].contiguous(), ids[:, 1:].contiguous()


def build(spec):
    torch.manual_seed(spec.get("seed", 0))
    cfg = model_config(dict(spec["shape"]), spec["vocab"], spec["seq"], eos_token_id=spec.get("eos", 53), pad_token_id=0)
    model = Qwen3_8MoeForCausalLM(cfg).train()
    return cfg, model


def dump_model(out, spec):
    cfg, model = build(spec)
    shape = spec["shape"]
    x, y = synthetic_tokens(spec["vocab"], spec.get("eos", 53), spec["batch"], spec["seq"], spec.get("mean_doc", 96), spec.get("seed", 0) + 1)
    record = {"spec": spec, "config": cfg.to_dict(), "x": x, "y": y,
              "state": {k: v.detach().clone() for k, v in model.state_dict().items()}, "phases": {}}
    wrapped = LossModel(model, shape["experts"], shape["topk"], ce=PlainCE())
    coef = (1.0, shape.get("aux_coef", 0.001), spec.get("mtp_coef", 0.3), spec.get("kl_coef", 0.05))
    for phase in ("dense", "sparse"):
        model.zero_grad(set_to_none=True)
        model.model.qsa_dense = phase == "dense"
        parts = wrapped(x, y)
        sum(c * p for c, p in zip(coef, parts)).backward()
        record["phases"][phase] = {"losses": [float(p) for p in parts],
                                   "grads": {n: p.grad.detach().clone() for n, p in model.named_parameters() if p.grad is not None}}
    opt = HybridOptimizer(model, lr=spec.get("lr", 1e-3), weight_decay=spec.get("wd", 0.1))
    opt.step()
    record["after_step"] = {n: p.detach().clone() for n, p in model.named_parameters()}
    torch.save(record, out)


def dump_ops(out):
    g = torch.Generator().manual_seed(7)
    rec = {}
    B, S, H, D = 2, 192, 3, 16
    q, k = torch.randn(B, S, H, D, generator=g), torch.randn(B, S, H, D, generator=g)
    v = torch.randn(B, S, H, 24, generator=g)
    gate = -torch.rand(B, S, H, generator=g) * 0.5
    beta = torch.rand(B, S, H, generator=g)
    chunk = getattr(M.torch_chunk_gated_delta_rule, "__wrapped__", M.torch_chunk_gated_delta_rule)
    recur = getattr(M.torch_recurrent_gated_delta_rule, "__wrapped__", M.torch_recurrent_gated_delta_rule)
    o_chunk, _ = chunk(q, k, v, g=gate, beta=beta, use_qk_l2norm_in_kernel=True)
    o_rec, state = recur(q, k, v, g=gate, beta=beta, initial_state=None, output_final_state=True, use_qk_l2norm_in_kernel=True)
    rec["gdn"] = dict(q=q, k=k, v=v, g=gate, beta=beta, chunk=o_chunk, recurrent=o_rec, final_state=state)
    logits = torch.randn(5, 7, 4, 4, generator=g)
    rec["sinkhorn"] = dict(logits=logits, out3=M._sinkhorn(logits, 3), out20=M._sinkhorn(logits, 20))
    router = tuple(torch.randn(64, 8, generator=g) for _ in range(3))
    rec["aux"] = dict(router=router, loss=M.load_balancing_loss_func(router, 8, 2))
    mats = torch.randn(3, 24, 40, generator=g)
    tall = torch.randn(48, 16, generator=g)
    rec["ns"] = dict(mats=mats, out=newton_schulz(mats).float(), tall=tall, tall_out=newton_schulz(tall).float())
    S = 512
    scores = torch.randn(2, S, S, generator=g)
    ar = torch.arange(S)
    lp = torch.log_softmax(scores.masked_fill(ar[None, :] > ar[:, None], -1e9), dim=-1)
    lp_blk = torch.logsumexp(lp.view(2, S, S // M.BLK, M.BLK), dim=-1)
    sel = {}
    for budget in (1, 3, 8, 16):
        num, idx = M.select_blocks(lp_blk, budget)
        sel[budget] = (num, idx)
    rec["select"] = dict(lp_blk=lp_blk, out=sel)
    qh, kh = torch.randn(1, 4, 256, 16, generator=g), torch.randn(1, 2, 256, 16, generator=g)
    rec["block_mass"] = dict(q=qh, k=kh, scale=0.25, out=M.block_mass(qh, kh, 0.25))
    torch.save(rec, out)


def dump_curve(out, spec):
    cfg, model = build(spec)
    shape = spec["shape"]
    torch.save({k: v.detach().clone() for k, v in model.state_dict().items()}, str(out) + ".init.pt")     # the other side starts from the same weights
    wrapped = LossModel(model, shape["experts"], shape["topk"], ce=PlainCE())
    opt = HybridOptimizer(model, lr=spec["lr"], weight_decay=spec.get("wd", 0.1))
    coef = (1.0, shape.get("aux_coef", 0.001), spec.get("mtp_coef", 0.3), spec.get("kl_coef", 0.05))
    rows = []
    for step in range(spec["steps"]):
        x, y = synthetic_tokens(spec["vocab"], spec.get("eos", 53), spec["batch"], spec["seq"], spec.get("mean_doc", 96), 1000 + step % spec.get("distinct_batches", 8))
        model.model.qsa_dense = step < spec.get("dense_steps", 0)
        parts = wrapped(x, y)
        sum(c * p for c, p in zip(coef, parts)).backward()
        gn = torch.nn.utils.clip_grad_norm_(model.parameters(), spec.get("clip", 1.0))
        opt.step()
        opt.zero_grad()
        rows.append([step] + [float(p) for p in parts] + [float(gn)])
    Path(out).write_text(json.dumps({"spec": spec, "columns": ["step", "ce", "aux", "mtp", "kl", "grad_norm"], "rows": rows}))


if __name__ == "__main__":
    mode, out = sys.argv[1], sys.argv[2]
    if mode == "model":
        dump_model(out, json.loads(sys.argv[3]))
    elif mode == "ops":
        dump_ops(out)
    elif mode == "curve":
        dump_curve(out, json.loads(sys.argv[3]))
    else:
        raise SystemExit(f"unknown mode {mode}")
