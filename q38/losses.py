"""Training objective of Q38: main CE, router balancing, MTP CE and indexer KL.

`LossModel.forward(x, y)` returns the four terms ``(ce, aux, mtp, kl)``; the trainer combines them as
``ce + aux_coef * aux + mtp_coef * mtp + kl_coef * kl``.  Vocabulary logits are never materialised on
the GPU path: the (hidden, tied embedding, target) triple goes to a fused linear + cross-entropy op.
Semantics follow the reference (q38/train.py:215-264):

* main CE: mean over all ``B*S`` targets;
* MTP: the MTP trunk reads the un-normalised hidden state and the embedding of the next token ``y``,
  predicts ``y`` shifted left by one; the last position and every position whose ``y`` is EOS are
  ignored; loss = summed CE / max(valid, 1);
* KL: mean over QSA layers of the per-layer indexer KL;
* aux: balancing loss over the routers of all layers plus the MTP block, recorded only during this
  forward (activation-checkpoint recomputation does not record again).
"""
import torch
import torch.nn.functional as F

from .models import RouterStats, modeling


def linear_cross_entropy(weight, hidden, target, reduction="mean"):
    """CE of ``hidden @ weight.T`` against ``target`` (ignore index -100); fused on the GPU."""
    if modeling.get_backend() is not None and hidden.is_cuda:
        return modeling.get_backend().linear_cross_entropy(weight, hidden, target, reduction)
    logits = F.linear(hidden, weight.to(hidden.dtype)).float()
    return F.cross_entropy(logits, target, ignore_index=-100, reduction=reduction)


class LossModel(torch.nn.Module):
    def __init__(self, lm, experts=None, topk=None, ce=None):
        super().__init__()
        self.lm = lm
        self.experts = experts or lm.config.num_experts
        self.topk = topk or lm.config.num_experts_per_tok
        # `ce(weight, hidden, target)` may be supplied (the reference tests pass a plain module).
        self.ce = ce
        self.last_stats = None

    def _ce(self, weight, hidden, target, reduction):
        if self.ce is not None and reduction == "mean":
            return self.ce(weight, hidden, target)
        return linear_cross_entropy(weight, hidden, target, reduction)

    def forward(self, x, y):
        m = self.lm
        stats = RouterStats(self.experts)
        blocks = m.moe_blocks()
        for block in blocks:
            block.stats_sink = stats
        try:
            hs, kls = m.model.trunk(x)
            mh = m.mtp_hidden(hs, y) if m.mtp is not None else None
        finally:
            for block in blocks:
                block.stats_sink = None
        dtype = m.model.compute_dtype or hs.dtype
        h = m.model.norm(hs, out_dtype=dtype)
        ce = self._ce(m.lm_head.weight, h.reshape(-1, h.size(-1)), y.reshape(-1), "mean")
        mtp_loss = ce.new_zeros(())
        if mh is not None:
            target = torch.cat([y[:, 1:], torch.full_like(y[:, :1], -100)], 1)
            target = target.masked_fill(y == m.config.eos_token_id, -100)
            valid = (target != -100).sum()
            mtp_loss = self._ce(m.lm_head.weight, mh.reshape(-1, mh.size(-1)), target.reshape(-1), "sum") / valid.clamp_min(1)
        kl = torch.stack(kls).mean() if kls else ce.new_zeros(())
        aux = stats.loss()
        if not torch.is_tensor(aux):
            aux = ce.new_zeros(())
        self.last_stats = stats
        return ce, aux, mtp_loss, kl
