"""Muon: Nesterov momentum followed by Newton-Schulz orthogonalisation of every matrix update.

Update of one matrix ``W[rows, cols]`` with gradient ``g`` (reference: q38/muon.py:12-25, 106-119):

    buf <- 0.95 buf + g;  u <- g + 0.95 buf
    X <- bf16(u) (transposed when rows > cols) / max(||u||_F, 1e-7)
    5 x { G = X X^T;  P = b G + c G G;  X <- a X + P X }      (a, b, c) = (3.4445, -4.7750, 2.0315), in bf16
    W <- W (1 - lr wd) - lr * 0.2 sqrt(max(rows, cols)) * X

Tensors with more than two dimensions are treated as stacks of matrices over the trailing two
dimensions (MoE experts ``[E, a, b]``; the depthwise conv weight ``[C, 1, 4]`` is C matrices of 1 x 4).

On a GPU the step is batched: all matrices of one shape are processed by one fused pre-pass
(momentum, Nesterov, Frobenius norm, bf16 cast), one batched Newton-Schulz chain on the tensor cores
and one fused apply kernel (`q38.ops`).  On CPU the per-parameter PyTorch path below is used; it is
also the oracle of the GPU tests.  ``owned`` restricts the step to a subset of (parameter, slice)
units, which is how the sharded data-parallel engine makes every rank update only the matrices it owns.
"""
import os

import torch

NS_COEFFICIENTS = (3.4445, -4.7750, 2.0315)
MAX_BATCH_ELEMENTS = 64 * 1024 * 1024      # bound on the temporaries of one batched Newton-Schulz call
MUON_MAX_CHUNK_ELEMENTS = MAX_BATCH_ELEMENTS  # the reference's name for the same bound (q38/muon.py:9)


@torch.no_grad()
def newton_schulz(G, steps=5, eps=1e-7):
    """Approximately orthogonalise ``G[..., rows, cols]`` (singular values -> about 1); computed in bf16."""
    a, b, c = NS_COEFFICIENTS
    X = G.to(torch.bfloat16)
    wide = X.size(-2) <= X.size(-1)
    if not wide:
        X = X.transpose(-2, -1)
    X = X / X.flatten(-2).norm(dim=-1).clamp(min=eps)[..., None, None]
    for _ in range(steps):
        gram = X @ X.transpose(-2, -1)
        X = a * X + (b * gram + c * (gram @ gram)) @ X
    return X if wide else X.transpose(-2, -1)


def update_scale(shape, rms_scale):
    return rms_scale * max(shape[-2], shape[-1]) ** 0.5


class Muon(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, momentum=0.95, weight_decay=0.1, ns_steps=5, rms_scale=0.2):
        super().__init__(params, dict(lr=lr, momentum=momentum, weight_decay=weight_decay, ns_steps=ns_steps,
                                      rms_scale=rms_scale))

    def _buffer(self, p):
        state = self.state[p]
        if "buf" not in state:
            state["buf"] = torch.zeros_like(p)
        return state["buf"]

    @torch.no_grad()
    def step(self, closure=None, params=None, grad_scale=None, slices=None, lr_tensor=None):
        """`params`: optional subset (the units this rank owns).  `grad_scale`: optional scalar tensor the
        gradients are multiplied with before use (the clip coefficient), without modifying `.grad`.
        `slices`: ``{id(param): slice}`` restricts a stacked parameter (experts ``[E, a, b]``) to a range of its matrices.
        `lr_tensor`: optional 0-dim CUDA tensor used instead of the groups' learning rate (CUDA-graph replay)."""
        keep = None if params is None else {id(p) for p in params}
        slices = slices or {}
        on_gpu = any(p.is_cuda for g in self.param_groups for p in g["params"])
        if not on_gpu or os.environ.get("Q38_MUON_BASELINE"):
            return self._reference_step(keep, grad_scale, slices)
        from ..ops import muon_batched_step
        for group in self.param_groups:
            by_shape = {}
            for p in group["params"]:
                if p.grad is not None and (keep is None or id(p) in keep):
                    by_shape.setdefault((p.device, p.dtype, tuple(p.shape[-2:])), []).append(p)
            for (_, _, (rows, cols)), plist in by_shape.items():
                per_call = max(1, MAX_BATCH_ELEMENTS // (rows * cols))
                views = []
                for p in plist:
                    buf = self._buffer(p)
                    sl = slices.get(id(p), slice(None))
                    views.append((p.view(-1, rows, cols)[sl], p.grad.view(-1, rows, cols)[sl], buf.view(-1, rows, cols)[sl]))
                muon_batched_step(views, per_call, lr=group["lr"] if lr_tensor is None else lr_tensor, momentum=group["momentum"],
                                  weight_decay=group["weight_decay"], ns_steps=group["ns_steps"],
                                  scale=update_scale((rows, cols), group["rms_scale"]), grad_scale=grad_scale)

    @torch.no_grad()
    def _reference_step(self, keep=None, grad_scale=None, slices=None):
        slices = slices or {}
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None or (keep is not None and id(p) not in keep):
                    continue
                sl = slices.get(id(p))
                target, grad, buf = p, p.grad, self._buffer(p)
                if sl is not None:
                    target, grad, buf = p[sl], grad[sl], buf[sl]
                if grad_scale is not None:
                    grad = grad * grad_scale
                buf.mul_(group["momentum"]).add_(grad)
                update = grad.add(buf, alpha=group["momentum"])
                ortho = newton_schulz(update, group["ns_steps"]).float()
                if group["weight_decay"]:
                    target.mul_(1 - group["lr"] * group["weight_decay"])
                target.add_(ortho, alpha=-group["lr"] * update_scale(p.shape, group["rms_scale"]))
