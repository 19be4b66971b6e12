"""Batched Muon step on the GPU: all matrices of one shape go through one Newton-Schulz chain.

Per call: stack up to `per_call` matrices, fused momentum/Nesterov/normalise, five NS iterations as batched
tensor-core GEMMs (``X X^T``, ``G G``, ``P X``: all three are plain ``A . B^T`` products because the Gram matrix and
the polynomial are symmetric), then decay + scaled update.  (Reference: q38/muon.py:58-104.)
"""
import torch

from ..optim.muon import NS_COEFFICIENTS


def _ns_chain(X, steps):
    """X: [n, m, k] bf16 with m <= k, already normalised.  Returns the orthogonalised stack (bf16)."""
    from . import gemm
    a, b, c = NS_COEFFICIENTS
    n, m, k = X.shape
    small = m < 16 or k % 8 or m % 8       # tiny / unaligned matrices (conv 1x4, routers of odd width): plain bmm
    for _ in range(steps):
        if small:
            G = X @ X.transpose(1, 2)
            X = a * X + (b * G + c * (G @ G)) @ X
            continue
        G = gemm(X, X)                                     # [n,m,m] = X X^T            (K-major x K-major)
        G2 = gemm(G, G)                                    # G symmetric: G G^T = G G
        P = (b * G + c * G2)
        PX = gemm(P, X, b_mn_major=True)                   # [n,m,k] = P X              (B stored [K=m, N=k])
        X = a * X + PX
    return X


@torch.no_grad()
def batched_step(views, per_call, lr, momentum, weight_decay, ns_steps, scale, grad_scale=None):
    """views: list of (param, grad, buf) each ``[n_i, rows, cols]`` fp32 views."""
    chunks, current, used = [], [], 0
    for p, g, buf in views:
        for ps, gs, bs in zip(p.split(per_call), g.split(per_call), buf.split(per_call)):
            if current and used + ps.shape[0] > per_call:
                chunks.append(current)
                current, used = [], 0
            current.append((ps, gs, bs))
            used += ps.shape[0]
    if current:
        chunks.append(current)
    for chunk in chunks:
        params, grads, bufs = map(list, zip(*chunk))
        if grad_scale is not None:
            grads = torch._foreach_mul(grads, grad_scale)
        torch._foreach_mul_(bufs, momentum)
        torch._foreach_add_(bufs, grads)
        updates = torch._foreach_add(grads, bufs, alpha=momentum)
        counts = [u.shape[0] for u in updates]
        U = torch.cat(updates) if len(updates) > 1 else updates[0]
        rows, cols = U.shape[-2:]
        X = U.to(torch.bfloat16)
        if rows > cols:
            X = X.transpose(1, 2).contiguous()
        X = X / X.flatten(1).norm(dim=-1).clamp_min(1e-7)[:, None, None]
        X = _ns_chain(X.contiguous(), ns_steps)
        if rows > cols:
            X = X.transpose(1, 2)
        if torch.is_tensor(lr):
            # learning rate in device memory: the whole step can be captured once and replayed with a new value
            pieces = list((X.float() * (lr * -scale)).split(counts))
            if weight_decay:
                torch._foreach_mul_(params, 1 - lr * weight_decay)
            torch._foreach_add_(params, pieces)
            continue
        pieces = list(X.float().split(counts))
        if weight_decay:
            torch._foreach_mul_(params, 1 - lr * weight_decay)
        torch._foreach_add_(params, pieces, alpha=-lr * scale)
