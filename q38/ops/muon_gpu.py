"""Muon on the GPU.

`FusedMuon` is the arena path the trainer uses: the matrices a rank owns are described once by small device tables and a
step is

    muon_prepass      one pass: clip, momentum, Nesterov, bf16 cast, per-matrix sum of squares        (csrc/muon.cu)
    muon_normalize    divide by the Frobenius norm                                                    (csrc/muon.cu)
    per matrix shape  five Newton-Schulz iterations, three batched tcgen05 GEMMs each:
                          G = X X^T;   P = c G G + b G (addend epilogue);   X' = P X + a X (addend epilogue)
    muon_apply        decay + scaled update + bf16 shadow                                              (csrc/muon.cu)

The bf16 work buffer keeps every matrix in the layout of its parameter and groups matrices of one shape contiguously, so a
shape needs one batched GEMM call per product however many parameters have it.  Tall matrices (rows > cols) are never
transposed: with X = U^T the Gram matrix is ``U^T U`` (both operands MN-major) and the update is ``U P + a U``.
Stacks of tiny matrices (min(rows, cols) <= 8) run in one shared-memory kernel per shape.

`batched_step` is the stand-alone path for parameters that do not live in an arena (tests, `Muon` used directly on GPU
tensors): the same chain, with the elementwise parts as PyTorch foreach ops.  (Reference: q38/muon.py:58-104.)
"""
import numpy as np
import torch

from ..optim.muon import NS_COEFFICIENTS

TILE = 4096               # elements per CTA of the elementwise kernels (MUON_TILE in csrc/muon.cu)
SMALL_ROWS = 8            # min(rows, cols) up to which the shared-memory kernel is used


def _gemm_shape_ok(m, k):
    return m >= 16 and m % 8 == 0 and k % 8 == 0


def _ns_chain_fused(X, Y, G, P, rows, cols, steps, err):
    """Five NS iterations on the stack ``X[n, rows, cols]`` (bf16, normalised); ping-pongs between X and Y and returns the buffer
    that holds the result.  G, P: ``[n, m, m]`` scratch with m = min(rows, cols)."""
    from . import load
    ops = load()
    a, b, c = NS_COEFFICIENTS
    tall = rows > cols
    src, dst = X, Y
    for _ in range(steps):
        if tall:
            ops.gemm_bf16_persistent(src, src, G, True, True, 1.0, False, err, -1, None, 0.0)             # G = U^T U
            ops.gemm_bf16_persistent(G, G, P, False, False, c, False, err, -1, G, b)                      # P = c G G + b G
            ops.gemm_bf16_persistent(src, P, dst, False, False, 1.0, False, err, -1, src, a)              # U' = U P + a U
        else:
            ops.gemm_bf16_persistent(src, src, G, False, False, 1.0, False, err, -1, None, 0.0)           # G = X X^T
            ops.gemm_bf16_persistent(G, G, P, False, False, c, False, err, -1, G, b)
            ops.gemm_bf16_persistent(P, src, dst, False, True, 1.0, False, err, -1, src, a)               # X' = P X + a X
        src, dst = dst, src
    return src


class FusedMuon:
    """Muon over the matrices described by ``entries = [(arena_offset, n_matrices, rows, cols), ...]`` of flat fp32 arenas."""

    def __init__(self, params, grads, buf, shadow, entries, rms_scale=0.2, ns_steps=5):
        self.params, self.grads, self.buf, self.shadow = params, grads, buf, shadow
        self.ns_steps = ns_steps
        dev = params.device
        groups = {}
        for offset, n, rows, cols in entries:
            groups.setdefault((rows, cols), []).append((offset, n))
        mats, tiles, scales, self.groups = [], [], [], []
        cursor = 0
        for (rows, cols), items in groups.items():
            cursor = (cursor + 63) // 64 * 64
            size = rows * cols
            count = sum(n for _, n in items)
            self.groups.append((rows, cols, cursor, count))
            scale = rms_scale * max(rows, cols) ** 0.5
            for offset, n in items:
                for i in range(n):
                    index = len(mats)
                    mats.append((offset + i * size, cursor, size, 0))
                    scales.append(scale)
                    tiles.extend((index, first) for first in range(0, size, TILE))
                    cursor += size
        self.work_numel = max(cursor, 64)
        as_dev = lambda array, dtype: torch.from_numpy(np.asarray(array, dtype=dtype)).to(dev)
        self.mats = as_dev(mats if mats else np.zeros((0, 4)), np.int64).reshape(-1, 4)
        self.tiles = as_dev(tiles if tiles else np.zeros((0, 2)), np.int32).reshape(-1, 2)
        self.scales = as_dev(scales, np.float32)
        self.sumsq = torch.zeros(max(len(mats), 1), dtype=torch.float32, device=dev)
        self.work = torch.zeros(self.work_numel, dtype=torch.bfloat16, device=dev)
        self.work2 = torch.zeros(self.work_numel, dtype=torch.bfloat16, device=dev)
        gram = max((count * min(r, c) ** 2 for r, c, _, count in self.groups if _gemm_shape_ok(min(r, c), max(r, c))), default=0)
        self.gram = torch.zeros(max(gram, 64), dtype=torch.bfloat16, device=dev)
        self.poly = torch.zeros(max(gram, 64), dtype=torch.bfloat16, device=dev)
        self.launches_per_step = 0

    def empty(self):
        return self.mats.shape[0] == 0

    @torch.no_grad()
    def step(self, lr, momentum, weight_decay, grad_scale=None, hyper=None, err=None):
        """`hyper`: optional CUDA fp32 tensor whose element 0 is the learning rate (replayable step); `lr` is used otherwise."""
        if self.empty():
            return
        from . import load
        ops = load()
        if grad_scale is not None:
            grad_scale = grad_scale.reshape(1).float()
        ops.muon_prepass(self.grads, self.buf, self.work, self.sumsq, self.mats, self.tiles, grad_scale, float(momentum), err)
        ops.muon_normalize(self.work, self.sumsq, self.mats, self.tiles, 1e-7, err)
        final = self.work2 if self.ns_steps % 2 else self.work
        for rows, cols, base, count in self.groups:
            size = rows * cols
            X = self.work[base:base + count * size].view(count, rows, cols)
            Y = self.work2[base:base + count * size].view(count, rows, cols)
            m, k = min(rows, cols), max(rows, cols)
            if _gemm_shape_ok(m, k):
                G = self.gram[:count * m * m].view(count, m, m)
                P = self.poly[:count * m * m].view(count, m, m)
                _ns_chain_fused(X, Y, G, P, rows, cols, self.ns_steps, err)
            elif m <= SMALL_ROWS and k <= 2048:
                dst = final[base:base + count * size].view(count, rows, cols)
                ops.muon_small_ns(X, dst, rows, cols, self.ns_steps, err)
            else:                                            # odd shapes: plain batched matmuls
                a, b, c = NS_COEFFICIENTS
                Z = X.transpose(1, 2) if rows > cols else X
                for _ in range(self.ns_steps):
                    gram = Z @ Z.transpose(1, 2)
                    Z = a * Z + (b * gram + c * (gram @ gram)) @ Z
                final[base:base + count * size].view(count, rows, cols).copy_(Z.transpose(1, 2) if rows > cols else Z)
        ops.muon_apply(self.params, self.shadow, final, self.mats, self.tiles, self.scales, hyper, float(lr), float(weight_decay), err)


def _ns_chain(X, steps):
    """X: [n, m, k] bf16 with m <= k, already normalised.  Returns the orthogonalised stack (bf16)."""
    a, b, c = NS_COEFFICIENTS
    n, m, k = X.shape
    if not _gemm_shape_ok(m, k):           # tiny / unaligned matrices (conv 1x4, 4-row projections): plain bmm
        for _ in range(steps):
            G = X @ X.transpose(1, 2)
            X = a * X + (b * G + c * (G @ G)) @ X
        return X
    from . import error_flag
    err = error_flag(X.device)
    Y, G, P = torch.empty_like(X), X.new_empty(n, m, m), X.new_empty(n, m, m)
    return _ns_chain_fused(X, Y, G, P, m, k, steps, err)


@torch.no_grad()
def batched_step(views, per_call, lr, momentum, weight_decay, ns_steps, scale, grad_scale=None):
    """Stand-alone path.  views: list of (param, grad, buf) each ``[n_i, rows, cols]`` fp32 views."""
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
            pieces = list((X.float() * (lr * -scale)).split(counts))
            if weight_decay:
                torch._foreach_mul_(params, 1 - lr * weight_decay)
            torch._foreach_add_(params, pieces)
            continue
        pieces = list(X.float().split(counts))
        if weight_decay:
            torch._foreach_mul_(params, 1 - lr * weight_decay)
        torch._foreach_add_(params, pieces, alpha=-lr * scale)
