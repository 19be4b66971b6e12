"""Kernel backend: the object the model file calls for every hot op when tensors live on a GPU.

Each method is a `torch.autograd.Function` (or a composition of them) over the CUDA kernels of `csrc/`.
A method that is absent makes the model use its PyTorch specification for that op; the set of present
methods is reported by `describe()` so a run records exactly which paths were native.
"""
import collections
import os

import torch

from . import error_flag, gemm, load


def _bf16_weight(weight):
    """bf16 copy of an fp32 master weight: the arena's shadow view when the trainer manages the parameter,
    otherwise a cached cast keyed on the tensor's version counter."""
    shadow = getattr(weight, "_q38_bf16", None)
    if shadow is not None:
        return shadow
    if weight.dtype == torch.bfloat16:
        return weight.detach()
    cached = getattr(weight, "_q38_cast", None)
    if cached is None or cached[0] != weight._version or cached[1].device != weight.device:
        cached = (weight._version, weight.detach().to(torch.bfloat16))
        weight._q38_cast = cached
    return cached[1]


class _Linear(torch.autograd.Function):
    """y = x W^T with bf16 operands; dgrad and wgrad run on the same tensor-core kernel with MN-major operands."""

    @staticmethod
    def forward(ctx, x, weight, backend):
        w = _bf16_weight(weight)
        x2 = x.reshape(-1, x.shape[-1])
        if x2.dtype != torch.bfloat16:
            x2 = x2.to(torch.bfloat16)
        x2 = x2.contiguous()
        y = backend.mm_nt(x2, w)
        ctx.save_for_backward(x2, weight)
        ctx.backend, ctx.in_shape, ctx.in_dtype = backend, x.shape, x.dtype
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        backend = ctx.backend
        dy2 = dy.reshape(-1, dy.shape[-1]).to(torch.bfloat16).contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = backend.mm_nn(dy2, _bf16_weight(weight)).view(ctx.in_shape).to(ctx.in_dtype)
        if ctx.needs_input_grad[1]:
            dw = backend.weight_grad(dy2, x2, weight)
        return dx, dw, None


class _MultiLinear(torch.autograd.Function):
    """Several projections of one input: ``y_i = x W_i^T``.  The point is the backward pass: the input gradient
    ``dx = sum_i dy_i W_i`` is built by a chain of GEMMs whose epilogue adds the running sum (addend with beta = 1), so autograd
    never launches elementwise additions of ``[tokens, hidden]`` tensors for an activation that feeds several projections."""

    @staticmethod
    def forward(ctx, x, backend, *weights):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.dtype != torch.bfloat16:
            x2 = x2.to(torch.bfloat16)
        x2 = x2.contiguous()
        outs = tuple(backend.mm_nt(x2, _bf16_weight(w)).view(*x.shape[:-1], w.shape[0]) for w in weights)
        ctx.save_for_backward(x2, *weights)
        ctx.backend, ctx.in_shape, ctx.in_dtype = backend, x.shape, x.dtype
        return outs

    @staticmethod
    def backward(ctx, *dys):
        x2, *weights = ctx.saved_tensors
        backend = ctx.backend
        dx = None
        dws = []
        for i, (dy, weight) in enumerate(zip(dys, weights)):
            if dy is None:
                dws.append(None)
                continue
            dy2 = dy.reshape(-1, dy.shape[-1]).to(torch.bfloat16).contiguous()
            if ctx.needs_input_grad[0]:
                w = _bf16_weight(weight)
                if dx is None:
                    dx = backend.mm_nn(dy2, w)
                elif w.shape[1] % 8 == 0 and backend.layouts["nn"] and os.environ.get("Q38_MULTI_LINEAR", "2") == "2":
                    gemm(_tma_rows(dy2), w, out=dx, b_mn_major=True, accumulate=True)          # dx += dy_i W_i: the TMA unit adds the tile
                elif w.shape[1] % 8 == 0 and backend.layouts["nn"]:
                    dx = gemm(_tma_rows(dy2), w, b_mn_major=True, addend=dx, beta=1.0)        # dx <- dy_i W_i + dx, one kernel
                else:
                    dx = dx + backend.mm_nn(dy2, w)
            dws.append(backend.weight_grad(dy2, x2, weight) if ctx.needs_input_grad[2 + i] else None)
        if dx is not None:
            dx = dx.view(ctx.in_shape).to(ctx.in_dtype)
        return (dx, None, *dws)


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps, out_dtype):
        ops = load()
        xc = x.contiguous()
        y, rstd = ops.rmsnorm_fwd(xc, weight.float().contiguous(), eps, out_dtype == torch.bfloat16)
        ctx.save_for_backward(xc, weight, rstd)
        return y if y.dtype == out_dtype else y.to(out_dtype)

    @staticmethod
    def backward(ctx, dy):
        x, weight, rstd = ctx.saved_tensors
        dyc = dy.contiguous()
        if dyc.dtype not in (torch.float32, torch.bfloat16):
            dyc = dyc.float()
        dx, dw = load().rmsnorm_bwd(dyc, x, weight.float().contiguous(), rstd)
        return dx, DEFERRED_GRADS.take(weight, dw), None, None


class _GatedRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate, weight, eps):
        xc, gc = x.contiguous(), gate.contiguous()
        ctx.save_for_backward(xc, gc, weight)
        ctx.eps = eps
        return load().gated_rmsnorm_fwd(xc, gc, weight.float().contiguous(), eps)

    @staticmethod
    def backward(ctx, dy):
        x, gate, weight = ctx.saved_tensors
        dx, dgate, dw = load().gated_rmsnorm_bwd(dy.contiguous(), x, gate, weight.float().contiguous(), ctx.eps)
        return dx, dgate, DEFERRED_GRADS.take(weight, dw), None


class _SideStream:
    """Weight gradients have no consumer until the optimizer step, so the trainer lets them run on a second stream where they
    fill the SMs that the latency-bound kernels of the backward chain (delta-rule scan, block attention) leave idle.

    `run(fn, *tensors)` makes the side stream wait for the work issued so far, runs `fn` there and tells the caching allocator
    that `tensors` are in use on that stream.  `join()` makes the current stream wait for everything issued on the side
    stream; the owner calls it after every backward pass (inside a CUDA-graph capture this is also what joins the forked
    branch back).  Disabled (fn runs inline) unless `enabled` is set."""

    def __init__(self):
        self.enabled = False
        self.stream = None
        self.pending = False

    def run(self, fn, *tensors):
        if not self.enabled:
            return fn()
        cur = torch.cuda.current_stream()
        if self.stream is None:
            self.stream = torch.cuda.Stream()
        self.stream.wait_stream(cur)
        with torch.cuda.stream(self.stream):
            out = fn()
        for t in tensors:
            t.record_stream(self.stream)
        self.pending = True
        return out

    def join(self):
        if self.pending:
            torch.cuda.current_stream().wait_stream(self.stream)
            self.pending = False


WGRAD_STREAM = _SideStream()


class _DeferredGrads:
    """Gradients of the small parameters (norm weights, conv taps, gate vectors, the mHC biases) collected during a backward pass
    and added into the parameters' gradient buffers by one multi-tensor launch at its end, instead of one `AccumulateGrad`
    addition kernel per parameter and micro-step (about 190 launches for q38_c2).  A backward that defers returns None for that
    parameter.  Only the trainer enables it (Q38_DEFER_SMALL_GRADS=0 keeps it off), because whoever runs the backward must call
    `flush()` afterwards (the trainer does so where it joins the weight-gradient stream); with `enabled` False every gradient
    is returned to autograd as usual."""

    def __init__(self):
        self.enabled = False
        self.targets, self.deltas = [], []

    def take(self, param, delta):
        """Queue `param.grad += delta` and return None, or return `delta` in the parameter's dtype when deferral does not apply."""
        grad = param.grad
        if not self.enabled or grad is None or grad.dtype != torch.float32 or delta.dtype != torch.float32 or not grad.is_contiguous():
            return delta.reshape(param.shape).to(param.dtype)
        self.targets.append(grad)
        self.deltas.append(delta.reshape(grad.shape))
        return None

    def flush(self):
        if self.targets:
            torch._foreach_add_(self.targets, self.deltas)
            self.targets, self.deltas = [], []


DEFERRED_GRADS = _DeferredGrads()


# Every product that leaves the hand-written GEMM for a library matmul is counted here by call site (shapes the tensor-core
# kernel does not take: a reduction dimension that is not a multiple of 8, a layout that failed its start-up self-check, the
# Q38_MHC_FP32_GEMM switch).  `Backend.describe()` reports the counter, and the benchmark prints it: empty means every product
# of the run went through the sm_100a kernels.
LIBRARY_FALLBACKS = collections.Counter()


def _fallback(site):
    LIBRARY_FALLBACKS[site] += 1


def _tma_rows(t):
    """A 2-D tensor whose row stride TMA accepts (a multiple of 16 bytes).  A narrow matrix, e.g. the [tokens, 21] gradient of a
    per-head gate projection, is copied into a buffer with padded rows and returned as a view of it; the tensor map still
    describes the true width, so the padding is never read."""
    n, per16 = t.shape[1], 16 // t.element_size()
    if n % per16 == 0 and t.is_contiguous():
        return t
    buf = torch.empty(t.shape[0], (n + per16 - 1) // per16 * per16, dtype=t.dtype, device=t.device)
    view = buf[:, :n]
    view.copy_(t)
    return view


def _mm32(a, b, layout, out_dtype=torch.float32):
    """Products of fp32 operands for the mHC low-rank path on the tensor cores.

    'nt' a[M,K] b[N,K]^T and 'nn' a[M,K] b[K,N] run as tf32 (fp32 data read by TMA, 10-bit mantissa math, fp32 accumulate);
    'nn' transposes the small operand so both are K-major.  'tn' a[K,M]^T b[K,N] (a weight gradient that reduces over the
    tokens) runs on bf16 copies with MN-major operands and fp32 accumulation."""
    a, b = a.float().contiguous(), b.float().contiguous()
    if os.environ.get("Q38_MHC_FP32_GEMM"):
        _fallback("mhc_fp32_switch")
        return a @ b.t() if layout == "nt" else (a @ b if layout == "nn" else a.t() @ b)
    if layout == "tn":
        if a.shape[1] % 8 or b.shape[1] % 8:
            _fallback("mhc_tn_unaligned")
            return a.t() @ b
        return gemm(a.to(torch.bfloat16), b.to(torch.bfloat16), a_mn_major=True, b_mn_major=True, out_dtype=torch.float32)
    if layout == "nn":
        b = b.t().contiguous()
    if a.shape[1] % 4 or a.data_ptr() % 16 or b.data_ptr() % 16:
        _fallback("mhc_tf32_unaligned")
        return (a @ b.t()).to(out_dtype)
    return gemm(a, b, out_dtype=out_dtype)


def _mhc_weight_grad(dL, Xf, A_w):
    """dA = dL^T Xf (reduction over tokens): bf16 operands, MN-major, split-K accumulated into A's gradient buffer."""
    grad = A_w.grad
    if (grad is not None and grad.dtype == torch.float32 and grad.is_contiguous() and dL.shape[1] % 8 == 0 and Xf.shape[1] % 8 == 0
            and not os.environ.get("Q38_MHC_FP32_GEMM")):
        a, b = dL.to(torch.bfloat16), Xf.to(torch.bfloat16)
        WGRAD_STREAM.run(lambda: gemm(a, b, out=grad, a_mn_major=True, b_mn_major=True, accumulate=True,
                                      splits=-1 if os.environ.get("Q38_DETERMINISTIC") == "1" else 0), a, b)
        return None
    return _mm32(dL, Xf, 'tn').to(A_w.dtype)


class _MhcLink:
    """Carries the gradient of a sub-layer's output stream from `_MhcPost.backward` to `_MhcPreNorm.backward`, which
    writes the complete gradient of the input stream in one pass (the residual-mix term is folded in there)."""
    __slots__ = ("dXo",)

    def __init__(self):
        self.dXo = None


class _MhcPreNorm(torch.autograd.Function):
    """(X, mHC parameters, norm weight) -> (normalised sub-layer input, coefficient rows)."""

    @staticmethod
    def forward(ctx, X, A_w, B_w, b_pre, b_post, b_res, alphas, norm_w, iters, eps, out_dtype, link):
        ops = load()
        B_, S, n, h = X.shape
        Xc = X.contiguous()
        Xf = Xc.view(B_ * S, n * h)
        Lraw = _mm32(Xf, A_w, 'nt')                           # low-rank projection: fp32 data, tf32 tensor-core math
        xout, coef, z, inv, rstd = ops.mhc_coef_fwd(Xc.view(B_ * S, n, h), Lraw, B_w.float().contiguous(), b_pre.float().contiguous(),
                                                    b_post.float().contiguous(), b_res.float().contiguous(), alphas.float().contiguous(),
                                                    norm_w.float().contiguous(), iters, eps, out_dtype == torch.bfloat16)
        ctx.save_for_backward(Xc, Lraw, coef, z, inv, rstd, A_w, B_w, b_pre, b_post, b_res, alphas, norm_w)
        ctx.iters, ctx.link, ctx.shape = iters, link, X.shape
        ctx.mark_non_differentiable(z)
        return xout.view(B_, S, h), coef

    @staticmethod
    def backward(ctx, dxout, dcoef):
        ops = load()
        Xc, Lraw, coef, z, inv, rstd, A_w, B_w, b_pre, b_post, b_res, alphas, norm_w = ctx.saved_tensors
        B_, S, n, h = ctx.shape
        T = B_ * S
        if dcoef is None:
            dcoef = torch.zeros_like(coef)
        dcoef = dcoef.contiguous()
        dLraw, c1, dxin, dBw, dbias, dnw, Xbf = ops.mhc_pre_bwd_a(
            dxout.reshape(T, h).contiguous(), Xc.view(T, n, h), Lraw, B_w.float().contiguous(), b_pre.float().contiguous(),
            b_post.float().contiguous(), b_res.float().contiguous(), alphas.float().contiguous(), norm_w.float().contiguous(),
            coef, z, inv, rstd, dcoef, ctx.iters)
        Xf = Xc.view(T, n * h)
        dA = _mhc_weight_grad(dLraw, Xf if os.environ.get("Q38_MHC_FP32_GEMM") else Xbf, A_w)
        # G = dL_raw A: the low-rank correction of the stream gradient, kept in bf16 between the GEMM and the combine kernel
        # (fp32 with Q38_MHC_FP32_GEMM); every other term of dX is fp32
        G = _mm32(dLraw, A_w, 'nn', torch.float32 if os.environ.get("Q38_MHC_FP32_GEMM") else torch.bfloat16)
        dXo = ctx.link.dXo if ctx.link.dXo is not None else torch.zeros_like(Xf)
        ctx.link.dXo = None
        dX = ops.mhc_pre_bwd_c(G.view(T, n, h), dXo.contiguous().view(T, n, h), Xc.view(T, n, h), dxin, coef, c1)
        take = DEFERRED_GRADS.take
        return (dX.view(B_, S, n, h), dA, take(B_w, dBw), take(b_pre, dbias[0:4]), take(b_post, dbias[4:8]), take(b_res, dbias[8:24]),
                take(alphas, dbias[24:27]), take(norm_w, dnw), None, None, None, None)


class _MhcPost(torch.autograd.Function):
    """X'_m = sum_n res[m,n] X_n + post_m y.  The gradient w.r.t. X is delivered through `link` (see `_MhcLink`)."""

    @staticmethod
    def forward(ctx, X, y, coef, link):
        B_, S, n, h = X.shape
        Xc, yc = X.contiguous(), y.contiguous()
        out = load().mhc_post_fwd(Xc.view(B_ * S, n, h), yc.view(B_ * S, h), coef)
        ctx.save_for_backward(Xc, yc, coef)
        ctx.link, ctx.shape = link, X.shape
        return out.view(B_, S, n, h)

    @staticmethod
    def backward(ctx, dXo):
        Xc, yc, coef = ctx.saved_tensors
        B_, S, n, h = ctx.shape
        dXo = dXo.contiguous()
        dy, dcoef = load().mhc_post_bwd(dXo.view(B_ * S, n, h), Xc.view(B_ * S, n, h), yc.view(B_ * S, h), coef)
        ctx.link.dXo = dXo
        return None, dy.view(B_, S, h), dcoef, None


class _ConvSilu(torch.autograd.Function):
    """Depthwise causal conv (kernel 4) + SiLU on [B,S,C] bf16; weight is the fp32 master [C,1,4]."""

    @staticmethod
    def forward(ctx, x, weight):
        xc = x.contiguous()
        w = weight.float().reshape(weight.shape[0], -1).contiguous()
        ctx.save_for_backward(xc, weight)
        return load().conv_silu_fwd(xc, w)

    @staticmethod
    def backward(ctx, dy):
        xc, weight = ctx.saved_tensors
        dx, dw = load().conv_silu_bwd(xc, weight.float().reshape(weight.shape[0], -1).contiguous(), dy.contiguous())
        return dx, DEFERRED_GRADS.take(weight, dw)


class _GdnScan(torch.autograd.Function):
    """Sequential pass of the chunked delta rule over prepared chunk operands (see csrc/gdn.cu)."""

    @staticmethod
    def forward(ctx, w, u, P, qg, kg, carry, B, H):
        w, u, P, qg, kg = (t.to(torch.bfloat16).contiguous() for t in (w, u, P, qg, kg))
        carry = carry.float().contiguous()
        o, vnew, states = load().gdn_scan_fwd(w, u, P, qg, kg, carry, B, H)
        ctx.save_for_backward(w, P, qg, kg, carry, vnew, states)
        ctx.dims = (B, H)
        return o

    @staticmethod
    def backward(ctx, do):
        w, P, qg, kg, carry, vnew, states = ctx.saved_tensors
        B, H = ctx.dims
        dw, du, dP, dqg, dkg, dd = load().gdn_scan_bwd(w, P, qg, kg, carry, vnew, states, do.to(torch.bfloat16).contiguous(), B, H)
        shape = w.shape
        return dw.view(shape), du.view(shape), dP.view(shape), dqg.view(shape), dkg.view(shape), dd.view(carry.shape), None, None


class _DeltaRule(torch.autograd.Function):
    """Chunked gated delta rule on a packed ``qkv [B,S,(2 Hk + Hv) 64]`` tensor (q | k | v per token, as the causal conv
    produces it): per-chunk preparation kernel (parallel over chunks) + sequential scan kernel.  The kernels read the
    three parts through strided views and write their gradients into one packed tensor, so no split/concat copies run."""

    @staticmethod
    def forward(ctx, qkv, g, beta, Hk, Hv):
        ops = load()
        qkv = qkv.contiguous()
        B, S, _ = qkv.shape
        q = qkv[..., :Hk * 64].unflatten(-1, (Hk, 64))
        k = qkv[..., Hk * 64:2 * Hk * 64].unflatten(-1, (Hk, 64))
        v = qkv[..., 2 * Hk * 64:].unflatten(-1, (Hv, 64))
        g, beta = g.float().contiguous(), beta.to(torch.bfloat16).contiguous()
        w, u, P, qg, kg, Tm, carry, _gc = ops.gdn_prep_fwd(q, k, v, g, beta)
        o, vnew, states = ops.gdn_scan_fwd(w, u, P, qg, kg, carry, B, Hv)
        ctx.save_for_backward(qkv, g, beta, Tm, w, P, qg, kg, carry, vnew, states)
        ctx.heads = (Hk, Hv)
        return o

    @staticmethod
    def backward(ctx, do):
        ops = load()
        qkv, g, beta, Tm, w, P, qg, kg, carry, vnew, states = ctx.saved_tensors
        Hk, Hv = ctx.heads
        B = qkv.shape[0]
        q = qkv[..., :Hk * 64].unflatten(-1, (Hk, 64))
        k = qkv[..., Hk * 64:2 * Hk * 64].unflatten(-1, (Hk, 64))
        v = qkv[..., 2 * Hk * 64:].unflatten(-1, (Hv, 64))
        dw, du, dP, dqg, dkg, dd = ops.gdn_scan_bwd(w, P, qg, kg, carry, vnew, states, do.to(torch.bfloat16).contiguous(), B, Hv)
        dqkv, dg, dbeta = ops.gdn_prep_bwd(q, k, v, g, beta, Tm, dw, du, dP, dqg, dkg, dd)
        return dqkv, dg, dbeta, None, None


class _IndexerKL(torch.autograd.Function):
    """Indexer distillation: KL between the dense main attention's block mass (target, no gradient) and the indexer's
    block distribution.  Returns (kl, lp_blk); only the indexer operands receive gradients."""

    @staticmethod
    def forward(ctx, qi, ki, wi, q_main, k_main, main_scale, idx_scale):
        ops = load()
        if q_main.shape[2] % 128 == 0 and q_main.is_contiguous() and k_main.is_contiguous() and os.environ.get("Q38_QSA_TC", "1") != "0":
            stats = ops.qsa_block_stats_tc(q_main, k_main, main_scale, error_flag(q_main.device))      # tcgen05 kernel (csrc/qsa_tc.cu)
        else:
            stats = ops.qsa_main_block_stats(q_main, k_main, main_scale)
        blse = ops.qsa_indexer_fwd(qi, ki, wi, idx_scale)
        P, lp_blk, kl_tok, dblse = ops.qsa_kl_combine(stats, blse, q_main.shape[1])
        ctx.save_for_backward(qi, ki, wi, blse, dblse)
        ctx.idx_scale = idx_scale
        ctx.mark_non_differentiable(lp_blk)
        return kl_tok.mean(), lp_blk

    @staticmethod
    def backward(ctx, dkl, _lp):
        qi, ki, wi, blse, dblse = ctx.saved_tensors
        tokens = qi.shape[0] * qi.shape[2]
        dqi, dki, dwi = load().qsa_indexer_bwd(qi, ki, wi, blse, dblse, 1.0 / tokens, ctx.idx_scale)
        return dqi * dkl.to(dqi.dtype), dki * dkl.to(dki.dtype), dwi * dkl, None, None, None, None


class _Embed(torch.autograd.Function):
    """Row gather; the backward adds the rows into the table's fp32 gradient buffer in place (atomics) when it exists."""

    @staticmethod
    def forward(ctx, weight, ids):
        ctx.save_for_backward(weight, ids)
        return torch.nn.functional.embedding(ids, weight)

    @staticmethod
    def backward(ctx, dout):
        weight, ids = ctx.saved_tensors
        in_place = weight.grad is not None and weight.grad.dtype == torch.float32 and weight.grad.is_contiguous()
        grad = weight.grad if in_place else torch.zeros_like(weight, dtype=torch.float32)
        load().embed_bwd(ids.long().contiguous(), dout.float().contiguous(), grad)
        return (None if in_place else grad.to(weight.dtype)), None


class _GdnGates(torch.autograd.Function):
    """(b, a) projections [.., Hv] bf16 -> beta = sigmoid(b) (bf16), g = -exp(A_log) softplus(a + dt_bias) (fp32), one kernel each way."""

    @staticmethod
    def forward(ctx, b_raw, a_raw, A_log, dt_bias):
        b_raw, a_raw = b_raw.contiguous(), a_raw.contiguous()
        beta, g = load().gdn_gates_fwd(b_raw, a_raw, A_log.float().contiguous(), dt_bias.float().contiguous())
        ctx.save_for_backward(b_raw, a_raw, A_log, dt_bias)
        return beta, g

    @staticmethod
    def backward(ctx, dbeta, dg):
        b_raw, a_raw, A_log, dt_bias = ctx.saved_tensors
        dbeta = torch.zeros_like(b_raw) if dbeta is None else dbeta.to(torch.bfloat16).contiguous()
        dg = torch.zeros(b_raw.shape, dtype=torch.float32, device=b_raw.device) if dg is None else dg.float().contiguous()
        db, da, dA, dbias = load().gdn_gates_bwd(dbeta, dg, b_raw, a_raw, A_log.float().contiguous(), dt_bias.float().contiguous())
        return db, da, DEFERRED_GRADS.take(A_log, dA), DEFERRED_GRADS.take(dt_bias, dbias)


class _SwiGLU(torch.autograd.Function):
    """silu(g) * u on bf16 tensors, one kernel each way."""

    @staticmethod
    def forward(ctx, g, u):
        g, u = g.contiguous(), u.contiguous()
        ctx.save_for_backward(g, u)
        return load().swiglu_fwd(g, u)

    @staticmethod
    def backward(ctx, dy):
        g, u = ctx.saved_tensors
        dg, du = load().swiglu_bwd(dy.contiguous(), g, u)
        return dg, du


class _SigmoidMul(torch.autograd.Function):
    """x * sigmoid(g) on bf16 tensors of equal shape (the output gate of the attention layer), one kernel each way."""

    @staticmethod
    def forward(ctx, x, g):
        x, g = x.contiguous(), g.contiguous()
        ctx.save_for_backward(x, g)
        return load().sigmoid_mul_fwd(x, g)

    @staticmethod
    def backward(ctx, dy):
        x, g = ctx.saved_tensors
        dx, dg = load().sigmoid_mul_bwd(dy.contiguous(), x, g)
        return dx, dg


class _GateAdd(torch.autograd.Function):
    """routed + sigmoid(logit) * shared for [T,h] bf16 rows and one logit per row (the shared-expert merge of the MoE block)."""

    @staticmethod
    def forward(ctx, routed, shared, logit):
        shared, logit = shared.contiguous(), logit.contiguous()
        ctx.save_for_backward(shared, logit)
        return load().gate_add_fwd(routed.contiguous(), shared, logit)

    @staticmethod
    def backward(ctx, dy):
        shared, logit = ctx.saved_tensors
        dy = dy.contiguous()
        dshared, dlogit = load().gate_add_bwd(dy, shared, logit)
        return dy, dshared, dlogit


class _HeadPrep(torch.autograd.Function):
    """Projection output [B,S,H,64] (or [B,S,H,128] = q | gate per head) -> (heads [B,H,S,64] after the optional per-head
    zero-centred RMSNorm and the partial rotary embedding, gate [B,S,H*64] or None), one kernel each way (csrc/qsa_prep.cu)."""

    @staticmethod
    def forward(ctx, src, weight, cos, sin, eps):
        src = src.contiguous()
        split = src.shape[-1] == 128
        w = None if weight is None else weight.float().contiguous()
        cos, sin = cos.float().contiguous(), sin.float().contiguous()
        out, gate, rstd = load().qsa_headprep_fwd(src, w, cos, sin, eps, split)
        ctx.save_for_backward(src, cos, sin, rstd, *(() if weight is None else (weight,)))
        ctx.split, ctx.has_w = split, weight is not None
        if split:
            return out, gate
        ctx.mark_non_differentiable(gate)
        return out, gate

    @staticmethod
    def backward(ctx, dout, dgate):
        src, cos, sin, rstd, *rest = ctx.saved_tensors
        weight = rest[0] if ctx.has_w else None
        w = None if weight is None else weight.float().contiguous()
        if dout is None:
            dout = torch.zeros(src.shape[0], src.shape[2], src.shape[1], 64, dtype=torch.bfloat16, device=src.device)
        if ctx.split and dgate is None:
            dgate = torch.zeros(src.shape[0], src.shape[1], src.shape[2] * 64, dtype=torch.bfloat16, device=src.device)
        dsrc, dw = load().qsa_headprep_bwd(dout.to(torch.bfloat16).contiguous(), dgate.to(torch.bfloat16).contiguous() if ctx.split else None,
                                           src, w, cos, sin, rstd)
        return dsrc, (None if weight is None else DEFERRED_GRADS.take(weight, dw)), None, None, None


def _head_prep(src, norm, cos, sin):
    """`src` [B,S,H,64|128] bf16; `norm` a zero-centred RMSNorm module or None.  Returns (heads, gate-or-None)."""
    weight, eps = (None, 0.0) if norm is None else (norm.weight, float(norm.eps))
    out, gate = _HeadPrep.apply(src, weight, cos, sin, eps)
    return out, (gate if src.shape[-1] == 128 else None)


class _BlockAttention(torch.autograd.Function):
    """GQA attention over the selected 64-token key blocks (or all causal blocks when `count` is None).
    q [B,nq,S,64], k/v [B,nkv,S,64] -> o [B,S,nq,64]."""

    @staticmethod
    def forward(ctx, q, k, v, count, index, scale):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        o, lse, sel = load().qsa_attn_fwd(q, k, v, count, index, scale)
        ctx.save_for_backward(q, k, v, o, lse, sel)
        ctx.scale = scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, sel = ctx.saved_tensors
        dq, dk, dv = load().qsa_attn_bwd(q, k, v, o, do.to(torch.bfloat16).contiguous(), lse, sel, ctx.scale)
        return dq, dk, dv, None, None, None


class _NGramEmbed(torch.autograd.Function):
    """ids -> rmsnorm(emb2[i2] + emb3[i3]) (bf16).  The backward adds the table gradients straight into the parameters' fp32
    gradient buffers with atomics (so the last bits depend on the order) and returns only d(norm weight) to autograd."""

    @staticmethod
    def forward(ctx, ids, emb2, emb3, norm_w, vocab, eos, eps):
        e, rstd, rows = load().ngram_fwd(ids.long().contiguous(), emb2, emb3, norm_w.float().contiguous(), vocab, eos, eps)
        ctx.save_for_backward(rows, rstd, emb2, emb3, norm_w)
        return e

    @staticmethod
    def backward(ctx, de):
        rows, rstd, emb2, emb3, norm_w = ctx.saved_tensors
        in_place = all(p.grad is not None and p.grad.dtype == torch.float32 and p.grad.is_contiguous() for p in (emb2, emb3))
        g2 = emb2.grad if in_place else torch.zeros_like(emb2)
        g3 = emb3.grad if in_place else torch.zeros_like(emb3)
        dw = load().ngram_bwd(de.to(torch.bfloat16).contiguous(), rows, emb2, emb3, norm_w.float().contiguous(), rstd, g2, g3)
        return None, (None if in_place else g2), (None if in_place else g3), DEFERRED_GRADS.take(norm_w, dw), None, None, None


class _Route(torch.autograd.Function):
    """bf16 router logits -> (top-k weights, indices, per-expert probability sums, per-expert assignment counts)."""

    @staticmethod
    def forward(ctx, logits, k):
        top_w, top_idx, probs, counts, prob_sum = load().moe_route_fwd(logits.contiguous(), k)
        ctx.save_for_backward(probs, top_idx, top_w)
        ctx.mark_non_differentiable(top_idx, counts)
        return top_w, top_idx, prob_sum, counts

    @staticmethod
    def backward(ctx, d_top_w, _idx, d_prob_sum, _counts):
        probs, top_idx, top_w = ctx.saved_tensors
        if d_top_w is None:
            d_top_w = torch.zeros_like(top_w)
        dps = None if d_prob_sum is None else d_prob_sum.float().contiguous()
        return load().moe_route_bwd(probs, top_idx, top_w, d_top_w.float().contiguous(), dps), None


class _Experts(torch.autograd.Function):
    """Routed experts over expert-sorted rows: gather -> grouped gate/up GEMM with SwiGLU epilogue -> grouped down GEMM ->
    weighted combine in slot order.  Backward runs the mirrored grouped GEMMs; weight gradients are accumulated in fp32
    straight into the parameters' gradient buffers when those exist."""

    @staticmethod
    def forward(ctx, x, top_w, top_idx, w_gate_up, w_down):
        ops, err = load(), error_flag(x.device)
        T, h = x.shape
        E, f2, _ = w_gate_up.shape
        k = top_idx.shape[1]
        perm, inv, offsets, sched = ops.moe_sort(top_idx, E)
        xs = ops.moe_gather(x.contiguous(), perm, k)
        hmid = torch.empty(T * k, f2 // 2, dtype=torch.bfloat16, device=x.device)
        gu = torch.empty(T * k, f2, dtype=torch.bfloat16, device=x.device)
        ops.moe_grouped_swiglu(xs, _bf16_weight(w_gate_up), hmid, gu, sched, err)
        ys = torch.empty(T * k, h, dtype=torch.bfloat16, device=x.device)
        ops.moe_grouped_gemm(hmid, _bf16_weight(w_down), ys, sched, False, err)
        out = ops.moe_combine_fwd(ys, inv, top_w)
        ctx.save_for_backward(xs, gu, hmid, ys, inv, offsets, sched, top_w, w_gate_up, w_down)
        ctx.dims = (T, k)
        return out

    @staticmethod
    def backward(ctx, dout):
        ops, err = load(), error_flag(dout.device)
        xs, gu, hmid, ys, inv, offsets, sched, top_w, w_gate_up, w_down = ctx.saved_tensors
        T, k = ctx.dims
        dy, d_top_w = ops.moe_combine_bwd(dout.to(torch.bfloat16).contiguous(), ys, inv, top_w)
        dgu = torch.empty_like(gu)
        ops.moe_grouped_dswiglu(dy, _bf16_weight(w_down), gu, dgu, sched, err)
        dxs = torch.empty_like(xs)
        ops.moe_grouped_gemm(dgu, _bf16_weight(w_gate_up), dxs, sched, True, err)
        dx = ops.moe_unpermute_sum(dxs, inv, T, k)

        def weight_grad(a, b, weight):
            grad = weight.grad
            if grad is not None and grad.dtype == torch.float32 and grad.is_contiguous():
                # accumulate in place; autograd gets no extra tensor
                WGRAD_STREAM.run(lambda: ops.moe_grouped_wgrad(a, b, grad, offsets, err), a, b, offsets)
                return None
            fresh = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
            ops.moe_grouped_wgrad(a, b, fresh, offsets, err)
            return fresh.to(weight.dtype)

        d_down = weight_grad(dy, hmid, w_down) if ctx.needs_input_grad[4] else None
        d_gate_up = weight_grad(dgu, xs, w_gate_up) if ctx.needs_input_grad[3] else None
        return dx, d_top_w, None, d_gate_up, d_down


def _nvtx(name):
    """With Q38_NVTX=1 every call of the decorated hook is an NVTX range (visible in Nsight timelines); otherwise a no-op."""
    def wrap(fn):
        if os.environ.get("Q38_NVTX") != "1":
            return fn

        def ranged(*args, **kwargs):
            torch.cuda.nvtx.range_push(name)
            try:
                return fn(*args, **kwargs)
            finally:
                torch.cuda.nvtx.range_pop()
        ranged.__name__, ranged.__doc__ = fn.__name__, fn.__doc__
        return ranged
    return wrap


class Backend:
    def __init__(self, self_check=True):
        self.ops = load()
        self.layouts = dict(nt=True, nn=True, tn=True)       # which GEMM operand layouts passed the self-check
        # True: chunk operands come from the PyTorch specification and only the scan runs in the CUDA kernel (debug aid)
        self.hybrid_delta_rule = bool(int(os.environ.get("Q38_GDN_HYBRID", "0")))
        # True: no atomically accumulated split-K; weight gradients are then bitwise reproducible from run to run
        self.deterministic = bool(int(os.environ.get("Q38_DETERMINISTIC", "0")))
        self.ep = None            # an `ExpertParallel` context when the experts are split over ranks
        self.selection_override = None   # optional iterator of (count, index) pairs that replaces the block selection (tests)
        self.fp8_ffn = False      # routed experts on block-scaled MXFP8 GEMMs (`q38.ops.fp8`); set by the trainer from --fp8_ffn
        if self_check:
            self._self_check()

    # ---- GEMM flavours (2-D, bf16 in, bf16 or fp32 out) ------------------------------------------------------
    def mm_nt(self, a, b, out_dtype=torch.bfloat16):
        """a[M,K] @ b[N,K]^T"""
        if a.shape[1] % 8 or not self.layouts["nt"]:
            _fallback("mm_nt")
            return (a @ b.t()).to(out_dtype)
        return gemm(a, b, out_dtype=out_dtype)

    def mm_nn(self, a, b, out_dtype=torch.bfloat16):
        """a[M,K] @ b[K,N]"""
        if b.shape[1] % 8 or not self.layouts["nn"]:
            _fallback("mm_nn")
            return (a @ b).to(out_dtype)
        return gemm(_tma_rows(a), b, b_mn_major=True, out_dtype=out_dtype)

    def mm_tn(self, a, b, out_dtype=torch.float32):
        """a[K,M]^T @ b[K,N]   (weight gradients: reduction over the token dimension)"""
        if not self.layouts["tn"]:
            _fallback("mm_tn")
            return (a.t() @ b).to(out_dtype)
        return gemm(_tma_rows(a), _tma_rows(b), a_mn_major=True, b_mn_major=True, out_dtype=out_dtype)

    def weight_grad(self, dy, x, weight):
        """dW = dy^T x.  When the parameter already has an fp32 gradient buffer (the trainer's arena) the product is
        accumulated straight into it with split-K and nothing is returned to autograd; otherwise a fresh tensor is returned."""
        grad = weight.grad
        fast = self.layouts["tn"] and grad is not None and grad.data_ptr() % 16 == 0 and grad.shape[-1] % 4 == 0
        if fast and grad.dtype == torch.float32 and grad.is_contiguous() and grad.dim() == 2:
            a, b = _tma_rows(dy), _tma_rows(x)
            WGRAD_STREAM.run(lambda: gemm(a, b, out=grad, a_mn_major=True, b_mn_major=True, accumulate=True, splits=-1 if self.deterministic else 0), a, b)
            return None
        return self.mm_tn(dy, x).to(weight.dtype)

    def _self_check(self):
        """Compare each operand layout of the tensor-core GEMM with a PyTorch matmul on a small problem.  A layout that
        disagrees is reported loudly and routed to the library matmul, so a wrong descriptor can never train silently."""
        gen = torch.Generator(device="cuda").manual_seed(1)
        a = torch.randn(200, 136, device="cuda", generator=gen).to(torch.bfloat16)
        b = torch.randn(72, 136, device="cuda", generator=gen).to(torch.bfloat16)
        bt = b.t().contiguous()
        at = a.t().contiguous()             # [136, 200]: reduction over 136 rows
        ct = torch.randn(136, 72, device="cuda", generator=gen).to(torch.bfloat16)
        tests = dict(nt=(lambda: gemm(a, b, out_dtype=torch.float32), a.float() @ b.float().t()),
                     nn=(lambda: gemm(a, bt, b_mn_major=True, out_dtype=torch.float32), a.float() @ bt.float()),
                     tn=(lambda: gemm(at, ct, a_mn_major=True, b_mn_major=True, out_dtype=torch.float32), at.float().t() @ ct.float()))
        for name, (run, expect) in tests.items():
            got = run()
            torch.cuda.synchronize()
            bad = int(error_flag().item())
            err = (got - expect).abs().max().item() / expect.abs().max().item()
            if bad or not err < 2e-2:
                error_flag().zero_()
                self.layouts[name] = False
                print(f"[q38.ops] WARNING: tensor-core GEMM layout '{name}' failed its self-check "
                      f"(rel err {err:.3e}, kernel error {bad}); using the library matmul for it", flush=True)

    # ---- hooks called by the model -----------------------------------------------------------------------------
    def linear(self, x, weight):
        return _Linear.apply(x, weight, self)

    def linears(self, x, *weights):
        """Projections of one input by several weights (tuple of outputs); their input gradients are summed inside the GEMMs."""
        # Default (Q38_MULTI_LINEAR=2): one autograd node for the group; in its backward the second and later input-gradient GEMMs
        # add their tiles onto the first one's output with the TMA unit's bf16 reduce-add, so no addition kernels run (measured
        # 703.7 vs 712.0 ms per q38_c2 step).  =1 reads the running sum in the GEMM epilogue instead, row by row, which measured
        # 1 % slower than separate additions; =0 is one autograd node per projection with autograd's own additions.
        if os.environ.get("Q38_MULTI_LINEAR", "2") not in ("1", "2"):
            return tuple(self.linear(x, w) for w in weights)
        return _MultiLinear.apply(x, self, *weights)

    def rmsnorm(self, x, weight, eps, out_dtype):
        return _RMSNorm.apply(x, weight, eps, out_dtype)

    def gated_rmsnorm(self, x, gate, weight, eps):
        if x.dtype != torch.bfloat16 or x.shape[-1] != 64:
            return None
        return _GatedRMSNorm.apply(x, gate, weight, eps)

    @_nvtx("q38.mhc_pre_norm")
    def mhc_pre_norm(self, mhc, norm, X, dtype):
        link = _MhcLink()
        x, coef = _MhcPreNorm.apply(X, mhc.A.weight, mhc.B.weight, mhc.b_pre, mhc.b_post, mhc.b_res, mhc.alphas, norm.weight,
                                    mhc.iters, norm.eps, dtype, link)
        return x, (X, coef, link)

    @_nvtx("q38.mhc_post")
    def mhc_post(self, mhc, y, state):
        X, coef, link = state
        return _MhcPost.apply(X, y, coef, link)

    def delta_rule(self, q, k, v, g, beta):
        """q,k [B,S,Hk,64], v [B,S,Hv,64] bf16, g fp32 / beta [B,S,Hv] -> o [B,S,Hv,64] bf16 (S a multiple of 64)."""
        if not self.hybrid_delta_rule:
            Hk, Hv = k.shape[2], v.shape[2]
            return _DeltaRule.apply(torch.cat([q.flatten(2), k.flatten(2), v.flatten(2)], dim=-1), g, beta, Hk, Hv)
        from ..models import modeling
        B, S, Hv = v.shape[0], v.shape[1], v.shape[2]
        ops = modeling.gdn_chunk_operands(q, k, v, g, beta)
        flat = lambda t: t.reshape(B * Hv, -1, 64, 64)
        return _GdnScan.apply(flat(ops["w"]), flat(ops["u"]), flat(ops["P"]), flat(ops["qg"]), flat(ops["kg"]),
                              ops["carry"].reshape(B * Hv, -1), B, Hv)

    @_nvtx("q38.gated_deltanet")
    def gated_deltanet(self, m, x):
        B, S, _ = x.shape
        if x.dtype != torch.bfloat16 or S % 64 or m.head_k_dim != 64 or m.head_v_dim != 64:
            return None
        from ..models import modeling
        F = torch.nn.functional
        p_qkv, z, p_b, p_a = self.linears(x, m.in_proj_qkv.weight, m.in_proj_z.weight, m.in_proj_b.weight, m.in_proj_a.weight)
        qkv = _ConvSilu.apply(p_qkv, m.conv1d.weight)
        beta, g = _GdnGates.apply(p_b, p_a, m.A_log, m.dt_bias)
        if self.hybrid_delta_rule:
            q, k, v = qkv.split([m.key_dim, m.key_dim, m.value_dim], dim=-1)
            o = self.delta_rule(q.reshape(B, S, -1, 64), k.reshape(B, S, -1, 64), v.reshape(B, S, -1, 64), g, beta)
        else:
            o = _DeltaRule.apply(qkv, g, beta, m.num_k_heads, m.num_v_heads)
        o = self.gated_rmsnorm(o.reshape(-1, 64), z.reshape(-1, 64), m.norm.weight, m.norm.variance_epsilon)
        return self.linear(o.reshape(B, S, -1), m.out_proj.weight)

    def indexer_block_logprobs(self, indexer, x, cos, sin, q_main=None, k_main=None, main_scale=None):
        """Indexer projections + score kernels.  With main q/k: (kl, lp_blk) for training; without: (None, lp_blk)."""
        from ..models import modeling
        B, S, _ = x.shape
        NI, D = indexer.n_ih, indexer.d_ih
        if D == 64 and cos.shape[-1] == 16 and x.dtype == torch.bfloat16:
            qi = _head_prep(self.linear(x, indexer.wq.weight).view(B, S, NI, D), None, cos, sin)[0]
            ki = _head_prep(self.linear(x, indexer.wk.weight).view(B, S, 1, D), None, cos, sin)[0][:, 0]
        else:
            qi = modeling.apply_rope(self.linear(x, indexer.wq.weight).view(B, S, NI, D).transpose(1, 2), cos, sin).contiguous()
            ki = modeling.apply_rope(self.linear(x, indexer.wk.weight).view(B, S, 1, D).transpose(1, 2), cos, sin)[:, 0].contiguous()
        wi = (self.linear(x, indexer.ww.weight).float() * NI ** -0.5).contiguous()
        if q_main is not None:
            return _IndexerKL.apply(qi, ki, wi, q_main, k_main, main_scale, D ** -0.5)
        ops = load()
        blse = ops.qsa_indexer_fwd(qi.detach(), ki.detach(), wi.detach(), D ** -0.5)
        return None, ops.qsa_kl_combine(None, blse, 1)[1]

    @_nvtx("q38.qsa_attention")
    def qsa_attention(self, attn, x, cos, sin, indexer, budget, dense, want_kl):
        from ..models import modeling
        F = torch.nn.functional
        B, S, _ = x.shape
        hd = attn.head_dim
        if x.dtype != torch.bfloat16 or hd != 64 or S % 64 or S > 8192 or (indexer is not None and (indexer.d_ih != 64 or indexer.n_ih > 4)):
            return None
        p_q, p_k, p_v = self.linears(x, attn.q_proj.weight, attn.k_proj.weight, attn.v_proj.weight)
        qg = p_q.view(B, S, -1, 2 * hd)
        if cos.shape[-1] == 16:
            q, gate = _head_prep(qg, attn.q_norm, cos, sin)
            k = _head_prep(p_k.view(B, S, -1, hd), attn.k_norm, cos, sin)[0]
        else:
            q, gate = qg[..., :hd], qg[..., hd:].reshape(B, S, -1)
            q = modeling.apply_rope(attn.q_norm(q).transpose(1, 2), cos, sin).contiguous()
            k = modeling.apply_rope(attn.k_norm(p_k.view(B, S, -1, hd)).transpose(1, 2), cos, sin).contiguous()
        v = p_v.view(B, S, -1, hd).transpose(1, 2)
        kl = lp_blk = None
        if indexer is not None and (want_kl or not dense):
            if want_kl:
                kl, lp_blk = self.indexer_block_logprobs(indexer, x.detach(), cos, sin, q.detach(), k.detach(), attn.scaling)
            elif os.environ.get("Q38_INDEXER_BASELINE"):
                with torch.no_grad():
                    _, lp_blk = self.indexer_block_logprobs(indexer, x.detach(), cos, sin)
            else:
                # no KL wanted (evaluation, or training steps that skip it): block selection only looks at the first query of each
                # 64-token block, so only those S/64 queries are scored -> lp_blk [B, nb, nb]  (reference: modeling_qwen3_8_moe.py:1126)
                with torch.no_grad():
                    qi, ki, wi = indexer.project(x.detach(), cos, sin)
                    if qi.dtype == torch.bfloat16 and ki.dtype == torch.bfloat16:
                        lp_blk = load().qsa_first_query_lp(qi[:, :, ::modeling.BLK].contiguous(), ki.reshape(B, S, -1).contiguous(),
                                                           wi[:, ::modeling.BLK].float().contiguous(), indexer.d_ih ** -0.5)
                    else:
                        score = indexer(x.detach(), cos, sin, block_queries=True)
                        pos = torch.arange(S, device=x.device)
                        score = score.masked_fill(pos[None, :] > pos[::modeling.BLK][:, None], -1e9)
                        lp_blk = score.log_softmax(-1).view(B, S // modeling.BLK, S // modeling.BLK, modeling.BLK).logsumexp(-1).contiguous()
        if dense or indexer is None:
            o = _BlockAttention.apply(q, k, v, None, None, attn.scaling)
        else:
            if self.selection_override is not None:              # numerics tests: attend to the blocks an fp32 run selected
                count, index = (t.to(q.device).contiguous() for t in next(self.selection_override))
            else:
                count, index = load().qsa_select(lp_blk, budget)
            if want_kl and modeling.QSA_STAT.get("on"):
                # debug statistic (reference: modeling_qwen3_8_moe.py:1136-1142): share of the dense attention mass that falls into
                # the selected blocks.  The kernels never form the block masses, so this recomputes them the slow way.
                with torch.no_grad():
                    P = modeling.block_mass(q.detach(), k.detach(), attn.scaling)
                    chosen = modeling.block_sparse_mask(count, index, S)[:, ::modeling.BLK, ::modeling.BLK].float()
                    modeling.QSA_STAT.setdefault("recall", []).append((P.view(B, S // modeling.BLK, modeling.BLK, -1) * chosen[:, :, None, :]).sum(-1).mean().item())
            o = _BlockAttention.apply(q, k, v, count, index, attn.scaling)
        o = o.reshape(B, S, -1)
        o = _SigmoidMul.apply(o, gate) if (o.numel() % 8 == 0 and o.dtype == torch.bfloat16 and gate.dtype == torch.bfloat16) else o * torch.sigmoid(gate)
        return self.linear(o, attn.o_proj.weight), kl

    def embedding(self, weight, ids):
        if weight.dtype != torch.float32 or not weight.is_contiguous():
            return torch.nn.functional.embedding(ids, weight)
        return _Embed.apply(weight, ids)

    @_nvtx("q38.ngram_delta")
    def ngram_delta(self, m, h, ids):
        """sigmoid(W h + b) * rmsnorm(emb2[i2] + emb3[i3]) with the hash, gather, norm and scatter-add backward in one kernel pair."""
        w2, w3 = m.emb2.weight, m.emb3.weight
        if (h.dtype != torch.bfloat16 or m.collect or w2.dtype != torch.float32 or m.hidden % 4 or not w2.is_contiguous() or not w3.is_contiguous()
                or m.norm.weight is None):
            i2, i3 = m.indices(ids)
            e = m.norm((m.emb2(i2) + m.emb3(i3)).float()).to(h.dtype)
        else:
            eos = -1 if m.eos_id is None else int(m.eos_id)
            e = _NGramEmbed.apply(ids, w2, w3, m.norm.weight, int(m.vocab), eos, float(m.norm.eps if m.norm.eps is not None else 1e-6))
        logit = self.linear(h, m.gate.weight) + m.gate.bias.to(h.dtype)
        if e.dtype == torch.bfloat16 and logit.dtype == torch.bfloat16 and e.shape == logit.shape and e.numel() % 8 == 0:
            return _SigmoidMul.apply(e, logit)                   # e * sigmoid(logit), one kernel each way
        return torch.sigmoid(logit) * e

    @_nvtx("q38.moe_block")
    def moe_block(self, block, x):
        experts = block.experts
        E, f, h = experts.num_experts, experts.intermediate_dim, experts.hidden_dim
        if x.dtype != torch.bfloat16 or E > 64 or block.gate.top_k > 8 or f % 16 or f > 256 or h % 8:
            return None
        shape = x.shape
        x2 = x.reshape(-1, h)
        shared = block.shared_expert
        logits, sg, su, gate_logit = self.linears(x2, block.gate.weight, shared.gate_proj.weight, shared.up_proj.weight, block.shared_expert_gate.weight)
        top_w, top_idx, prob_sum, counts = _Route.apply(logits, block.gate.top_k)
        if block._recording():
            block.stats_sink.add(counts, prob_sum, x2.shape[0])
        # Expert parallelism is the training path.  Without gradients (validation, export checks) the replicated path runs on
        # the full expert tensors, which the engine assembles from the ranks' slices first (`GradEngine.gather_experts`).
        if self.ep is not None and torch.is_grad_enabled():
            from ..parallel.ep import _ExpertsEP
            routed = _ExpertsEP.apply(x2, top_w, top_idx, experts.gate_up_proj, experts.down_proj, self.ep, self.ep.layer_index(block))
        elif self.fp8_ffn:
            from .fp8 import ExpertsFP8
            routed = ExpertsFP8.apply(x2, top_w, top_idx, experts.gate_up_proj, experts.down_proj, _bf16_weight, WGRAD_STREAM)
        else:
            routed = _Experts.apply(x2, top_w, top_idx, experts.gate_up_proj, experts.down_proj)
        mid = _SwiGLU.apply(sg, su) if sg.numel() % 8 == 0 else torch.nn.functional.silu(sg) * su
        if h % 8 == 0 and gate_logit.shape[1] == 1:
            return _GateAdd.apply(routed, self.linear(mid, shared.down_proj.weight), gate_logit).reshape(shape)
        return (routed + torch.sigmoid(gate_logit) * self.linear(mid, shared.down_proj.weight)).reshape(shape)

    @_nvtx("q38.linear_cross_entropy")
    def linear_cross_entropy(self, weight, hidden, target, reduction):
        """Chunked logits + CE; logits of one chunk only ever exist, in fp32."""
        return _chunked_linear_ce(self, weight, hidden, target, reduction)

    def describe(self):
        native = sorted(n for n in ("linear", "rmsnorm", "gated_rmsnorm", "mhc_pre_norm", "mhc_post", "gated_deltanet",
                                    "qsa_attention", "moe_block", "ngram_delta", "embedding", "linear_cross_entropy") if hasattr(self, n))
        return dict(native=native, gemm_layouts=self.layouts, library_matmul_fallbacks=dict(LIBRARY_FALLBACKS), fp8_ffn=bool(self.fp8_ffn))


class _LinearCE(torch.autograd.Function):
    """Sum of token cross-entropies of ``hidden @ weight^T`` (ignore index -100) without fp32 logits.

    Forward, per chunk of rows: vocabulary GEMM (bf16 logits) -> in-place CE kernel that leaves softmax - onehot in the
    logits buffer.  The gradient buffers are kept (bf16) and the backward is two GEMMs: d(hidden) = dlogits W and
    d(W) += dlogits^T hidden (split-K, accumulated into the tied embedding's gradient), both scaled by the upstream gradient."""

    @staticmethod
    def forward(ctx, hidden, weight, target, backend, rows):
        ops = load()
        h2 = hidden.reshape(-1, hidden.shape[-1]).to(torch.bfloat16).contiguous()
        w = _bf16_weight(weight)
        total = torch.zeros((), dtype=torch.float32, device=hidden.device)
        grads = []
        for o in range(0, h2.shape[0], rows):
            logits = backend.mm_nt(h2[o:o + rows], w)
            total = total + ops.ce_inplace(logits, target[o:o + rows].contiguous()).sum()
            grads.append(logits)
        ctx.save_for_backward(h2, weight, *grads)
        ctx.backend, ctx.rows, ctx.shape, ctx.dtype = backend, rows, hidden.shape, hidden.dtype
        return total

    @staticmethod
    def backward(ctx, g):
        h2, weight, *grads = ctx.saved_tensors
        backend, rows = ctx.backend, ctx.rows
        w = _bf16_weight(weight)
        gs = g.to(torch.bfloat16)
        dh = torch.empty_like(h2)
        need_w = ctx.needs_input_grad[1]
        dw_total = None
        for i, dl in enumerate(grads):
            o = i * rows
            dh[o:o + rows] = backend.mm_nn(dl, w)
            if need_w:
                part = backend.weight_grad(dl, (h2[o:o + rows] * gs), weight)
                if part is not None:
                    dw_total = part if dw_total is None else dw_total + part
        return (dh * gs).view(ctx.shape).to(ctx.dtype), dw_total, None, None, None


def _chunked_linear_ce(backend, weight, hidden, target, reduction, rows=8192):
    V = weight.shape[0]
    if hidden.shape[-1] % 8 == 0 and V % 8 == 0 and V <= 16384:
        total = _LinearCE.apply(hidden, weight, target, backend, rows)
        if reduction == "sum":
            return total
        return total / (target != -100).sum().clamp_min(1)
    return _chunked_linear_ce_reference(backend, weight, hidden, target, reduction, rows)


def _chunked_linear_ce_reference(backend, weight, hidden, target, reduction, rows=8192):
    total = hidden.new_zeros((), dtype=torch.float32)
    count = (target != -100).sum()
    for o in range(0, hidden.shape[0], rows):
        logits = backend.linear(hidden[o:o + rows], weight).float()
        total = total + torch.nn.functional.cross_entropy(logits, target[o:o + rows], ignore_index=-100, reduction="sum")
    if reduction == "sum":
        return total
    return total / count.clamp_min(1)
