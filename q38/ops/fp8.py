"""Routed experts with block-scaled MXFP8 GEMMs (``--fp8_ffn 1``).

Same data flow as the bf16 expert path (`q38.ops.backend._Experts`): sort pairs by expert, grouped gate/up product, SwiGLU,
grouped down product, weighted combine; backward mirrors it.  The four activation-by-weight products (gate/up, down, and the
two input-gradient products) run on `tcgen05.mma.kind::mxf8f6f4.block_scale` with E4M3 operands and one E8M0 scale per 32
elements of the reduction dimension (`csrc/mxfp8.cu`); activations are quantised per product by a kernel driven by the expert
tile schedule (for the first product the gather through the sort permutation is fused into it).  Weight gradients stay in
bf16 with fp32 accumulation, master weights stay fp32 / bf16 and are never touched.

Weights are quantised from the bf16 shadow where they are used (four forms per expert block: each weight with 32-element
blocks along either of its two axes, because the forward and the input-gradient product contract different axes).

The reference has no FP8 path; its FFN runs in bf16 (q38/inference.py padded/grouped experts).  Numerics: the test
`tests/test_gpu_fp8.py` bounds the error against the bf16 path.
"""
import torch

from . import error_flag, load

def _quantised(weight_bf16, transpose):
    """(q, sf, bn) of `weight_bf16` [E, A, B]: 32-element blocks along B, or along A of the transposed view when `transpose`.

    Quantised at every use: the kernels of a micro-step are replayed from a CUDA graph, so a cached tensor would have to keep
    its address across optimizer steps; re-reading the bf16 weights costs about 1 GB of traffic per micro-step for q38_c2,
    well under one per cent of the step."""
    lib = load()
    view = weight_bf16.transpose(1, 2) if transpose else weight_bf16
    bn = int(lib.mxfp8_pick_bn(view.shape[1]))
    q, sf = lib.mxfp8_quantize_weight(view, bn)
    return q, sf, bn


def supported(h, f):
    """Reduction lengths must be multiples of 16 bytes for TMA: hidden size, expert width and twice the expert width."""
    return h % 16 == 0 and f % 16 == 0


class ExpertsFP8(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, top_w, top_idx, w_gate_up, w_down, bf16_weight, wgrad_stream):
        lib, err = load(), error_flag(x.device)
        T, h = x.shape
        E, f2, _ = w_gate_up.shape
        f, k, P = f2 // 2, top_idx.shape[1], T * top_idx.shape[1]
        wgu, wd = bf16_weight(w_gate_up), bf16_weight(w_down)
        perm, inv, offsets, sched = lib.moe_sort(top_idx, E)
        x = x.contiguous()
        xq, sfx = lib.mxfp8_quantize_rows(x, perm, k, sched, P)                       # gather + quantise
        q, sf, bn = _quantised(wgu, False)
        gu = torch.empty(P, f2, dtype=torch.bfloat16, device=x.device)
        lib.mxfp8_grouped_gemm(xq, sfx, q, sf, gu, sched, bn, err)
        hmid = lib.swiglu_fwd(gu[:, :f].contiguous(), gu[:, f:].contiguous())
        hq, sfh = lib.mxfp8_quantize_rows(hmid, None, 1, sched, P)
        q, sf, bn = _quantised(wd, False)
        ys = torch.empty(P, h, dtype=torch.bfloat16, device=x.device)
        lib.mxfp8_grouped_gemm(hq, sfh, q, sf, ys, sched, bn, err)
        out = lib.moe_combine_fwd(ys, inv, top_w)
        ctx.save_for_backward(x, perm, gu, hmid, ys, inv, offsets, sched, top_w, w_gate_up, w_down)
        ctx.dims, ctx.bf16_weight, ctx.wgrad_stream = (T, k), bf16_weight, wgrad_stream
        return out

    @staticmethod
    def backward(ctx, dout):
        lib, err = load(), error_flag(dout.device)
        x, perm, gu, hmid, ys, inv, offsets, sched, top_w, w_gate_up, w_down = ctx.saved_tensors
        T, k = ctx.dims
        P, f = T * k, hmid.shape[1]
        wgu, wd = ctx.bf16_weight(w_gate_up), ctx.bf16_weight(w_down)
        dy, d_top_w = lib.moe_combine_bwd(dout.to(torch.bfloat16).contiguous(), ys, inv, top_w)
        dyq, sfdy = lib.mxfp8_quantize_rows(dy, None, 1, sched, P)
        q, sf, bn = _quantised(wd, True)                          # [E, f, h]: contraction over h
        dh = torch.empty(P, f, dtype=torch.bfloat16, device=dout.device)
        lib.mxfp8_grouped_gemm(dyq, sfdy, q, sf, dh, sched, bn, err)
        dg, du = lib.swiglu_bwd(dh, gu[:, :f].contiguous(), gu[:, f:].contiguous())
        dgu = torch.cat([dg, du], dim=1)
        dguq, sfdgu = lib.mxfp8_quantize_rows(dgu, None, 1, sched, P)
        q, sf, bn = _quantised(wgu, True)                      # [E, h, 2f]: contraction over 2f
        dxs = torch.empty(P, x.shape[1], dtype=torch.bfloat16, device=dout.device)
        lib.mxfp8_grouped_gemm(dguq, sfdgu, q, sf, dxs, sched, bn, err)
        dx = lib.moe_unpermute_sum(dxs, inv, T, k)
        xs = lib.moe_gather(x, perm, k)                                                # bf16 rows for the weight gradient

        def weight_grad(a, b, weight):
            grad = weight.grad
            if grad is not None and grad.dtype == torch.float32 and grad.is_contiguous():
                ctx.wgrad_stream.run(lambda: lib.moe_grouped_wgrad(a, b, grad, offsets, err), a, b, offsets)
                return None
            fresh = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
            lib.moe_grouped_wgrad(a, b, fresh, offsets, err)
            return fresh.to(weight.dtype)

        d_down = weight_grad(dy, hmid, w_down) if ctx.needs_input_grad[4] else None
        d_gate_up = weight_grad(dgu, xs, w_gate_up) if ctx.needs_input_grad[3] else None
        return dx, d_top_w, None, d_gate_up, d_down, None, None
