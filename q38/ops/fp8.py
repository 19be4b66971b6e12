"""Routed experts with block-scaled MXFP8 GEMMs (``--fp8_ffn 1``).

Same data flow as the bf16 expert path (`q38.ops.backend._Experts`): sort pairs by expert, grouped gate/up product, SwiGLU,
grouped down product, weighted combine; backward mirrors it.  The four activation-by-weight products (gate/up, down, and the
two input-gradient products) run on `tcgen05.mma.kind::mxf8f6f4.block_scale` with E4M3 operands and one E8M0 scale per 32
elements of the reduction dimension (`csrc/mxfp8.cu`); activations are quantised per product by a kernel driven by the expert
tile schedule (for the first product the gather through the sort permutation is fused into it).  Weight gradients stay in
bf16 with fp32 accumulation, master weights stay fp32 / bf16 and are never touched.

Weights are quantised from the bf16 shadow once per optimizer step by `refresh_weights` (the trainer calls it before the
micro-steps) into persistent buffers, four forms per expert block; without a trainer they are quantised at each use.

The reference has no FP8 path; its FFN runs in bf16 (q38/inference.py padded/grouped experts).  Numerics: the test
`tests/test_gpu_fp8.py` bounds the error against the bf16 path.
"""
import torch

from . import error_flag, load

_PERSISTENT = {}          # (id(parameter), transpose) -> (q, sf, bn) in buffers whose addresses never change


def _quantise(weight_bf16, transpose):
    lib = load()
    view = weight_bf16.transpose(1, 2) if transpose else weight_bf16
    bn = int(lib.mxfp8_pick_bn(view.shape[1]))
    q, sf = lib.mxfp8_quantize_weight(view, bn)
    return q, sf, bn


@torch.no_grad()
def refresh_weights(model, bf16_weight):
    """Quantise the expert weights of `model` once, into persistent buffers (four forms per expert block: each weight with its
    32-element blocks along either axis, because the forward and the input-gradient product contract different axes).

    The trainer calls this at the start of every optimizer step, outside the captured micro-step: the micro-steps of the step
    (replayed CUDA graphs) then read the same buffers, so the weights are quantised once per step instead of once per use."""
    for module in model.modules():
        gate_up, down = getattr(module, "gate_up_proj", None), getattr(module, "down_proj", None)
        if not (torch.is_tensor(gate_up) and torch.is_tensor(down) and gate_up.dim() == 3 and down.dim() == 3):
            continue
        for weight in (gate_up, down):
            for transpose in (False, True):
                q, sf, bn = _quantise(bf16_weight(weight), transpose)
                held = _PERSISTENT.get((id(weight), transpose))
                if held is not None and held[0].shape == q.shape and held[1].shape == sf.shape and held[0].device == q.device:
                    held[0].copy_(q)
                    held[1].copy_(sf)
                else:
                    _PERSISTENT[(id(weight), transpose)] = (q, sf, bn)


def drop_weights():
    _PERSISTENT.clear()


def _quantised(weight, weight_bf16, transpose):
    """(q, sf, bn) of an expert weight: the per-step persistent copy while training, a fresh quantisation otherwise (evaluation
    runs after the optimizer step, when the persistent copy is one step old)."""
    if torch.is_grad_enabled():
        held = _PERSISTENT.get((id(weight), transpose))
        if held is not None and held[0].device == weight_bf16.device:
            return held
    return _quantise(weight_bf16, transpose)


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
        q, sf, bn = _quantised(w_gate_up, wgu, False)
        gu = torch.empty(P, f2, dtype=torch.bfloat16, device=x.device)
        lib.mxfp8_grouped_gemm(xq, sfx, q, sf, gu, sched, bn, err)
        hmid = lib.swiglu_fwd(gu[:, :f].contiguous(), gu[:, f:].contiguous())
        hq, sfh = lib.mxfp8_quantize_rows(hmid, None, 1, sched, P)
        q, sf, bn = _quantised(w_down, wd, False)
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
        q, sf, bn = _quantised(w_down, wd, True)                          # [E, f, h]: contraction over h
        dh = torch.empty(P, f, dtype=torch.bfloat16, device=dout.device)
        lib.mxfp8_grouped_gemm(dyq, sfdy, q, sf, dh, sched, bn, err)
        dg, du = lib.swiglu_bwd(dh, gu[:, :f].contiguous(), gu[:, f:].contiguous())
        dgu = torch.cat([dg, du], dim=1)
        dguq, sfdgu = lib.mxfp8_quantize_rows(dgu, None, 1, sched, P)
        q, sf, bn = _quantised(w_gate_up, wgu, True)                      # [E, h, 2f]: contraction over 2f
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
