"""Expert parallelism: experts are split evenly over the data-parallel ranks (``E / world`` per GPU).

Per MoE layer and micro-step (forward):

    route + counting sort (local)  ->  publish per-expert counts to all peers  ->  barrier
    ep_plan (every rank derives where its rows land on each owner and the owner's tile schedule)
    ep_dispatch: fused permute + send, rows stored straight into the owner's receive buffer       ->  barrier
    owner: grouped gate/up GEMM + SwiGLU, grouped down GEMM whose epilogue stores every output row
           into the source rank's buffer at the row's sorted position (combine transfer fused in)   ->  barrier
    source: weighted combine in slot order

The backward mirrors it (gradient rows travel to the owner, d(x) rows travel back through the GEMM epilogue).  Expert
weights and their optimizer state are touched only by their owner; their gradients already contain the tokens of every
rank, so they are scaled by ``1 / world`` instead of being reduced.  Receive buffers are sized by a capacity factor over
the balanced load; an overflow (extreme routing skew) is reported through the kernel error flag, never written out of
bounds, and the step must be rerun with a larger factor.
"""
import torch

from .. import ops
from ..ops.backend import _bf16_weight


class ExpertParallel:
    def __init__(self, transport, rank, world, hidden, ffn, experts, topk, tokens, layers, capacity_factor=4.0):
        if experts % world:
            raise ValueError("the number of experts must be a multiple of the number of ranks")
        self.t, self.rank, self.world = transport, rank, world
        self.hidden, self.ffn, self.experts, self.topk = hidden, ffn, experts, topk
        self.local_experts = experts // world
        self.pairs = tokens * topk
        self.capacity = (int(capacity_factor * self.pairs) + 127) // 128 * 128
        dev = transport.device
        alloc = transport.allocate_named
        self.counts = alloc("ep_counts", world * experts, torch.int32)
        self.recv_dy = alloc("ep_recv_dy", self.capacity * hidden, torch.bfloat16).view(self.capacity, hidden)
        self.back_dx = alloc("ep_back_dx", self.pairs * hidden, torch.bfloat16).view(self.pairs, hidden)
        self.recv_x, self.ret_rank, self.ret_row, self.back_y = [], [], [], []
        for i in range(layers):
            self.recv_x.append(alloc(f"ep_recv_x{i}", self.capacity * hidden, torch.bfloat16).view(self.capacity, hidden))
            self.ret_rank.append(alloc(f"ep_ret_rank{i}", self.capacity, torch.int32))
            self.ret_row.append(alloc(f"ep_ret_row{i}", self.capacity, torch.int32))
            self.back_y.append(alloc(f"ep_back_y{i}", self.pairs * hidden, torch.bfloat16).view(self.pairs, hidden))
        transport.exchange()
        self.layer_of = {}

    def peers(self, name):
        return self.t.peers[name]

    def local_slice(self):
        return slice(self.rank * self.local_experts, (self.rank + 1) * self.local_experts)

    def layer_index(self, block):
        return self.layer_of.setdefault(id(block), len(self.layer_of))


class _ExpertsEP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, top_w, top_idx, w_gate_up, w_down, ep, layer):
        lib, err = ops.load(), ops.error_flag(x.device)
        T, h = x.shape
        k, E = top_idx.shape[1], ep.experts
        if T * k > ep.pairs:
            raise RuntimeError(f"expert-parallel buffers were sized for at most {ep.pairs} routed pairs, got {T * k}")
        sl = ep.local_slice()
        wgu, wd = _bf16_weight(w_gate_up)[sl], _bf16_weight(w_down)[sl]
        perm, inv, offsets, _ = lib.moe_sort(top_idx, E)
        lib.ep_publish_counts(offsets, ep.rank, ep.peers("ep_counts"))
        ep.t.barrier()
        send_base, recv_offsets, sched, status = lib.ep_plan(ep.counts, ep.rank, ep.world, ep.capacity, err)
        xc = x.contiguous()
        lib.ep_dispatch(xc, perm, top_idx.reshape(-1), offsets, send_base, k, ep.local_experts, ep.capacity, True, ep.rank,
                        ep.peers(f"ep_recv_x{layer}"), ep.peers(f"ep_ret_rank{layer}"), ep.peers(f"ep_ret_row{layer}"))
        ep.t.barrier()
        rows = ep.recv_x[layer]
        f = wgu.shape[1] // 2
        hmid = torch.empty(ep.capacity, f, dtype=torch.bfloat16, device=x.device)
        gu = torch.empty(ep.capacity, 2 * f, dtype=torch.bfloat16, device=x.device)
        lib.moe_grouped_swiglu(rows, wgu, hmid, gu, sched, err)
        lib.moe_grouped_gemm_return(hmid, wd, ep.back_y[layer], sched, False, err, ep.ret_rank[layer], ep.ret_row[layer], ep.peers(f"ep_back_y{layer}"))
        ep.t.barrier()
        out = lib.moe_combine_fwd(ep.back_y[layer], inv, top_w)
        ctx.save_for_backward(perm, inv, offsets, send_base, recv_offsets, sched, top_w, top_idx, gu, hmid, w_gate_up, w_down)
        ctx.ep, ctx.layer, ctx.dims = ep, layer, (T, k)
        return out

    @staticmethod
    def backward(ctx, dout):
        lib, err = ops.load(), ops.error_flag(dout.device)
        perm, inv, offsets, send_base, recv_offsets, sched, top_w, top_idx, gu, hmid, w_gate_up, w_down = ctx.saved_tensors
        ep, layer = ctx.ep, ctx.layer
        T, k = ctx.dims
        sl = ep.local_slice()
        wgu, wd = _bf16_weight(w_gate_up)[sl], _bf16_weight(w_down)[sl]
        dy, d_top_w = lib.moe_combine_bwd(dout.to(torch.bfloat16).contiguous(), ep.back_y[layer], inv, top_w)
        lib.ep_dispatch(dy, perm, top_idx.reshape(-1), offsets, send_base, k, ep.local_experts, ep.capacity, False, ep.rank,
                        ep.peers("ep_recv_dy"), ep.peers(f"ep_ret_rank{layer}"), ep.peers(f"ep_ret_row{layer}"))
        ep.t.barrier()
        dgu = torch.empty_like(gu)
        lib.moe_grouped_dswiglu(ep.recv_dy, wd, gu, dgu, sched, err)
        lib.moe_grouped_gemm_return(dgu, wgu, ep.back_dx, sched, True, err, ep.ret_rank[layer], ep.ret_row[layer], ep.peers("ep_back_dx"))

        def weight_grad(a, b, weight):
            grad = weight.grad
            if grad is not None and grad.dtype == torch.float32 and grad.is_contiguous():
                lib.moe_grouped_wgrad(a, b, grad[sl], recv_offsets, err)
                return None
            fresh = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
            lib.moe_grouped_wgrad(a, b, fresh[sl], recv_offsets, err)
            return fresh.to(weight.dtype)

        d_down = weight_grad(ep.recv_dy, hmid, w_down)
        d_gate_up = weight_grad(dgu, ep.recv_x[layer], w_gate_up)
        ep.t.barrier()
        dx = lib.moe_unpermute_sum(ep.back_dx, inv, T, k)
        return dx, d_top_w, None, d_gate_up, d_down, None, None
