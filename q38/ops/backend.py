"""Kernel backend: the object the model file calls for every hot op when tensors live on a GPU.

Each method is a `torch.autograd.Function` (or a composition of them) over the CUDA kernels of `csrc/`.
A method that is absent makes the model use its PyTorch specification for that op; the set of present
methods is reported by `describe()` so a run records exactly which paths were native.
"""
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
            dw = backend.mm_tn(dy2, x2).to(weight.dtype)
        return dx, dw, None


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
        return dx, dw.to(weight.dtype), None, None


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
        return dx, dgate, dw.to(weight.dtype), None


class Backend:
    def __init__(self, self_check=True):
        self.ops = load()
        self.layouts = dict(nt=True, nn=True, tn=True)       # which GEMM operand layouts passed the self-check
        if self_check:
            self._self_check()

    # ---- GEMM flavours (2-D, bf16 in, bf16 or fp32 out) ------------------------------------------------------
    def mm_nt(self, a, b, out_dtype=torch.bfloat16):
        """a[M,K] @ b[N,K]^T"""
        if a.shape[1] % 8 or not self.layouts["nt"]:
            return (a @ b.t()).to(out_dtype)
        return gemm(a, b, out_dtype=out_dtype)

    def mm_nn(self, a, b, out_dtype=torch.bfloat16):
        """a[M,K] @ b[K,N]"""
        if a.shape[1] % 8 or b.shape[1] % 8 or not self.layouts["nn"]:
            return (a @ b).to(out_dtype)
        return gemm(a, b, b_mn_major=True, out_dtype=out_dtype)

    def mm_tn(self, a, b, out_dtype=torch.float32):
        """a[K,M]^T @ b[K,N]   (weight gradients: reduction over the token dimension)"""
        if a.shape[1] % 8 or b.shape[1] % 8 or not self.layouts["tn"]:
            return (a.t() @ b).to(out_dtype)
        return gemm(a, b, a_mn_major=True, b_mn_major=True, out_dtype=out_dtype)

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

    def rmsnorm(self, x, weight, eps, out_dtype):
        return _RMSNorm.apply(x, weight, eps, out_dtype)

    def gated_rmsnorm(self, x, gate, weight, eps):
        if x.dtype != torch.bfloat16 or x.shape[-1] != 64:
            return None
        return _GatedRMSNorm.apply(x, gate, weight, eps)

    def linear_cross_entropy(self, weight, hidden, target, reduction):
        """Chunked logits + CE; logits of one chunk only ever exist, in fp32."""
        return _chunked_linear_ce(self, weight, hidden, target, reduction)

    def describe(self):
        native = sorted(n for n in ("linear", "rmsnorm", "gated_rmsnorm", "mhc_pre_norm", "mhc_post", "gated_deltanet",
                                    "qsa_attention", "moe_block", "ngram_delta", "linear_cross_entropy") if hasattr(self, n))
        return dict(native=native, gemm_layouts=self.layouts)


def _chunked_linear_ce(backend, weight, hidden, target, reduction, rows=8192):
    total = hidden.new_zeros((), dtype=torch.float32)
    count = (target != -100).sum()
    for o in range(0, hidden.shape[0], rows):
        logits = backend.linear(hidden[o:o + rows], weight).float()
        total = total + torch.nn.functional.cross_entropy(logits, target[o:o + rows], ignore_index=-100, reduction="sum")
    if reduction == "sum":
        return total
    return total / count.clamp_min(1)
