"""Numerics of every CUDA kernel against a plain PyTorch fp32 evaluation of the same op (run on a B200)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from q38 import ops as module
    module.install()
    assert module.loaded_library() is not None and module.loaded_library().endswith("_C.so")
    yield module
    module.check_errors()


def rel_err(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-12)).item()


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 256, 576), (200, 72, 136), (1000, 2240, 576), (333, 21, 576), (4096, 576, 1344)])
def test_gemm_k_major(ops, M, N, K):
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    ref = a.float() @ b.float().t()
    out32 = ops.gemm(a, b, out_dtype=torch.float32)
    out16 = ops.gemm(a, b, out_dtype=torch.bfloat16)
    ops.check_errors()
    assert rel_err(out32, ref) < 1e-3
    assert rel_err(out16, ref) < 1e-2


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (200, 136, 72), (576, 2240, 16384), (288, 576, 1280)])
def test_gemm_mn_major_operands(ops, M, N, K):
    torch.manual_seed(1)
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    at, bt = a.t().contiguous(), b.t().contiguous()            # [K, M], [K, N]
    ref = a.float() @ b.float().t()
    nn = ops.gemm(a, bt, b_mn_major=True, out_dtype=torch.float32)
    tn = ops.gemm(at, bt, a_mn_major=True, b_mn_major=True, out_dtype=torch.float32)
    tk = ops.gemm(at, b, a_mn_major=True, out_dtype=torch.float32)
    ops.check_errors()
    assert rel_err(nn, ref) < 1e-3, "B MN-major"
    assert rel_err(tn, ref) < 1e-3, "A and B MN-major"
    assert rel_err(tk, ref) < 1e-3, "A MN-major"


def test_gemm_batched_accumulate_alpha(ops):
    torch.manual_seed(2)
    a = torch.randn(5, 288, 576, device="cuda").to(torch.bfloat16)
    b = torch.randn(5, 288, 576, device="cuda").to(torch.bfloat16)
    c = torch.randn(5, 288, 288, device="cuda")
    ref = c + 0.5 * torch.bmm(a.float(), b.float().transpose(1, 2))
    ops.gemm(a, b, out=c, alpha=0.5, accumulate=True)
    ops.check_errors()
    assert rel_err(c, ref) < 1e-3


@pytest.mark.parametrize("dim,in_dtype,out_dtype", [(576, torch.float32, torch.bfloat16), (64, torch.bfloat16, torch.bfloat16),
                                                    (448, torch.float32, torch.float32)])
def test_rmsnorm(ops, dim, in_dtype, out_dtype):
    from q38.ops.backend import _RMSNorm
    torch.manual_seed(3)
    x = torch.randn(777, dim, device="cuda").to(in_dtype).requires_grad_()
    w = (0.1 * torch.randn(dim, device="cuda")).requires_grad_()
    dy = torch.randn(777, dim, device="cuda").to(out_dtype)
    y = _RMSNorm.apply(x, w, 1e-6, out_dtype)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().clone().requires_grad_()
    yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-6) * (1 + wr)
    yr.backward(dy.float())
    assert rel_err(y, yr) < (1e-2 if out_dtype == torch.bfloat16 else 1e-5)
    assert rel_err(x.grad, xr.grad) < (2e-2 if in_dtype == torch.bfloat16 else 1e-4)
    assert rel_err(w.grad, wr.grad) < 1e-3


def test_gated_rmsnorm(ops):
    from q38.ops.backend import _GatedRMSNorm
    torch.manual_seed(4)
    x = torch.randn(1000, 64, device="cuda").to(torch.bfloat16).requires_grad_()
    g = torch.randn(1000, 64, device="cuda").to(torch.bfloat16).requires_grad_()
    w = (1 + 0.1 * torch.randn(64, device="cuda")).requires_grad_()
    dy = torch.randn(1000, 64, device="cuda").to(torch.bfloat16)
    y = _GatedRMSNorm.apply(x, g, w, 1e-6)
    y.backward(dy)
    xr, gr, wr = (t.detach().float().requires_grad_() for t in (x, g, w))
    yr = wr * (xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-6)) * torch.nn.functional.silu(gr)
    yr.backward(dy.float())
    assert rel_err(y, yr) < 2e-2 and rel_err(x.grad, xr.grad) < 3e-2 and rel_err(g.grad, gr.grad) < 3e-2
    assert rel_err(w.grad, wr.grad) < 1e-2


def test_adamw_flat_and_sum_squares(ops):
    torch.manual_seed(5)
    n = 100_003
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    ref = torch.nn.Parameter(p.clone())
    ref.grad = g.clone() * 0.5
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    shadow = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    scale = torch.tensor(0.5, device="cuda")
    for step in (1, 2, 3):
        opt.step()
        ops.adamw_flat(p, g, m, v, step, 1e-2, 0.1, 0.9, 0.95, 1e-8, grad_scale=scale, shadow=shadow)
    assert rel_err(p, ref.detach()) < 1e-5
    assert torch.equal(shadow, p.to(torch.bfloat16))
    assert abs(ops.sum_squares(g).item() / g.double().pow(2).sum().item() - 1) < 1e-6


def test_linear_autograd(ops):
    from q38.models import modeling
    backend = modeling.get_backend()
    torch.manual_seed(6)
    x = torch.randn(4, 96, 576, device="cuda").to(torch.bfloat16).requires_grad_()
    w = (0.05 * torch.randn(1344, 576, device="cuda")).requires_grad_()
    dy = torch.randn(4, 96, 1344, device="cuda").to(torch.bfloat16)
    y = backend.linear(x, w)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().clone().requires_grad_()
    yr = xr @ wr.to(torch.bfloat16).float().t()
    yr.backward(dy.float())
    assert rel_err(y, yr) < 1e-2 and rel_err(x.grad, xr.grad) < 1e-2 and rel_err(w.grad, wr.grad) < 1e-2
    assert w.grad.dtype == torch.float32


def test_muon_gpu_matches_reference(ops, monkeypatch):
    from q38.optim.muon import Muon
    torch.manual_seed(7)
    shapes = [(8, 32, 16), (48, 96), (6, 1, 4), (3, 288, 576)]
    fast = [torch.nn.Parameter(torch.randn(s, device="cuda")) for s in shapes]
    slow = [torch.nn.Parameter(p.detach().clone()) for p in fast]
    for p, q in zip(fast, slow):
        p.grad = torch.randn_like(p)
        q.grad = p.grad.clone()
    a, b = Muon(fast, lr=1e-3), Muon(slow, lr=1e-3)
    a.step()
    monkeypatch.setenv("Q38_MUON_BASELINE", "1")
    b.step()
    for p, q in zip(fast, slow):
        torch.testing.assert_close(p, q, rtol=1e-3, atol=2e-4)
        torch.testing.assert_close(a.state[p]["buf"], b.state[q]["buf"], rtol=0, atol=0)


@pytest.mark.parametrize("h,iters,dtype", [(128, 5, torch.bfloat16), (576, 20, torch.bfloat16), (64, 3, torch.float32)])
def test_mhc_sublayer_matches_specification(ops, h, iters, dtype):
    """pre -> (toy sub-layer) -> post through the fused kernels against the PyTorch mHC module, values and all gradients."""
    from q38.models import modeling
    backend = modeling.get_backend()
    torch.manual_seed(8)
    mhc = modeling.MHC(h, 4, max(1, round(h / 8)), slot=1, iters=iters).cuda()
    with torch.no_grad():
        mhc.B.weight.normal_(0, 0.3)
        mhc.alphas.fill_(0.7)
        mhc.b_res.add_(torch.randn(4, 4, device="cuda"))
    norm = modeling.Qwen3_8MoeRMSNorm(h).cuda()
    with torch.no_grad():
        norm.weight.normal_(0, 0.1)
    X = torch.randn(2, 96, 4, h, device="cuda")
    W = (torch.randn(h, h, device="cuda") / h ** 0.5)
    dXo = torch.randn(2, 96, 4, h, device="cuda")

    def run(fast):
        Xl = X.clone().requires_grad_()
        for p in list(mhc.parameters()) + list(norm.parameters()):
            p.grad = None
        if fast:
            x, state = backend.mhc_pre_norm(mhc, norm, Xl, dtype)
        else:
            xin, state = mhc.pre(Xl)
            x = norm(xin, out_dtype=dtype)
        y = (x.float() @ W).to(dtype)
        out = backend.mhc_post(mhc, y, state) if fast else mhc.post(y, state)
        out.backward(dXo)
        grads = {n: p.grad.clone() for n, p in list(mhc.named_parameters()) + [("norm", norm.weight)]}
        return x, out, Xl.grad, grads

    xa, oa, ga, pa = run(True)
    xb, ob, gb, pb = run(False)
    tol = 2e-2 if dtype == torch.bfloat16 else 2e-3          # the low-rank projection runs in tf32 (10-bit mantissa)
    assert rel_err(xa, xb) < tol and rel_err(oa, ob) < tol
    assert rel_err(ga, gb) < tol
    for name in pb:
        assert rel_err(pa[name], pb[name]) < 3 * tol, name


def test_moe_sort_is_a_stable_sort(ops):
    torch.manual_seed(9)
    T, k, E = 3000, 5, 64
    idx = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)]).to(torch.int32)
    idx[:500] = torch.tensor([3, 1, 4, 15, 9], dtype=torch.int32, device="cuda")          # heavy skew
    perm, inv, offsets, sched = ops.load().moe_sort(idx, E)
    order = torch.sort(idx.reshape(-1).long(), stable=True).indices
    assert torch.equal(perm.long(), order)
    assert torch.equal(inv.long()[order], torch.arange(T * k, device="cuda"))
    counts = torch.bincount(idx.reshape(-1).long(), minlength=E)
    assert torch.equal(offsets.long(), torch.cat([counts.new_zeros(1), counts.cumsum(0)]))
    n_tiles = int(sched[0])
    tiles = sched[1:1 + 3 * n_tiles].view(-1, 3)
    assert int(tiles[:, 2].sum()) == T * k and n_tiles == int(((counts + 127) // 128).sum())
    for e, row0, rows in tiles.tolist():
        assert offsets[e] <= row0 and row0 + rows <= offsets[e + 1] and 0 < rows <= 128


@pytest.mark.parametrize("T,h,f,E,k", [(700, 128, 32, 8, 2), (4096, 576, 144, 64, 5)])
def test_moe_block_matches_specification(ops, T, h, f, E, k):
    from types import SimpleNamespace
    from q38.models import modeling, RouterStats
    torch.manual_seed(10)
    cfg = SimpleNamespace(num_experts=E, num_experts_per_tok=k, hidden_size=h, moe_intermediate_size=f, shared_expert_intermediate_size=f)
    block = modeling.Qwen3_8MoeSparseMoeBlock(cfg).cuda().train()
    with torch.no_grad():
        for p in block.parameters():
            p.normal_(0, 0.05)
        block.gate.weight.normal_(0, 0.5)
    x = torch.randn(1, T, h, device="cuda").to(torch.bfloat16)
    dy = torch.randn(1, T, h, device="cuda").to(torch.bfloat16)
    backend = modeling.get_backend()

    def run(fast):
        modeling.set_backend(backend if fast else None)
        try:
            for p in block.parameters():
                p.grad = None
            xl = x.clone().requires_grad_()
            block.stats_sink = RouterStats(E)
            y = block(xl)
            aux = block.stats_sink.loss()
            block.stats_sink = None
            (y.float() * dy.float()).sum().add(aux * 3.0).backward()
            return y, aux, xl.grad, {n: p.grad.clone() for n, p in block.named_parameters()}
        finally:
            modeling.set_backend(backend)

    ya, auxa, gxa, pa = run(True)
    ops.check_errors()
    yb, auxb, gxb, pb = run(False)
    assert rel_err(ya, yb) < 3e-2 and abs(auxa.item() - auxb.item()) < 1e-2 * abs(auxb.item())
    assert rel_err(gxa, gxb) < 5e-2
    for name in pb:
        assert rel_err(pa[name], pb[name]) < 5e-2, name


@pytest.mark.parametrize("T,h,f,E,k", [(700, 128, 32, 8, 2), (4096, 576, 144, 64, 5), (3000, 320, 208, 16, 3)])
def test_persistent_grouped_kernels_match_the_one_tile_kernels(ops, T, h, f, E, k):
    """The persistent grouped expert GEMM (one CTA per SM, two TMEM accumulator sets) against the one-tile-per-CTA kernels and
    against an fp32 per-expert product, for the three epilogues."""
    raw = ops.load()
    torch.manual_seed(31)
    idx = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)]).to(torch.int32)
    perm, inv, offsets, sched = raw.moe_sort(idx, E)[:4]
    P = T * k
    rows = torch.randn(P, h, device="cuda").to(torch.bfloat16)
    wgu = (0.05 * torch.randn(E, 2 * f, h, device="cuda")).to(torch.bfloat16)
    wd = (0.05 * torch.randn(E, h, f, device="cuda")).to(torch.bfloat16)
    dy = torch.randn(P, h, device="cuda").to(torch.bfloat16)
    err = ops.error_flag()
    got = {}
    try:
        for mode in (1, 0):
            raw.moe_set_persistent(mode)
            hmid = torch.zeros(P, f, device="cuda", dtype=torch.bfloat16); gu = torch.zeros(P, 2 * f, device="cuda", dtype=torch.bfloat16)
            raw.moe_grouped_swiglu(rows, wgu, hmid, gu, sched, err)
            y = torch.zeros(P, h, device="cuda", dtype=torch.bfloat16)
            raw.moe_grouped_gemm(hmid, wd, y, sched, False, err)
            dgu = torch.zeros(P, 2 * f, device="cuda", dtype=torch.bfloat16)
            raw.moe_grouped_dswiglu(dy, wd, gu, dgu, sched, err)
            dx = torch.zeros(P, h, device="cuda", dtype=torch.bfloat16)
            raw.moe_grouped_gemm(dgu, wgu, dx, sched, True, err)
            gw = torch.zeros(E, 2 * f, h, device="cuda")
            for _ in range(2):                                   # the second pass accumulates onto the first
                raw.moe_grouped_wgrad(dgu, rows, gw, offsets, err)
            gd = torch.zeros(E, h, f, device="cuda")
            raw.moe_grouped_wgrad(dy, hmid, gd, offsets, err)
            got[mode] = (hmid, gu, y, dgu, dx, gw, gd)
    finally:
        raw.moe_set_persistent(-1)
    ops.check_errors()
    for a, b, name in zip(got[1], got[0], ("hmid", "gu", "y", "dgu", "dx", "grad gate_up", "grad down")):
        assert rel_err(a, b) < 1e-6, name
    off = offsets.tolist()
    ref_gw = torch.stack([got[1][3][off[e]:off[e + 1]].float().T @ rows[off[e]:off[e + 1]].float() for e in range(E)])
    assert rel_err(got[1][5], 2 * ref_gw) < 1e-3
    ref_gu = torch.zeros(P, 2 * f, device="cuda")
    for e in range(E):
        ref_gu[off[e]:off[e + 1]] = rows[off[e]:off[e + 1]].float() @ wgu[e].float().T
    assert rel_err(got[1][1], ref_gu) < 1e-2
    ref_h = torch.nn.functional.silu(ref_gu[:, :f]) * ref_gu[:, f:]
    assert rel_err(got[1][0], ref_h) < 2e-2


def test_moe_weight_gradients_accumulate_in_place(ops):
    from q38.ops.backend import _Experts
    torch.manual_seed(11)
    T, h, f, E, k = 900, 128, 32, 8, 2
    wgu = torch.nn.Parameter(0.05 * torch.randn(E, 2 * f, h, device="cuda"))
    wd = torch.nn.Parameter(0.05 * torch.randn(E, h, f, device="cuda"))
    x = torch.randn(T, h, device="cuda").to(torch.bfloat16)
    idx = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)]).to(torch.int32)
    w = torch.rand(T, k, device="cuda")
    out = _Experts.apply(x, w, idx, wgu, wd)
    out.float().sum().backward()
    first = (wgu.grad.clone(), wd.grad.clone())
    out = _Experts.apply(x, w, idx, wgu, wd)
    out.float().sum().backward()                      # second pass accumulates into the existing buffers
    ops.check_errors()
    assert rel_err(wgu.grad, 2 * first[0]) < 1e-5 and rel_err(wd.grad, 2 * first[1]) < 1e-5


@pytest.mark.parametrize("hybrid", [True, False])
@pytest.mark.parametrize("B,S,Hk,Hv", [(1, 128, 1, 2), (2, 512, 2, 6)])
def test_delta_rule_scan_matches_specification(ops, B, S, Hk, Hv, hybrid):
    from q38.models import modeling
    backend = modeling.get_backend()
    backend.hybrid_delta_rule = hybrid
    torch.manual_seed(12)
    q = torch.randn(B, S, Hk, 64, device="cuda").to(torch.bfloat16)
    k = torch.randn(B, S, Hk, 64, device="cuda").to(torch.bfloat16)
    v = torch.randn(B, S, Hv, 64, device="cuda").to(torch.bfloat16)
    g = -torch.rand(B, S, Hv, device="cuda") * 0.5
    beta = torch.rand(B, S, Hv, device="cuda").to(torch.bfloat16)
    do = torch.randn(B, S, Hv, 64, device="cuda").to(torch.bfloat16)

    def run(fast):
        leaves = [t.clone().requires_grad_() for t in (q, k, v, g, beta)]
        o = backend.delta_rule(*leaves) if fast else modeling.gated_delta_rule_chunked(*leaves)
        (o.float() * do.float()).sum().backward()
        return o, [t.grad for t in leaves]

    try:
        oa, ga = run(True)
    finally:
        backend.hybrid_delta_rule = False
    ops.check_errors()
    ob, gb = run(False)
    assert rel_err(oa, ob) < 3e-2
    for name, a, b in zip("q k v g beta".split(), ga, gb):
        assert rel_err(a, b) < 6e-2, name


def test_conv_silu(ops):
    from q38.models import modeling
    from q38.ops.backend import _ConvSilu
    torch.manual_seed(13)
    x = torch.randn(2, 200, 96, device="cuda").to(torch.bfloat16)
    w = (0.5 * torch.randn(96, 1, 4, device="cuda"))
    dy = torch.randn(2, 200, 96, device="cuda").to(torch.bfloat16)
    xa, wa = x.clone().requires_grad_(), w.clone().requires_grad_()
    ya = _ConvSilu.apply(xa, wa)
    ya.backward(dy)
    xb, wb = x.float().requires_grad_(), w.to(torch.bfloat16).float().requires_grad_()
    yb = modeling.causal_conv_silu(xb, wb)
    yb.backward(dy.float())
    assert rel_err(ya, yb) < 2e-2 and rel_err(xa.grad, xb.grad) < 2e-2 and rel_err(wa.grad, wb.grad) < 2e-2


@pytest.mark.parametrize("B,S,nq,nkv", [(1, 256, 4, 2), (2, 512, 6, 2)])
def test_indexer_kl_and_selection_match_specification(ops, B, S, nq, nkv):
    from q38.models import modeling
    backend = modeling.get_backend()
    torch.manual_seed(14)
    h = 128
    indexer = modeling.Indexer(h, 4, 64).cuda()
    x = torch.randn(B, S, h, device="cuda").to(torch.bfloat16)
    q = torch.randn(B, nq, S, 64, device="cuda").to(torch.bfloat16)
    k = torch.randn(B, nkv, S, 64, device="cuda").to(torch.bfloat16)
    cos, sin = modeling.rope_tables(torch.arange(S, device="cuda")[None], 16, 1e7, torch.float32)
    # specification (fp32 score pipeline of the model file)
    for p in indexer.parameters():
        p.grad = None
    modeling.set_backend(None)
    try:
        score = indexer(x, cos, sin)
        pos = torch.arange(S, device="cuda")
        lp = score.masked_fill(pos[None, :] > pos[:, None], -1e9).log_softmax(-1)
        lp_ref = lp.view(B, S, S // 64, 64).logsumexp(-1)
        P = modeling.block_mass(q, k, 0.125)
        kl_ref = torch.where(P > 0, P * (P.clamp(min=1e-12).log() - lp_ref), torch.zeros_like(P)).sum(-1).mean()
        (kl_ref * 7.0).backward()
        ref_grads = {n: p.grad.clone() for n, p in indexer.named_parameters()}
    finally:
        modeling.set_backend(backend)
    for p in indexer.parameters():
        p.grad = None
    kl, lp_blk = backend.indexer_block_logprobs(indexer, x, cos, sin, q, k, 0.125)
    (kl * 7.0).backward()
    ops.check_errors()
    assert abs(kl.item() - kl_ref.item()) < 2e-2 * abs(kl_ref.item()) + 1e-4, (kl.item(), kl_ref.item())
    causal = (torch.arange(S // 64, device="cuda")[None, :] <= (pos // 64)[:, None])
    assert (lp_blk - lp_ref)[:, causal].abs().max() < 5e-2
    for name, g in indexer.named_parameters():
        assert rel_err(g.grad, ref_grads[name]) < 8e-2, name
    count, index = ops.load().qsa_select(lp_blk, 3)
    c_ref, i_ref = modeling.select_blocks(lp_blk, 3)
    assert torch.equal(count, c_ref)
    slot = torch.arange(index.shape[-1], device="cuda")[None, None, :] < count[..., None]
    assert torch.equal(torch.where(slot, index, -1).sort(-1).values, torch.where(slot, i_ref, -1).sort(-1).values)


@pytest.mark.parametrize("M,N,K", [(300, 72, 2304), (256, 2304, 72), (72, 512, 4096)])
def test_gemm_tf32(ops, M, N, K):
    """fp32 operands consumed as tf32 by the tensor cores (K-major operands)."""
    torch.manual_seed(15)
    a, b = torch.randn(M, K, device="cuda"), torch.randn(N, K, device="cuda")
    got = ops.gemm(a, b, out_dtype=torch.float32)
    ops.check_errors()
    assert rel_err(got, a @ b.t()) < 3e-3            # 10-bit mantissa operands, fp32 accumulation


@pytest.mark.parametrize("splits", [0, 3, 7])
def test_gemm_split_k_accumulates(ops, splits):
    torch.manual_seed(17)
    a = torch.randn(4096, 64, device="cuda").to(torch.bfloat16)       # [K, M]: reduction over 4096 rows
    b = torch.randn(4096, 576, device="cuda").to(torch.bfloat16)
    c = torch.randn(64, 576, device="cuda")
    ref = c + a.float().t() @ b.float()
    ops.gemm(a, b, out=c, a_mn_major=True, b_mn_major=True, accumulate=True, splits=splits)
    ops.check_errors()
    assert rel_err(c, ref) < 1e-3


def test_fused_linear_cross_entropy(ops):
    from q38.models import modeling
    backend = modeling.get_backend()
    torch.manual_seed(18)
    T, h, V = 3000, 128, 10112
    hid = torch.randn(T, h, device="cuda").to(torch.bfloat16).requires_grad_()
    w = (0.1 * torch.randn(V, h, device="cuda")).requires_grad_()
    tgt = torch.randint(0, V, (T,), device="cuda")
    tgt[::7] = -100
    for reduction in ("mean", "sum"):
        hid.grad = w.grad = None
        loss = backend.linear_cross_entropy(w, hid, tgt, reduction)
        (loss * 0.37).backward()
        ops.check_errors()
        hr, wr = hid.detach().float().requires_grad_(), w.detach().to(torch.bfloat16).float().requires_grad_()
        ref = torch.nn.functional.cross_entropy(hr @ wr.t(), tgt, ignore_index=-100, reduction=reduction)
        (ref * 0.37).backward()
        assert abs(loss.item() - ref.item()) < 5e-3 * abs(ref.item())
        assert rel_err(hid.grad, hr.grad) < 3e-2 and rel_err(w.grad, wr.grad) < 3e-2


@pytest.mark.parametrize("M,N,K", [(16384, 2240, 576), (4096, 10112, 576), (20000, 80, 200)])
def test_gemm_persistent_many_tiles_per_cta(ops, M, N, K, monkeypatch):
    """More tiles than SMs: the smem ring and the two TMEM accumulators wrap around several times per CTA."""
    torch.manual_seed(11)
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    monkeypatch.setattr(ops, "PERSISTENT_GEMM", True)
    persistent = ops.gemm(a, b, out_dtype=torch.bfloat16)
    # weight-gradient shape: both operands MN-major views with a row stride, reduction over M, split-K into a zeroed fp32 buffer
    wgrad = torch.zeros(64, 72, device="cuda")
    ops.gemm(a[:, :64], a[:, :72], out=wgrad, a_mn_major=True, b_mn_major=True, accumulate=True, splits=0)
    monkeypatch.setattr(ops, "PERSISTENT_GEMM", False)
    single = ops.gemm(a, b, out_dtype=torch.bfloat16)
    ops.check_errors()
    ref = a.float() @ b.float().t()
    assert rel_err(persistent, ref) < 1e-2
    assert torch.equal(persistent, single)
    assert rel_err(wgrad, a[:, :64].float().t() @ a[:, :72].float()) < 1e-3


@pytest.mark.parametrize("out_features", [21, 1])
def test_linear_with_narrow_output(ops, out_features):
    """Per-head gate projections ([tokens, 21]) and the shared-expert gate ([tokens, 1]): their gradients have rows that are no
    multiple of 16 bytes and reach the tensor-core GEMM through padded-row views."""
    from q38.models import modeling
    backend = modeling.get_backend()
    torch.manual_seed(12)
    x = torch.randn(700, 576, device="cuda").to(torch.bfloat16).requires_grad_()
    w = (0.05 * torch.randn(out_features, 576, device="cuda")).requires_grad_()
    w.grad = torch.zeros_like(w)                                  # the trainer's arena provides the fp32 gradient buffer
    dy = torch.randn(700, out_features, device="cuda").to(torch.bfloat16)
    launches = ops.launch_count()
    y = backend.linear(x, w)
    y.backward(dy)
    assert ops.launch_count() - launches == 3                     # forward, dgrad and wgrad all ran on the extension's GEMM
    ops.check_errors()
    xr, wr = x.detach().float().requires_grad_(), w.detach().clone().requires_grad_()
    yr = xr @ wr.to(torch.bfloat16).float().t()
    yr.backward(dy.float())
    assert rel_err(y, yr) < 1e-2 and rel_err(x.grad, xr.grad) < 1e-2 and rel_err(w.grad, wr.grad) < 1e-2


def test_ngram_embedding_matches_specification(ops):
    """Hash rows (EOS-aware context), gather + RMSNorm forward, and the scatter-add backward against the PyTorch module."""
    from q38.models import modeling
    backend = modeling.get_backend()
    torch.manual_seed(13)
    h, vocab, rows, eos = 128, 1000, 4099, 7
    m = modeling.NGramEmbedding(h, vocab, rows, eos).cuda()
    with torch.no_grad():
        m.norm.weight.normal_(1.0, 0.2)
    ids = torch.randint(0, vocab, (3, 257), device="cuda")
    ids[:, ::23] = eos
    ids[0, :3] = torch.tensor([eos, 5, eos])
    hid = torch.randn(3, 257, h, device="cuda").to(torch.bfloat16)
    dout = torch.randn(3, 257, h, device="cuda").to(torch.bfloat16)
    _, _, got_rows = ops.load().ngram_fwd(ids, m.emb2.weight, m.emb3.weight, m.norm.weight.float(), vocab, eos, 1e-6)
    i2, i3 = m.indices(ids)
    assert torch.equal(got_rows[..., 0].long(), i2) and torch.equal(got_rows[..., 1].long(), i3)

    def run(fast):
        for p in m.parameters():
            p.grad = None
        hx = hid.clone().requires_grad_()
        out = backend.ngram_delta(m, hx, ids) if fast else m.delta(hx.float(), ids)
        out.backward(dout if fast else dout.float())
        return out, hx.grad, {n: p.grad.clone() for n, p in m.named_parameters()}

    modeling.set_backend(None)
    try:
        ref_out, ref_dh, ref_g = run(False)
    finally:
        modeling.set_backend(backend)
    out, dh, g = run(True)
    assert rel_err(out, ref_out) < 2e-2 and rel_err(dh, ref_dh) < 2e-2
    for name in ref_g:
        assert rel_err(g[name], ref_g[name]) < 2e-2, name


@pytest.mark.parametrize("with_norm,split", [(True, True), (True, False), (False, False)])
def test_qsa_head_preparation(ops, with_norm, split):
    """Per-head zero-centred RMSNorm + partial RoPE + move to [B,H,S,64] (+ gate split) in one kernel, values and gradients."""
    from q38.models import modeling
    from q38.ops.backend import _head_prep
    torch.manual_seed(14)
    B, S, H = 2, 192, 5
    width = 128 if split else 64
    src = torch.randn(B, S, H, width, device="cuda").to(torch.bfloat16)
    norm = modeling.Qwen3_8MoeRMSNorm(64).cuda() if with_norm else None
    if norm is not None:
        with torch.no_grad():
            norm.weight.normal_(0, 0.2)
    cos, sin = modeling.rope_tables(torch.arange(S, device="cuda")[None], 16, 1e7, torch.float32)
    dq = torch.randn(B, H, S, 64, device="cuda").to(torch.bfloat16)
    dg = torch.randn(B, S, H * 64, device="cuda").to(torch.bfloat16)

    def run(fast):
        x = src.clone().requires_grad_()
        if norm is not None:
            norm.weight.grad = None
        if fast:
            q, gate = _head_prep(x, norm, cos, sin)
        else:
            backend = modeling.get_backend()
            modeling.set_backend(None)
            try:
                xf = x.float()
                q = xf[..., :64]
                q = norm(q) if norm is not None else q
                q = modeling.apply_rope(q.transpose(1, 2), cos, sin)
                gate = xf[..., 64:].reshape(B, S, -1) if split else None
            finally:
                modeling.set_backend(backend)
        loss = (q.float() * dq.float()).sum() + ((gate.float() * dg.float()).sum() if split else 0.0)
        loss.backward()
        return q, gate, x.grad, (norm.weight.grad.clone() if norm is not None else None)

    qa, ga, dxa, dwa = run(True)
    qb, gb, dxb, dwb = run(False)
    assert qa.shape == (B, H, S, 64) and rel_err(qa, qb) < 1e-2
    assert rel_err(dxa, dxb) < 2e-2
    if split:
        assert torch.equal(ga.float(), gb.float().to(torch.bfloat16).float())
    if with_norm:
        assert rel_err(dwa, dwb) < 2e-2


def test_gdn_gates(ops):
    """beta = sigmoid(b), g = -exp(A_log) softplus(a + dt_bias) and their gradients (incl. the per-head parameter sums)."""
    from q38.ops.backend import _GdnGates
    torch.manual_seed(15)
    T, H = 1000, 21
    b = torch.randn(2, T // 2, H, device="cuda").to(torch.bfloat16)
    a = (3 * torch.randn(2, T // 2, H, device="cuda")).to(torch.bfloat16)
    a[0, 0, 0] = 30.0                                            # softplus linear branch
    A_log = torch.randn(H, device="cuda").requires_grad_()
    dt_bias = torch.randn(H, device="cuda").requires_grad_()
    dbeta = torch.randn_like(b)
    dg = torch.randn(2, T // 2, H, device="cuda")

    def run(fast):
        bb, aa = b.clone().requires_grad_(), a.clone().requires_grad_()
        A_log.grad = dt_bias.grad = None
        if fast:
            beta, g = _GdnGates.apply(bb, aa, A_log, dt_bias)
        else:
            beta = bb.float().sigmoid()
            g = -A_log.float().exp() * torch.nn.functional.softplus(aa.float() + dt_bias.float())
        (beta.float() * dbeta.float()).sum().backward(retain_graph=True)
        (g * dg).sum().backward()
        return beta, g, bb.grad, aa.grad, A_log.grad.clone(), dt_bias.grad.clone()

    got, ref = run(True), run(False)
    for x, y, tol in zip(got, ref, (1e-2, 1e-5, 2e-2, 2e-2, 1e-3, 1e-3)):
        assert rel_err(x, y) < tol


def _masked_attention_reference(q, k, v, count, index, scale):
    """fp32 masked-softmax attention over the selected blocks (dense causal when count is None): q [B,nq,S,64], k/v [B,nkv,S,64]."""
    from q38.models import modeling
    B, nq, S, _ = q.shape
    rep = nq // k.shape[1]
    kf, vf = k.float().repeat_interleave(rep, 1), v.float().repeat_interleave(rep, 1)
    s = (q.float() @ kf.transpose(-1, -2)) * scale
    if count is None:
        mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()[None].expand(B, -1, -1)
    else:
        mask = modeling.block_sparse_mask(count, index, S)
    s = s.masked_fill(~mask[:, None], float("-inf"))
    return (s.softmax(-1) @ vf).transpose(1, 2)           # [B,S,nq,64]


@pytest.mark.parametrize("B,S,nq,nkv,budget", [(1, 256, 4, 2, None), (2, 512, 22, 2, None), (2, 512, 22, 2, 1), (1, 1024, 6, 2, 3),
                                                (1, 1024, 4, 2, 8), (1, 256, 4, 1, 8)])
def test_block_attention_forward_and_gradients(ops, B, S, nq, nkv, budget):
    """Isolated check of the block-sparse / dense attention kernels: dense, budgets 1 / 3 / 8, fewer blocks than the budget, GQA 11:1."""
    from q38.models import modeling
    from q38.ops.backend import _BlockAttention
    torch.manual_seed(31)
    q = torch.randn(B, nq, S, 64, device="cuda").to(torch.bfloat16).requires_grad_()
    k = torch.randn(B, nkv, S, 64, device="cuda").to(torch.bfloat16).requires_grad_()
    v = torch.randn(B, nkv, S, 64, device="cuda").to(torch.bfloat16).requires_grad_()
    do = torch.randn(B, S, nq, 64, device="cuda").to(torch.bfloat16)
    count = index = None
    if budget is not None:
        nb = S // 64
        lp = torch.randn(B, nb, nb, device="cuda").log_softmax(-1)
        count, index = modeling.select_blocks(lp, budget)
        count, index = count.contiguous(), index.contiguous()
    out = _BlockAttention.apply(q, k, v, count, index, 0.125)
    out.backward(do)
    ops.check_errors()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = _masked_attention_reference(qr, kr, vr, count, index, 0.125)
    ref.backward(do.float())
    assert rel_err(out, ref) < 2e-2
    assert rel_err(q.grad, qr.grad) < 2e-2 and rel_err(k.grad, kr.grad) < 2e-2 and rel_err(v.grad, vr.grad) < 2e-2


def test_elementwise_gates_match_specification(ops):
    from q38.ops.backend import _GateAdd, _SigmoidMul, _SwiGLU
    torch.manual_seed(32)
    T, h = 777, 576
    bf = lambda *shape: torch.randn(*shape, device="cuda").to(torch.bfloat16).requires_grad_()
    fp = lambda t: t.detach().float().requires_grad_()
    dy = torch.randn(T, h, device="cuda").to(torch.bfloat16)
    g, u = bf(T, h), bf(T, h)
    _SwiGLU.apply(g, u).backward(dy)
    gr, ur = fp(g), fp(u)
    ref = torch.nn.functional.silu(gr) * ur
    ref.backward(dy.float())
    assert rel_err(_SwiGLU.apply(g, u), ref) < 1e-2 and rel_err(g.grad, gr.grad) < 1e-2 and rel_err(u.grad, ur.grad) < 1e-2
    x, gate = bf(T, h), bf(T, h)
    _SigmoidMul.apply(x, gate).backward(dy)
    xr, gater = fp(x), fp(gate)
    ref = xr * torch.sigmoid(gater)
    ref.backward(dy.float())
    assert rel_err(_SigmoidMul.apply(x, gate), ref) < 1e-2 and rel_err(x.grad, xr.grad) < 1e-2 and rel_err(gate.grad, gater.grad) < 1e-2
    routed, shared, logit = bf(T, h), bf(T, h), bf(T, 1)
    _GateAdd.apply(routed, shared, logit).backward(dy)
    rr, sr, lr_ = fp(routed), fp(shared), fp(logit)
    ref = rr + torch.sigmoid(lr_) * sr
    ref.backward(dy.float())
    assert rel_err(_GateAdd.apply(routed, shared, logit), ref) < 1e-2
    assert rel_err(routed.grad, rr.grad) < 1e-2 and rel_err(shared.grad, sr.grad) < 1e-2 and rel_err(logit.grad, lr_.grad) < 2e-2


def test_embedding_gradient_scatter(ops):
    torch.manual_seed(33)
    V, h = 1000, 96
    ids = torch.randint(0, V, (4, 300), device="cuda")
    ids[0, :50] = 5                                           # many hits on one row
    dout = torch.randn(4, 300, h, device="cuda")
    grad = torch.ones(V, h, device="cuda")                    # accumulates into what is there
    ops.load().embed_bwd(ids.contiguous(), dout.contiguous(), grad)
    ref = torch.ones(V, h, device="cuda").index_add_(0, ids.view(-1), dout.view(-1, h))
    torch.testing.assert_close(grad, ref, rtol=1e-5, atol=1e-4)


def test_cross_entropy_kernel_with_ignored_rows(ops):
    torch.manual_seed(34)
    rows, V = 300, 10112
    logits = torch.randn(rows, V, device="cuda").to(torch.bfloat16)
    target = torch.randint(0, V, (rows,), device="cuda")
    target[::3] = -100
    for all_ignored in (False, True):
        t = torch.full_like(target, -100) if all_ignored else target
        work = logits.clone()
        loss = ops.load().ce_inplace(work, t)
        ref = torch.nn.functional.cross_entropy(logits.float(), t, ignore_index=-100, reduction="none")
        torch.testing.assert_close(loss.float(), ref, rtol=2e-3, atol=2e-3)
        grad_ref = torch.softmax(logits.float(), -1)
        valid = t != -100
        grad_ref[valid, t[valid]] -= 1.0
        grad_ref[~valid] = 0.0
        assert (work.float() - grad_ref).abs().max() < 1e-2
        assert work[~valid].abs().max() == 0                  # ignored rows contribute neither loss nor gradient


@pytest.mark.parametrize("B,S,nq,nkv", [(1, 128, 2, 1), (2, 512, 6, 2), (1, 1024, 22, 2), (1, 384, 4, 2)])
def test_block_statistics_on_tcgen05_match_fp32(ops, B, S, nq, nkv):
    """Per (query, key block) max and sum-exp of the main attention scores from the tcgen05 kernel against an fp32 evaluation
    and against the warp-MMA kernel it replaces."""
    torch.manual_seed(35)
    q = (2.0 * torch.randn(B, nq, S, 64, device="cuda")).to(torch.bfloat16)
    k = torch.randn(B, nkv, S, 64, device="cuda").to(torch.bfloat16)
    lib = ops.load()
    got = lib.qsa_block_stats_tc(q, k, 0.125, ops.error_flag(q.device))
    old = lib.qsa_main_block_stats(q, k, 0.125)
    ops.check_errors()
    nb = S // 64
    scores = (q.float() @ k.float().repeat_interleave(nq // nkv, 1).transpose(-1, -2)) * 0.125
    pos = torch.arange(S, device="cuda")
    scores = scores.masked_fill(pos[None, :] > pos[:, None], float("-inf")).view(B, nq, S, nb, 64)
    ref_max = scores.max(-1).values
    ref_sum = (scores - ref_max.clamp_min(-1e30)[..., None]).exp().sum(-1)
    causal = (torch.arange(nb, device="cuda")[None, :] <= (pos // 64)[:, None]).expand(B, nq, S, nb)
    for name, stats in (("tcgen05", got), ("warp", old)):
        assert (stats[..., 0] - ref_max)[causal].abs().max() < 2e-3, name
        assert ((stats[..., 1] - ref_sum)[causal].abs() / ref_sum[causal]).max() < 2e-3, name


@pytest.mark.parametrize("B,S,NI", [(1, 128, 4), (2, 1024, 4), (1, 4096, 2)])
def test_first_query_indexer_log_probabilities(ops, B, S, NI):
    """Block log-probabilities of the indexer for the first query of every block (the selection-only path of evaluation) against
    the specification: scores of those queries, causal mask, log-softmax over keys, log-sum-exp per 64-key block."""
    torch.manual_seed(41)
    nb = S // 64
    qi = torch.randn(B, NI, S, 64, device="cuda").to(torch.bfloat16)
    ki = torch.randn(B, S, 64, device="cuda").to(torch.bfloat16)
    wi = torch.rand(B, S, NI, device="cuda") * NI ** -0.5
    got = ops.load().qsa_first_query_lp(qi[:, :, ::64].contiguous(), ki, wi[:, ::64].contiguous(), 0.125)
    ops.check_errors()
    scores = torch.matmul(qi[:, :, ::64].float(), ki[:, None].float().transpose(-1, -2)).to(torch.bfloat16).float()      # [B,NI,nb,S], bf16 like the matmul output
    score = torch.einsum("bhts,bth->bts", torch.relu(scores) * 0.125, wi[:, ::64])
    pos = torch.arange(S, device="cuda")
    score = score.masked_fill(pos[None, :] > pos[::64][:, None], -1e9)
    ref = score.log_softmax(-1).view(B, nb, nb, 64).logsumexp(-1)
    causal = torch.ones(nb, nb, device="cuda").tril().bool()
    assert (got - ref)[:, causal].abs().max().item() < 2e-3
    assert (got[:, ~causal] < -1e8).all()


@pytest.mark.parametrize("M,N,K,batch", [(512, 256, 128, 1), (4096, 2240, 576, 1), (1000, 200, 72, 1), (768, 96, 320, 3)])
def test_gemm_on_sm_pairs(ops, M, N, K, batch):
    """The cta_group::2 kernel (two CTAs per 256-row tile, each loading half of B) against the fp32 product, for bf16 and fp32
    outputs, a scale factor, ragged edges, batches and accumulation into a bf16 output."""
    torch.manual_seed(43)
    lib, err = ops.load(), ops.error_flag()
    a = (0.1 * torch.randn(batch, M, K, device="cuda")).to(torch.bfloat16)
    b = (0.1 * torch.randn(batch, N, K, device="cuda")).to(torch.bfloat16)
    ref = torch.matmul(a.float(), b.float().transpose(1, 2))
    out = torch.empty(batch, M, N, device="cuda", dtype=torch.bfloat16)
    assert lib.gemm_pair(a, b, out, 1.0, False, err)
    out32 = torch.empty(batch, M, N, device="cuda", dtype=torch.float32)
    assert lib.gemm_pair(a, b, out32, 0.5, False, err)
    before = out.clone()
    assert lib.gemm_pair(a, b, out, 1.0, True, err)
    ops.check_errors()
    assert rel_err(before, ref) < 5e-3 and rel_err(out32, 0.5 * ref) < 1e-5
    assert rel_err(out, before.float() + ref) < 5e-3
    small = torch.empty(1, 128, 64, device="cuda", dtype=torch.bfloat16)
    assert not lib.gemm_pair(a[:1, :128], b[:1, :64], small, 1.0, False, err)          # fewer than 256 rows: left to the one-CTA kernel


def test_gemm_accumulates_into_bf16_output(ops):
    """`out += A B^T` with a bf16 output: the epilogue hands the tile to the TMA unit, which adds it in bf16."""
    torch.manual_seed(36)
    a = (0.1 * torch.randn(1000, 288, device="cuda")).to(torch.bfloat16)
    w = (0.1 * torch.randn(288, 576, device="cuda")).to(torch.bfloat16)            # [K, N]: MN-major B, as in an input-gradient product
    out = torch.randn(1000, 576, device="cuda").to(torch.bfloat16)
    before = out.clone()
    ops.gemm(a, w, out=out, b_mn_major=True, accumulate=True)
    ref = before.float() + a.float() @ w.float()
    assert rel_err(out, ref) < 1e-2
