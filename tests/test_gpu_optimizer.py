"""Optimizer-side kernels on a B200: the fused Muon step on flat arenas, the GEMM addend epilogue that carries the
Newton-Schulz polynomial, the tiny-matrix Newton-Schulz kernel, the shadow cast, and the rule that every kernel that writes
parameters or optimizer state returns without writing once the device error word is set."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from q38 import ops as module
    module.install()
    yield module
    module.check_errors()


def rel_err(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-12)).item()


def fro_err(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


# Newton-Schulz runs in bf16 and each iteration amplifies a last-bit difference of its input a few times, so two correct
# bf16 evaluations with different rounding points (the kernels round G, the polynomial and the update once each; the PyTorch
# chain rounds after every elementwise op) differ by a few per cent.  The yardstick is therefore the exact (fp64) iteration:
# a kernel may be at most twice as far from it as the PyTorch bf16 chain is (with a floor of 2 %).
def exact_newton_schulz(x, steps=5):
    a, b, c = 3.4445, -4.7750, 2.0315
    X = x.double()
    wide = X.shape[-2] <= X.shape[-1]
    if not wide:
        X = X.transpose(-2, -1)
    for _ in range(steps):
        G = X @ X.transpose(-2, -1)
        X = a * X + (b * G + c * (G @ G)) @ X
    return (X if wide else X.transpose(-2, -1)).float()


def ns_close(got, bf16_chain, exact):
    allowed = max(2.0 * fro_err(bf16_chain, exact), 2e-2)
    return fro_err(got, exact) <= allowed, (fro_err(got, exact), fro_err(bf16_chain, exact))


@pytest.mark.parametrize("batch,M,N,K,a_mn,b_mn", [(3, 96, 96, 96, False, False), (2, 288, 576, 288, False, True), (5, 576, 144, 144, False, False),
                                                   (4, 144, 144, 576, True, True), (1, 200, 72, 136, False, False)])
def test_gemm_addend_epilogue(ops, batch, M, N, K, a_mn, b_mn):
    torch.manual_seed(1)
    a = torch.randn(batch, K, M, device="cuda") if a_mn else torch.randn(batch, M, K, device="cuda")
    b = torch.randn(batch, K, N, device="cuda") if b_mn else torch.randn(batch, N, K, device="cuda")
    a, b = (0.1 * a).to(torch.bfloat16), (0.1 * b).to(torch.bfloat16)
    cin = torch.randn(batch, M, N, device="cuda").to(torch.bfloat16)
    out = ops.gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn, alpha=2.0315, addend=cin, beta=-4.775)
    af = a.float().transpose(1, 2) if a_mn else a.float()
    bf = b.float() if b_mn else b.float().transpose(1, 2)
    ref = 2.0315 * (af @ bf) - 4.775 * cin.float()
    assert rel_err(out, ref) < 1e-2
    plain = ops.gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn, alpha=0.5)          # the addend is optional
    assert rel_err(plain, 0.5 * (af @ bf)) < 1e-2


def reference_muon(param, grad, buf, lr, momentum, wd, rms_scale, steps, grad_scale):
    """PyTorch statement of one Muon update of a stack ``[n, rows, cols]`` (q38.optim.muon arithmetic): returns the new
    parameters with the bf16 chain, the new parameters with the exact iteration on the same normalised bf16 input, and buf."""
    from q38.optim.muon import newton_schulz
    g = grad * grad_scale
    buf = momentum * buf + g
    update = g + momentum * buf
    scale = rms_scale * max(param.shape[-2], param.shape[-1]) ** 0.5
    X = update.to(torch.bfloat16)
    X = X / X.flatten(-2).norm(dim=-1).clamp(min=1e-7)[..., None, None]
    decayed = param * (1 - lr * wd)
    return decayed - lr * scale * newton_schulz(update, steps).float(), decayed - lr * scale * exact_newton_schulz(X, steps), buf


def test_fused_muon_arena_step_matches_reference(ops):
    from q38.ops.muon_gpu import FusedMuon
    torch.manual_seed(2)
    shapes = [(8, 48, 96), (8, 96, 24), (64, 1, 4), (2, 4, 96), (3, 24, 72), (1, 96, 96), (2, 288, 576), (5, 48, 96), (1, 20, 50)]
    entries, cursor = [], 64
    for n, rows, cols in shapes:
        entries.append((cursor, n, rows, cols))
        cursor = (cursor + n * rows * cols + 63) // 64 * 64
    numel = cursor + 128
    params = torch.randn(numel, device="cuda")
    grads = torch.randn(numel, device="cuda")
    buf = 0.3 * torch.randn(numel, device="cuda")
    shadow = torch.zeros(numel, device="cuda", dtype=torch.bfloat16)
    before = params.clone()
    expected = {}
    for (offset, n, rows, cols) in entries:
        view = lambda t: t[offset:offset + n * rows * cols].view(n, rows, cols).clone()
        expected[offset] = reference_muon(view(params), view(grads), view(buf), 1e-2, 0.95, 0.1, 0.2, 5, 0.5)
    plan = FusedMuon(params, grads, buf, shadow, entries)
    err = ops.error_flag(params.device)
    hyper = torch.tensor([1e-2, 0.0, 0.0, 0.0], device="cuda")
    plan.step(lr=123.0, momentum=0.95, weight_decay=0.1, grad_scale=torch.tensor(0.5, device="cuda"), hyper=hyper, err=err)
    touched = torch.zeros(numel, dtype=torch.bool, device="cuda")
    for (offset, n, rows, cols) in entries:
        size = n * rows * cols
        new_p, exact_p, new_buf = expected[offset]
        old = before[offset:offset + size].view(n, rows, cols)
        got = params[offset:offset + size].view(n, rows, cols)
        ok, detail = ns_close(got - old, new_p - old, exact_p - old)        # compare the applied steps
        assert ok, (rows, cols, detail)
        torch.testing.assert_close(buf[offset:offset + size].view(n, rows, cols), new_buf, rtol=1e-6, atol=1e-6)
        assert torch.equal(shadow[offset:offset + size], params[offset:offset + size].to(torch.bfloat16))
        touched[offset:offset + size] = True
    assert torch.equal(params[~touched], before[~touched]), "elements outside the listed matrices were modified"
    # a second step reuses the tables and the cleared sums of squares
    plan.step(lr=1e-2, momentum=0.95, weight_decay=0.1, err=err)
    assert torch.isfinite(params).all()


def test_small_newton_schulz_kernel(ops):
    from q38.optim.muon import newton_schulz
    torch.manual_seed(3)
    for n, rows, cols in ((40, 1, 4), (6, 4, 576), (5, 96, 8), (3, 7, 33)):
        x = torch.randn(n, rows, cols, device="cuda")
        x = (x / x.flatten(1).norm(dim=1)[:, None, None]).to(torch.bfloat16).contiguous()
        out = torch.empty_like(x)
        ops.load().muon_small_ns(x, out, rows, cols, 5, None)
        ref = newton_schulz(x.float().cpu(), 5).float().cuda()
        ok, detail = ns_close(out, ref, exact_newton_schulz(x))
        assert ok, (rows, cols, detail)


def test_cast_shadow_except(ops):
    params = torch.randn(4096 * 3, device="cuda")
    shadow = torch.full((4096 * 3,), 7.0, device="cuda", dtype=torch.bfloat16)
    ops.load().cast_shadow_except(params, shadow, 4096, 2048, None)
    expect = params.to(torch.bfloat16)
    expect[4096:6144] = 7.0
    assert torch.equal(shadow, expect)


def test_update_kernels_write_nothing_when_the_error_word_is_set(ops):
    """What a rank does after a peer missed a barrier: the error word is set and every kernel of the step that writes
    parameters, moments, the shadow or peer memory must return without writing.  (The word is set from the host here.)"""
    from q38.ops.muon_gpu import FusedMuon
    torch.manual_seed(4)
    err = ops.error_flag(torch.device("cuda", torch.cuda.current_device()))
    n = 8 * 48 * 96
    params, grads, buf = torch.randn(n + 64, device="cuda"), torch.randn(n + 64, device="cuda"), torch.randn(n + 64, device="cuda")
    shadow = torch.zeros(n + 64, device="cuda", dtype=torch.bfloat16)
    m, v = torch.zeros(n + 64, device="cuda"), torch.zeros(n + 64, device="cuda")
    plan = FusedMuon(params, grads, buf, shadow, [(0, 8, 48, 96)])
    snapshot = [t.clone() for t in (params, buf, shadow, m, v)]
    err.fill_(4)
    try:
        plan.step(lr=1e-2, momentum=0.95, weight_decay=0.1, err=err)
        ops.adamw_flat(params, grads, m, v, 1, 1e-2, 0.1, 0.9, 0.95, 1e-8, shadow=shadow, err=err)
        ops.load().cast_shadow_except(params, shadow, 0, 0, err)
        ops.load().p2p_all_gather(params, None, [params.data_ptr()], [], 0, 0, n, err)
        torch.cuda.synchronize()
        for now, then in zip((params, buf, shadow, m, v), snapshot):
            assert torch.equal(now, then)
        with pytest.raises(RuntimeError, match="peer flag"):
            ops.check_errors()
    finally:
        err.zero_()
    plan.step(lr=1e-2, momentum=0.95, weight_decay=0.1, err=err)                 # with the word cleared the same calls update
    assert not torch.equal(params, snapshot[0])
