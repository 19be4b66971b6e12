"""Block-scaled MXFP8 expert path on a B200: quantisation kernels and the grouped tcgen05 GEMM of kind mxf8f6f4.block_scale.

The oracle decodes the kernels' own E4M3 bytes and E8M0 scales in PyTorch and multiplies in fp32, so a wrong scale-factor
arrangement in tensor memory (the part of the format no compiler checks) shows up as an O(1) error, while the comparison with
the unquantised product bounds the quantisation error itself."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from q38 import ops as module
    module.install()
    yield module
    module.check_errors()


def decode_scales(sf, tiles, blocks_per_tile, chunks, rows_per_tile, nblocks):
    """Tile-major scale bytes -> float [tiles, rows_per_tile, nblocks] (2^(byte - 127))."""
    sf = sf.view(tiles, blocks_per_tile, chunks, 512).long()
    r = torch.arange(rows_per_tile, device=sf.device)
    kb = torch.arange(nblocks, device=sf.device)
    block, rin = r // 128, r % 128
    offset = (rin % 32)[:, None] * 16 + (rin // 32)[:, None] * 4 + (kb % 4)[None, :]
    picked = sf[:, block[:, None].expand(-1, nblocks), (kb // 4)[None, :].expand(rows_per_tile, -1), offset]
    return torch.exp2(picked.float() - 127.0)


def dequant(q, scales_per_row):
    """q uint8 [R, K] (e4m3), scales [R, ceil(K/32)] -> fp32 [R, K]."""
    vals = q.view(torch.float8_e4m3fn).float()
    K = q.shape[1]
    return vals * scales_per_row.repeat_interleave(32, dim=1)[:, :K]


@pytest.mark.parametrize("T,k,E,K,N", [(128, 1, 1, 128, 128), (700, 2, 8, 576, 288), (2048, 5, 64, 144, 576), (300, 2, 4, 288, 576)])
def test_mxfp8_grouped_gemm_matches_dequantised_product(ops, T, k, E, K, N):
    lib = ops.load()
    torch.manual_seed(41)
    x = torch.randn(T, K, device="cuda").to(torch.bfloat16)
    w = (0.05 * torch.randn(E, N, K, device="cuda"))
    idx = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)]).to(torch.int32).contiguous()
    perm, inv, offsets, sched = lib.moe_sort(idx, E)
    P = T * k
    bn = int(lib.mxfp8_pick_bn(N))
    aq, sfa = lib.mxfp8_quantize_rows(x, perm, k, sched, P)
    wq, sfw = lib.mxfp8_quantize_weight(w, bn)
    out = torch.zeros(P, N, dtype=torch.bfloat16, device="cuda")
    lib.mxfp8_grouped_gemm(aq, sfa, wq, sfw, out, sched, bn, ops.error_flag(x.device))
    ops.check_errors()
    # decode: activations by schedule tile, weights by (expert, N tile)
    nblocks, chunks = (K + 31) // 32, (K + 127) // 128
    sched_host = sched.tolist()
    ntiles, max_tiles = sched_host[0], (len(sched_host) - 1) // 3
    a_scales = decode_scales(sfa, max_tiles, 1, chunks, 128, nblocks)
    row_scale = torch.ones(P, nblocks, device="cuda")
    expert_of_row = torch.zeros(P, dtype=torch.long, device="cuda")
    for t in range(ntiles):
        e, row0, rows = sched_host[1 + 3 * t: 4 + 3 * t]
        row_scale[row0:row0 + rows] = a_scales[t, :rows]
        expert_of_row[row0:row0 + rows] = e
    a_deq = dequant(aq, row_scale)
    tiles_n = (N + bn - 1) // bn
    w_scales = decode_scales(sfw, E * tiles_n, 1, chunks, 128, nblocks).view(E, tiles_n, 128, nblocks)[:, :, :bn].reshape(E, tiles_n * bn, nblocks)[:, :N]
    w_deq = dequant(wq.view(E * N, K), w_scales.reshape(E * N, nblocks)).view(E, N, K)
    ref = torch.einsum("pk,pnk->pn", a_deq, w_deq[expert_of_row])
    err = ((out.float() - ref).abs().max() / ref.abs().max()).item()
    assert err < 1e-2, f"kernel vs dequantised operands: {err}"
    # quantisation error against the bf16 operands
    xs = x[(perm.long() // k)].float()
    exact = torch.einsum("pk,pnk->pn", xs, w.to(torch.bfloat16).float()[expert_of_row])
    rel = ((ref - exact).norm() / exact.norm()).item()
    assert rel < 5e-2, f"quantisation error {rel}"
    # the quantiser never saturates and reproduces the operands to E4M3 precision
    assert ((a_deq - xs).abs().max() / xs.abs().max()).item() < 0.07


def test_fp8_expert_block_tracks_the_bf16_block(ops):
    """Forward and every gradient of the MXFP8 expert path against the bf16 expert path on the same inputs."""
    from q38.ops.backend import WGRAD_STREAM, _Experts, _bf16_weight
    from q38.ops.fp8 import ExpertsFP8
    torch.manual_seed(42)
    T, h, f, E, k = 1500, 576, 144, 64, 5
    x = torch.randn(T, h, device="cuda").to(torch.bfloat16)
    top_idx = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)]).to(torch.int32).contiguous()
    top_w = torch.softmax(torch.randn(T, k, device="cuda"), -1)
    dout = torch.randn(T, h, device="cuda").to(torch.bfloat16)
    results = []
    for fn, extra in ((_Experts, ()), (ExpertsFP8, (_bf16_weight, WGRAD_STREAM))):
        xi = x.clone().requires_grad_()
        tw = top_w.clone().requires_grad_()
        wgu = (0.04 * torch.randn(E, 2 * f, h, device="cuda", generator=torch.Generator("cuda").manual_seed(1))).requires_grad_()
        wd = (0.04 * torch.randn(E, h, f, device="cuda", generator=torch.Generator("cuda").manual_seed(2))).requires_grad_()
        out = fn.apply(xi, tw, top_idx, wgu, wd, *extra)
        out.backward(dout)
        WGRAD_STREAM.join()
        ops.check_errors()
        results.append((out.detach().float(), xi.grad.float(), tw.grad.float(), wgu.grad.float(), wd.grad.float()))
    for name, a, b in zip(("out", "dx", "d_top_w", "d_gate_up", "d_down"), results[1], results[0]):
        # E4M3 keeps three mantissa bits: about 3 % RMS error per quantised operand, two chained products in the forward
        rel = ((a - b).norm() / b.norm()).item()
        assert rel < 1e-1, (name, rel)


def test_training_with_fp8_experts_follows_the_bf16_run(ops):
    """30 optimizer steps of a small model with --fp8_ffn 1 and 0 from the same weights and data: the loss curves stay together."""
    from types import SimpleNamespace
    from q38.presets import model_config
    from q38.train import TRAIN_DEFAULTS, Trainer
    dev = torch.device("cuda", 0)
    cfg = model_config(dict(layers=4, hidden=128, heads=4, kv_heads=2, lin_k_heads=2, lin_v_heads=6, experts=8, topk=2, moe_ffn=32, shared_ffn=32,
                            ngram_rows=1024, mhc_iters=3, qsa_blocks=2), 512, 256, eos_token_id=7, pad_token_id=0)
    curves = []
    for fp8 in (0, 1):
        torch.manual_seed(0)
        args = SimpleNamespace(**{**TRAIN_DEFAULTS, "aux_coef": 0.001, "lr": 3e-3, "grad_sync": "collective", "fp8_ffn": fp8, "micro_bs": 2, "seq": 256})
        trainer = Trainer(cfg, args, dev)
        gen = torch.Generator().manual_seed(5)
        batches = [torch.randint(1, 512, (2, 256), generator=gen).pin_memory() for _ in range(3)]      # three batches, revisited
        losses = []
        for step in range(30):
            x = batches[step % 3]
            y = x.roll(-1, 1).pin_memory()
            losses.append(trainer.read_step(trainer.train_step([(x, y)], lr=3e-3, dense=step < 2))[0])
        trainer.close()
        curves.append(losses)
    bf16, fp8 = curves
    assert fp8[-1] < fp8[0] - 0.1, fp8
    tail = slice(20, 30)
    mean = lambda v: sum(v) / len(v)
    assert abs(mean(fp8[tail]) - mean(bf16[tail])) < 0.02 * mean(bf16[tail]), (mean(fp8[tail]), mean(bf16[tail]))
