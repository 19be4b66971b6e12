"""Per-kernel benchmark at the shapes of a preset: device time (CUDA events), achieved FLOP/s or bytes/s and the
fraction of the measured roofline.

  python -m q38.utils.kernel_bench --preset q38_c2 [--kernels gemm,moe,mhc,gdn,qsa,conv,fp8,muon,ce,ngram] [--iters 20] [--json out.json]

Denominators come from ``MEASURED_PEAKS.json`` at the repository root when present (copy bandwidth and cuBLAS bf16
throughput measured on the same pool), otherwise 6.65 TB/s and 1.59 PFLOP/s.  Inputs are larger than the 126 MB L2 or
are rotated through a pool that is, so DRAM figures are not flattered by cache hits.  This is also the small, single
kernel workload that `ncu` captures are taken on (one kernel family per run, a few GB resident).
"""
import argparse
import json
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        p = json.loads(path.read_text())
        return dict(hbm_gbs=p["hbm_gbs"], tflops=p["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, source="fallback")


def timeit(fn, iters, warmup=5):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / iters * 1e-3


def report(rows, name, seconds, flops=0.0, bytes_=0.0, pk=None):
    tf, gb = flops / seconds / 1e12, bytes_ / seconds / 1e9
    frac = max(tf / pk["tflops"], gb / pk["hbm_gbs"])
    bound = "compute" if tf / pk["tflops"] >= gb / pk["hbm_gbs"] else "memory"
    rows.append(dict(kernel=name, us=seconds * 1e6, tflops=tf, gbs=gb, bound=bound, fraction_of_roofline=frac, peaks=pk["source"]))
    print(f"{name:46s} {seconds * 1e6:9.1f} us  {tf:8.1f} TFLOP/s  {gb:8.1f} GB/s  {frac * 100:5.1f}% of {pk['source']} {bound} roofline", flush=True)


def bench_gemm(rows, shape, T, iters, pk):
    from .. import ops
    h = shape["hidden"]
    conv = 2 * shape["lin_k_heads"] * 64 + shape["lin_v_heads"] * 64
    cases = [("qkv_proj fwd (NT)", T, conv, h), ("out_proj fwd (NT)", T, h, shape["lin_v_heads"] * 64), ("lm_head chunk (NT)", 8192, 10112, h)]
    for name, M, N, K in cases:
        a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        t = timeit(lambda: ops.gemm(a, b, out=out), iters)
        report(rows, f"gemm_bf16 {name} {M}x{N}x{K}", t, flops=2.0 * M * N * K, bytes_=2.0 * (M * K + N * K + M * N), pk=pk)
    M, N, K = T, h, conv                                         # dgrad: dy[T,conv] @ W[conv,h]
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    w = torch.randn(K, N, device="cuda").to(torch.bfloat16)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    t = timeit(lambda: ops.gemm(a, w, out=out, b_mn_major=True), iters)
    report(rows, f"gemm_bf16 qkv_proj dgrad (NN) {M}x{N}x{K}", t, flops=2.0 * M * N * K, bytes_=2.0 * (M * K + N * K + M * N), pk=pk)
    dy = torch.randn(T, conv, device="cuda").to(torch.bfloat16)
    x = torch.randn(T, h, device="cuda").to(torch.bfloat16)
    grad = torch.zeros(conv, h, device="cuda")
    t = timeit(lambda: ops.gemm(dy, x, out=grad, a_mn_major=True, b_mn_major=True, accumulate=True, splits=0), iters)
    report(rows, f"gemm_bf16 qkv_proj wgrad (TN split-K) {conv}x{h}x{T}", t, flops=2.0 * conv * h * T, bytes_=2.0 * T * (conv + h) + 8.0 * conv * h, pk=pk)
    Xf = torch.randn(T, 4 * h, device="cuda")
    A = torch.randn(max(1, round(h / 8)), 4 * h, device="cuda")
    t = timeit(lambda: ops.gemm(Xf, A, out_dtype=torch.float32), iters)
    report(rows, f"gemm tf32 mhc low-rank {T}x{A.shape[0]}x{4 * h}", t, flops=2.0 * T * A.shape[0] * 4 * h, bytes_=4.0 * (T * 4 * h + A.numel() + T * A.shape[0]), pk=pk)


def bench_moe(rows, shape, T, iters, pk):
    from ..ops.backend import _Experts
    from .. import ops
    h, f, E, k = shape["hidden"], shape["moe_ffn"], shape["experts"], shape["topk"]
    lib = ops.load()
    x = torch.randn(T, h, device="cuda").to(torch.bfloat16)
    wgu = (0.05 * torch.randn(E, 2 * f, h, device="cuda")).to(torch.bfloat16)
    wd = (0.05 * torch.randn(E, h, f, device="cuda")).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)]).to(torch.int32)
    err = ops.error_flag()
    perm, inv, offsets, sched = lib.moe_sort(idx, E)
    t = timeit(lambda: lib.moe_sort(idx, E), iters)
    report(rows, f"moe_sort (3 kernels) P={T * k}", t, bytes_=4.0 * T * k * 4, pk=pk)
    xs = lib.moe_gather(x, perm, k)
    t = timeit(lambda: lib.moe_gather(x, perm, k), iters)
    report(rows, f"moe_gather {T * k}x{h}", t, bytes_=2.0 * T * k * h * 2, pk=pk)
    hmid = torch.empty(T * k, f, device="cuda", dtype=torch.bfloat16)
    gu = torch.empty(T * k, 2 * f, device="cuda", dtype=torch.bfloat16)
    t = timeit(lambda: lib.moe_grouped_swiglu(xs, wgu, hmid, gu, sched, err), iters)
    report(rows, f"moe_grouped_swiglu {T * k}x{2 * f}x{h}", t, flops=2.0 * T * k * 2 * f * h, bytes_=2.0 * (T * k * (h + 3 * f) + E * 2 * f * h), pk=pk)
    ys = torch.empty(T * k, h, device="cuda", dtype=torch.bfloat16)
    t = timeit(lambda: lib.moe_grouped_gemm(hmid, wd, ys, sched, False, err), iters)
    report(rows, f"moe_grouped_gemm down {T * k}x{h}x{f}", t, flops=2.0 * T * k * h * f, bytes_=2.0 * (T * k * (h + f) + E * h * f), pk=pk)
    dgu = torch.empty_like(gu)
    t = timeit(lambda: lib.moe_grouped_dswiglu(ys, wd, gu, dgu, sched, err), iters)
    report(rows, f"moe_grouped_dswiglu {T * k}x{f}x{h}", t, flops=2.0 * T * k * h * f, bytes_=2.0 * (T * k * (h + 4 * f) + E * h * f), pk=pk)
    grad = torch.zeros(E, 2 * f, h, device="cuda")
    t = timeit(lambda: lib.moe_grouped_wgrad(dgu, xs, grad, offsets, err), iters)
    report(rows, f"moe_grouped_wgrad gate_up {E}x{2 * f}x{h}", t, flops=2.0 * T * k * 2 * f * h, bytes_=2.0 * T * k * (2 * f + h) + 8.0 * grad.numel(), pk=pk)


def bench_mhc(rows, shape, T, iters, pk):
    from .. import ops
    lib = ops.load()
    h = shape["hidden"]
    r = max(1, round(h / 8))
    X = torch.randn(T, 4, h, device="cuda")
    L = torch.randn(T, r, device="cuda")
    Bw = 0.1 * torch.randn(24, r, device="cuda")
    bp, bq, br, al, nw = (torch.zeros(4, device="cuda"), torch.zeros(4, device="cuda"), torch.zeros(16, device="cuda"),
                          torch.full((3,), 0.1, device="cuda"), torch.zeros(h, device="cuda"))
    out = lib.mhc_coef_fwd(X, L, Bw, bp, bq, br, al, nw, 20, 1e-6, True)
    t = timeit(lambda: lib.mhc_coef_fwd(X, L, Bw, bp, bq, br, al, nw, 20, 1e-6, True), iters)
    report(rows, f"mhc_coef_fwd T={T} h={h}", t, bytes_=4.0 * T * 4 * h + 2.0 * T * h, pk=pk)
    y = torch.randn(T, h, device="cuda").to(torch.bfloat16)
    coef = out[1]
    t = timeit(lambda: lib.mhc_post_fwd(X, y, coef), iters)
    report(rows, f"mhc_post_fwd T={T} h={h}", t, bytes_=8.0 * T * 4 * h + 2.0 * T * h, pk=pk)
    t = timeit(lambda: lib.mhc_post_bwd(X, X, y, coef), iters)
    report(rows, f"mhc_post_bwd T={T} h={h}", t, bytes_=8.0 * T * 4 * h + 4.0 * T * h, pk=pk)


def bench_gdn(rows, shape, T, iters, pk, seq=4096):
    from .. import ops
    lib = ops.load()
    B, Hk, Hv = T // seq, shape["lin_k_heads"], shape["lin_v_heads"]
    qkv = torch.randn(B, seq, (2 * Hk + Hv) * 64, device="cuda").to(torch.bfloat16)
    q = qkv[..., :Hk * 64].unflatten(-1, (Hk, 64))
    k = qkv[..., Hk * 64:2 * Hk * 64].unflatten(-1, (Hk, 64))
    v = qkv[..., 2 * Hk * 64:].unflatten(-1, (Hv, 64))
    g = -torch.rand(B, seq, Hv, device="cuda") * 0.1
    beta = torch.rand(B, seq, Hv, device="cuda").to(torch.bfloat16)
    t = timeit(lambda: lib.gdn_prep_fwd(q, k, v, g, beta), iters)
    chunks = B * Hv * seq // 64
    report(rows, f"gdn_prep_fwd B={B} Hv={Hv}", t, flops=chunks * 5 * 2.0 * 64 ** 3, bytes_=chunks * 6 * 8192.0 + 2.0 * qkv.numel(), pk=pk)
    w, u, P, qg, kg, Tm, carry, _ = lib.gdn_prep_fwd(q, k, v, g, beta)
    t = timeit(lambda: lib.gdn_scan_fwd(w, u, P, qg, kg, carry, B, Hv), iters)
    report(rows, f"gdn_scan_fwd B={B} Hv={Hv}", t, flops=chunks * 4 * 2.0 * 64 ** 3, bytes_=chunks * 8 * 8192.0, pk=pk)
    o, vnew, states = lib.gdn_scan_fwd(w, u, P, qg, kg, carry, B, Hv)
    do = torch.randn_like(o)
    t = timeit(lambda: lib.gdn_scan_bwd(w, P, qg, kg, carry, vnew, states, do, B, Hv), iters)
    report(rows, f"gdn_scan_bwd B={B} Hv={Hv}", t, flops=chunks * 9 * 2.0 * 64 ** 3, bytes_=chunks * 12 * 8192.0, pk=pk)
    dw, du, dP, dqg, dkg, dd = lib.gdn_scan_bwd(w, P, qg, kg, carry, vnew, states, do, B, Hv)
    t = timeit(lambda: lib.gdn_prep_bwd(q, k, v, g, beta, Tm, dw, du, dP, dqg, dkg, dd), iters)
    report(rows, f"gdn_prep_bwd B={B} Hv={Hv}", t, flops=chunks * 14 * 2.0 * 64 ** 3, bytes_=chunks * 6 * 8192.0 + 4.0 * qkv.numel(), pk=pk)


def bench_qsa(rows, shape, T, iters, pk, seq=4096):
    from .. import ops
    lib = ops.load()
    B, nq, nkv = T // seq, shape["heads"], shape["kv_heads"]
    q = torch.randn(B, nq, seq, 64, device="cuda").to(torch.bfloat16)
    k = torch.randn(B, nkv, seq, 64, device="cuda").to(torch.bfloat16)
    v = torch.randn(B, nkv, seq, 64, device="cuda").to(torch.bfloat16)
    causal_tiles = B * (seq // 64) * (seq // 64 + 1) // 2
    t = timeit(lambda: lib.qsa_main_block_stats(q, k, 0.125), iters)
    report(rows, f"qsa_main_block_stats B={B} nq={nq}", t, flops=nq * causal_tiles * 2.0 * 64 ** 3, bytes_=8.0 * B * nq * seq * (seq // 64) / 2, pk=pk)
    if seq % 128 == 0:
        from .. import ops as ops_module
        err = ops_module.error_flag()
        t = timeit(lambda: lib.qsa_block_stats_tc(q, k, 0.125, err), iters)
        report(rows, f"qsa_block_stats_tc (tcgen05) B={B} nq={nq}", t, flops=nq * causal_tiles * 2.0 * 64 ** 3, bytes_=8.0 * B * nq * seq * (seq // 64) / 2, pk=pk)
    qi = torch.randn(B, 4, seq, 64, device="cuda").to(torch.bfloat16)
    ki = torch.randn(B, seq, 64, device="cuda").to(torch.bfloat16)
    wi = torch.rand(B, seq, 4, device="cuda")
    t = timeit(lambda: lib.qsa_indexer_fwd(qi, ki, wi, 0.125), iters)
    report(rows, f"qsa_indexer_fwd B={B}", t, flops=4 * causal_tiles * 2.0 * 64 ** 3, pk=pk)
    blse = lib.qsa_indexer_fwd(qi, ki, wi, 0.125)
    dblse = torch.randn_like(blse) * 1e-3
    t = timeit(lambda: lib.qsa_indexer_bwd(qi, ki, wi, blse, dblse, 1.0 / (B * seq), 0.125), iters)
    report(rows, f"qsa_indexer_bwd (q and k kernels) B={B}", t, flops=3 * 4 * causal_tiles * 2.0 * 64 ** 3, pk=pk)
    lp = torch.randn(B, seq // 64, seq // 64, device="cuda")
    count, index = lib.qsa_select(lp, shape["qsa_blocks"])
    t = timeit(lambda: lib.qsa_attn_fwd(q, k, v, count, index, 0.125), iters)
    tiles = int(count.sum().item()) * nq
    report(rows, f"qsa_attn_fwd sparse B={B} nq={nq}", t, flops=tiles * 2 * 2.0 * 64 ** 3, bytes_=2.0 * (2 * q.numel()), pk=pk)
    o, lse, sel = lib.qsa_attn_fwd(q, k, v, count, index, 0.125)
    do = torch.randn_like(o)
    t = timeit(lambda: lib.qsa_attn_bwd(q, k, v, o, do, lse, sel, 0.125), iters)
    report(rows, f"qsa_attn_bwd sparse B={B} nq={nq}", t, flops=tiles * 7 * 2.0 * 64 ** 3, bytes_=2.0 * (4 * q.numel()), pk=pk)


def bench_conv(rows, shape, T, iters, pk, seq=4096):
    from .. import ops
    lib = ops.load()
    C = 2 * shape["lin_k_heads"] * 64 + shape["lin_v_heads"] * 64
    x = torch.randn(T // seq, seq, C, device="cuda").to(torch.bfloat16)
    w = torch.randn(C, 4, device="cuda")
    t = timeit(lambda: lib.conv_silu_fwd(x, w), iters)
    report(rows, f"conv_silu_fwd C={C}", t, bytes_=4.0 * x.numel(), pk=pk)
    t = timeit(lambda: lib.conv_silu_bwd(x, w, x), iters)
    report(rows, f"conv_silu_bwd C={C}", t, bytes_=6.0 * x.numel(), pk=pk)


BENCHES = dict(gemm=bench_gemm, moe=bench_moe, mhc=bench_mhc, gdn=bench_gdn, qsa=bench_qsa, conv=bench_conv)


def bench_fp8(rows, shape, T, iters, pk):
    """Block-scaled MXFP8 expert products (csrc/mxfp8.cu): quantisation kernels and the grouped mxf8f6f4 GEMM."""
    from .. import ops
    h, f, E, k = shape["hidden"], shape["moe_ffn"], shape["experts"], shape["topk"]
    lib, err = ops.load(), ops.error_flag()
    P = T * k
    x = torch.randn(T, h, device="cuda").to(torch.bfloat16)
    wgu = (0.05 * torch.randn(E, 2 * f, h, device="cuda")).to(torch.bfloat16)
    wd = (0.05 * torch.randn(E, h, f, device="cuda")).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)]).to(torch.int32)
    perm, inv, offsets, sched = lib.moe_sort(idx, E)
    t = timeit(lambda: lib.mxfp8_quantize_rows(x, perm, k, sched, P), iters)
    report(rows, f"mxfp8_quantize_rows (gather) {P}x{h}", t, bytes_=P * h * 3.0 + P * h / 32, pk=pk)
    xq, sfx = lib.mxfp8_quantize_rows(x, perm, k, sched, P)
    bn = int(lib.mxfp8_pick_bn(2 * f))
    t = timeit(lambda: lib.mxfp8_quantize_weight(wgu, bn), iters)
    report(rows, f"mxfp8_quantize_weight {E}x{2 * f}x{h}", t, bytes_=3.0 * wgu.numel(), pk=pk)
    q, sf = lib.mxfp8_quantize_weight(wgu, bn)
    gu = torch.empty(P, 2 * f, device="cuda", dtype=torch.bfloat16)
    t = timeit(lambda: lib.mxfp8_grouped_gemm(xq, sfx, q, sf, gu, sched, bn, err), iters)
    report(rows, f"mxfp8_grouped_gemm gate_up {P}x{2 * f}x{h}", t, flops=2.0 * P * 2 * f * h, bytes_=P * h + 2.0 * P * 2 * f + E * 2 * f * h, pk=pk)
    hmid = torch.randn(P, f, device="cuda").to(torch.bfloat16)
    hq, sfh = lib.mxfp8_quantize_rows(hmid, None, 1, sched, P)
    bn = int(lib.mxfp8_pick_bn(h))
    q, sf = lib.mxfp8_quantize_weight(wd, bn)
    ys = torch.empty(P, h, device="cuda", dtype=torch.bfloat16)
    t = timeit(lambda: lib.mxfp8_grouped_gemm(hq, sfh, q, sf, ys, sched, bn, err), iters)
    report(rows, f"mxfp8_grouped_gemm down {P}x{h}x{f}", t, flops=2.0 * P * h * f, bytes_=P * f + 2.0 * P * h + E * h * f, pk=pk)


def bench_muon(rows, shape, T, iters, pk):
    """Fused Muon step (csrc/muon.cu + Newton-Schulz on the persistent GEMM) on the expert matrices of 4 layers."""
    from .. import ops
    from ..ops.muon_gpu import FusedMuon
    h, f, E = shape["hidden"], shape["moe_ffn"], shape["experts"]
    entries, cursor = [], 0
    for _ in range(4):
        for r, c in ((2 * f, h), (h, f)):
            entries.append((cursor, E, r, c))
            cursor += E * r * c
    params, grads, buf = (torch.randn(cursor, device="cuda") for _ in range(3))
    shadow = torch.zeros(cursor, device="cuda", dtype=torch.bfloat16)
    plan = FusedMuon(params, grads, buf, shadow, entries)
    err = ops.error_flag()
    lib = ops.load()
    t = timeit(lambda: lib.muon_prepass(grads, buf, plan.work, plan.sumsq, plan.mats, plan.tiles, None, 0.95, err), iters)
    report(rows, f"muon_prepass {cursor / 1e6:.1f}M elements", t, bytes_=14.0 * cursor, pk=pk)
    lib.muon_normalize(plan.work, plan.sumsq, plan.mats, plan.tiles, 1e-7, err)
    t = timeit(lambda: lib.muon_apply(params, shadow, plan.work, plan.mats, plan.tiles, plan.scales, None, 1e-3, 0.1, err), iters)
    report(rows, f"muon_apply {cursor / 1e6:.1f}M elements", t, bytes_=12.0 * cursor, pk=pk)
    flops = 0.0
    for _, n, r, c in entries:
        m, kk = min(r, c), max(r, c)
        flops += n * 5 * (4.0 * m * m * kk + 2.0 * m ** 3)
    t = timeit(lambda: plan.step(1e-3, 0.95, 0.1, err=err), max(3, iters // 4), warmup=2)
    report(rows, f"muon step (prepass + 5 NS iterations + apply), {len(entries) * E} matrices", t, flops=flops, bytes_=26.0 * cursor, pk=pk)


def bench_ce(rows, shape, T, iters, pk):
    """In-place cross-entropy over one vocabulary chunk of bf16 logits: loss per row out, d(logits) left in the logits buffer."""
    from .. import ops
    lib = ops.load()
    vocab, chunk = 10112, 8192
    logits = [torch.randn(chunk, vocab, device="cuda").to(torch.bfloat16) for _ in range(2)]      # 2 x 166 MB: rotated, larger than L2
    target = torch.randint(0, vocab, (chunk,), device="cuda")
    state = {"i": 0}

    def step():
        state["i"] ^= 1
        lib.ce_inplace(logits[state["i"]], target)

    t = timeit(step, iters)
    report(rows, f"ce_inplace {chunk}x{vocab}", t, bytes_=4.0 * chunk * vocab, pk=pk)


def bench_ngram(rows, shape, T, iters, pk, seq=4096):
    """Bigram/trigram hash embedding: gather + sum + RMSNorm forward, scatter-add backward into the fp32 tables."""
    from .. import ops
    from ..presets import model_config
    lib = ops.load()
    cfg = model_config(dict(shape), 10112, seq)
    h, table_rows = shape["hidden"], cfg.ngram_rows
    emb2 = torch.randn(table_rows, h, device="cuda") * 0.02
    emb3 = torch.randn(table_rows, h, device="cuda") * 0.02
    norm_w = torch.ones(h, device="cuda")
    ids = torch.randint(1, 10112, (T // seq, seq), device="cuda")
    t = timeit(lambda: lib.ngram_fwd(ids, emb2, emb3, norm_w, 10112, 53, 1e-6), iters)
    report(rows, f"ngram_fwd T={T} h={h} rows={table_rows}", t, bytes_=T * h * (2 * 4 + 2.0), pk=pk)
    e, rstd, picked = lib.ngram_fwd(ids, emb2, emb3, norm_w, 10112, 53, 1e-6)
    de = torch.randn_like(e)
    g2, g3 = torch.zeros_like(emb2), torch.zeros_like(emb3)
    t = timeit(lambda: lib.ngram_bwd(de, picked, emb2, emb3, norm_w, rstd, g2, g3), iters)
    report(rows, f"ngram_bwd T={T} h={h}", t, bytes_=T * h * (2.0 + 2 * 4 + 2 * 8), pk=pk)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--preset", default="q38_c2")
    ap.add_argument("--tokens", type=int, default=16384, help="tokens per micro-batch (micro_bs * seq)")
    ap.add_argument("--kernels", default=",".join(BENCHES))
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", default="")
    a = ap.parse_args(argv)
    from .. import ops
    from ..presets import load_preset
    ops.install()
    shape = load_preset(a.preset)["model"]
    pk = peaks()
    rows = []
    torch.manual_seed(0)
    BENCHES.update(fp8=bench_fp8, muon=bench_muon, ce=bench_ce, ngram=bench_ngram)
    for name in a.kernels.split(","):
        BENCHES[name](rows, shape, a.tokens, a.iters, pk)
    ops.check_errors()
    if a.json:
        Path(a.json).write_text(json.dumps(dict(preset=a.preset, tokens=a.tokens, peaks=pk, rows=rows), indent=1) + "\n")
    return rows


if __name__ == "__main__":
    main()
