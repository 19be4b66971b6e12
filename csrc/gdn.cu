// Gated DeltaNet: chunked gated delta rule (chunk = 64 tokens, head dims 64), forward and backward.
//
// Per (batch, value head) and chunk c, with S the [k-dim x v-dim] state at the chunk start:
//     v_new = u - w S                  o = qg S + P v_new                  S' = d S + kg^T v_new
// where (prepared per chunk, all independent of S and therefore fully parallel over chunks)
//     gc = cumsum(g) inside the chunk,  Gamma_ij = exp(gc_i - gc_j)
//     Tm = (I + tril(beta_i (k_i.k_j) Gamma_ij, -1))^-1,   w = Tm (beta e^gc k),   u = Tm (beta v)
//     P  = tril((q_i.k_j) Gamma_ij),   qg = q e^gc,   kg = k e^(gc_last - gc),   d = e^gc_last
// with q, k L2-normalised and q scaled by 64^-1/2.
//
// Kernels
//   gdn_scan_fwd   one CTA per (batch, value head): the sequential pass over chunks.  The fp32 state lives in the
//                  accumulator registers of eight warps (16 k-rows x 32 v-columns each); every product is a 64x64x64
//                  bf16 mma.sync with fp32 accumulation; chunk operands are prefetched with cp.async one chunk ahead.
//                  The chain per chunk is latency bound (three dependent products), which is why this pass uses
//                  register-resident warp MMAs instead of the TMEM round trips of tcgen05.
//   gdn_scan_bwd   the reverse pass: dS' -> (dw, du, dP, dqg, dkg, dd) per chunk and dS.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"
#include "host.h"
#include "mma_tile.cuh"

namespace q38 {

// ---------------------------------------------------------------------------------------------------------------------
// Forward scan.  Chunk operands w,u,P,qg,kg: [BH, NT, 64, 64] bf16; dch: [BH, NT] fp32.
// Outputs: o [B, S, H, 64] bf16 (token-major), vnew [BH, NT, 64, 64] bf16, states [BH, NT, 64, 64] bf16 (chunk-start S).
// ---------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gdn_scan_fwd_kernel(const bf16* __restrict__ w, const bf16* __restrict__ u, const bf16* __restrict__ P,
                                                           const bf16* __restrict__ qg, const bf16* __restrict__ kg, const float* __restrict__ dch,
                                                           bf16* __restrict__ o, bf16* __restrict__ vnew, bf16* __restrict__ states, int NT, int H) {
  extern __shared__ __align__(16) uint8_t smem_bytes[];
  bf16* sm = reinterpret_cast<bf16*>(smem_bytes);
  // two buffers of five operand tiles, then the bf16 copies of S and v_new
  bf16* Sb = sm + 10 * TILE_ELEMS;
  bf16* Vn = Sb + TILE_ELEMS;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x, b = bh / H, hv = bh % H;
  const long long tile = 64 * 64;
  const bf16* srcs[5] = {w + (long long)bh * NT * tile, u + (long long)bh * NT * tile, P + (long long)bh * NT * tile,
                         qg + (long long)bh * NT * tile, kg + (long long)bh * NT * tile};
  auto prefetch = [&](int c, int buf) {
#pragma unroll
    for (int t = 0; t < 5; ++t) load_tile_async_256(sm + (buf * 5 + t) * TILE_ELEMS, srcs[t] + (long long)c * tile, 64, tid);
    cp_async_commit();
  };
  // eight warps: warp w keeps rows 16 (w & 3).. and v-columns 32 (w >> 2).. of the fp32 state in registers
  float S[4][4];
  zero_acc(S);
  prefetch(0, 0);
  for (int c = 0; c < NT; ++c) {
    const int buf = c & 1;
    if (c + 1 < NT) { prefetch(c + 1, buf ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    acc_to_smem_h(S, Sb, warp, lane);
    acc_to_global_h(S, states + ((long long)bh * NT + c) * tile, 64, warp, lane);
    __syncthreads();                                   // operand tiles of chunk c and Sb are visible
    const bf16* Wt = sm + (buf * 5 + 0) * TILE_ELEMS;
    const bf16* Ut = Wt + TILE_ELEMS;
    const bf16* Pt = Ut + TILE_ELEMS;
    const bf16* Qt = Pt + TILE_ELEMS;
    const bf16* Kt = Qt + TILE_ELEMS;
    float acc[4][4];
    zero_acc(acc);
    mma64h<false, false>(Wt, Sb, acc, warp, lane);     // w S
    {
      const int r = 16 * (warp & 3) + (lane >> 2), c0 = 32 * (warp >> 2) + 2 * (lane & 3);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const __nv_bfloat162 u0 = *reinterpret_cast<const __nv_bfloat162*>(Ut + r * LDS + 8 * nt + c0);
        const __nv_bfloat162 u1 = *reinterpret_cast<const __nv_bfloat162*>(Ut + (r + 8) * LDS + 8 * nt + c0);
        acc[nt][0] = __low2float(u0) - acc[nt][0]; acc[nt][1] = __high2float(u0) - acc[nt][1];
        acc[nt][2] = __low2float(u1) - acc[nt][2]; acc[nt][3] = __high2float(u1) - acc[nt][3];
      }
    }
    acc_to_smem_h(acc, Vn, warp, lane);                // v_new (bf16) for the two products below
    acc_to_global_h(acc, vnew + ((long long)bh * NT + c) * tile, 64, warp, lane);
    float out[4][4];
    zero_acc(out);
    mma64h<false, false>(Qt, Sb, out, warp, lane);     // qg S
    __syncthreads();                                   // Vn complete
    mma64h<false, false>(Pt, Vn, out, warp, lane);     // + P v_new
    acc_to_global_h(out, o + (((long long)b * NT * 64 + (long long)c * 64) * H + hv) * 64, (long long)H * 64, warp, lane);
    const float d = dch[(long long)bh * NT + c];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) { S[nt][0] *= d; S[nt][1] *= d; S[nt][2] *= d; S[nt][3] *= d; }
    mma64h<true, false>(Kt, Vn, S, warp, lane);        // + kg^T v_new
    __syncthreads();                                   // everyone is done with Sb, Vn and this buffer
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Backward scan (reverse over chunks).  Inputs: the forward operands, vnew, states, and do [B,S,H,64].
// Outputs per chunk: dw, du, dP, dqg, dkg [BH,NT,64,64] bf16 and dd [BH,NT] fp32.
// ---------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gdn_scan_bwd_kernel(const bf16* __restrict__ w, const bf16* __restrict__ P, const bf16* __restrict__ qg,
                                                           const bf16* __restrict__ kg, const float* __restrict__ dch, const bf16* __restrict__ vnew,
                                                           const bf16* __restrict__ states, const bf16* __restrict__ dout, bf16* __restrict__ dw,
                                                           bf16* __restrict__ du, bf16* __restrict__ dP, bf16* __restrict__ dqg, bf16* __restrict__ dkg,
                                                           float* __restrict__ dd, int NT, int H) {
  extern __shared__ __align__(16) uint8_t smem_bytes[];
  bf16* sm = reinterpret_cast<bf16*>(smem_bytes);
  // two buffers of seven tiles: w, P, qg, kg, vnew, state, do ; then dS (bf16) and dv_new (bf16)
  bf16* dSb = sm + 14 * TILE_ELEMS;
  bf16* dVn = dSb + TILE_ELEMS;
  __shared__ float red[8];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x, b = bh / H, hv = bh % H;
  const long long tile = 64 * 64, base = (long long)bh * NT * tile;
  auto prefetch = [&](int c, int buf) {
    bf16* dst = sm + buf * 7 * TILE_ELEMS;
    load_tile_async_256(dst + 0 * TILE_ELEMS, w + base + (long long)c * tile, 64, tid);
    load_tile_async_256(dst + 1 * TILE_ELEMS, P + base + (long long)c * tile, 64, tid);
    load_tile_async_256(dst + 2 * TILE_ELEMS, qg + base + (long long)c * tile, 64, tid);
    load_tile_async_256(dst + 3 * TILE_ELEMS, kg + base + (long long)c * tile, 64, tid);
    load_tile_async_256(dst + 4 * TILE_ELEMS, vnew + base + (long long)c * tile, 64, tid);
    load_tile_async_256(dst + 5 * TILE_ELEMS, states + base + (long long)c * tile, 64, tid);
    load_tile_async_256(dst + 6 * TILE_ELEMS, dout + (((long long)b * NT * 64 + (long long)c * 64) * H + hv) * 64, (long long)H * 64, tid);
    cp_async_commit();
  };
  const int r = 16 * (warp & 3) + (lane >> 2), c0 = 32 * (warp >> 2) + 2 * (lane & 3);
  float dS[4][4];
  zero_acc(dS);
  prefetch(NT - 1, (NT - 1) & 1);
  for (int c = NT - 1; c >= 0; --c) {
    const int buf = c & 1;
    if (c > 0) { prefetch(c - 1, buf ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    acc_to_smem_h(dS, dSb, warp, lane);
    __syncthreads();
    const bf16* Wt = sm + buf * 7 * TILE_ELEMS;
    const bf16* Pt = Wt + TILE_ELEMS;
    const bf16* Qt = Pt + TILE_ELEMS;
    const bf16* Kt = Qt + TILE_ELEMS;
    const bf16* Vt = Kt + TILE_ELEMS;
    const bf16* St = Vt + TILE_ELEMS;
    const bf16* Dt = St + TILE_ELEMS;
    const long long off = base + (long long)c * tile;
    float acc[4][4];
    // dv_new = P^T dO + kg dS'
    zero_acc(acc);
    mma64h<true, false>(Pt, Dt, acc, warp, lane);
    mma64h<false, false>(Kt, dSb, acc, warp, lane);
    acc_to_smem_h(acc, dVn, warp, lane);
    acc_to_global_h(acc, du + off, 64, warp, lane);
    // dd = <dS', S>   (fragment of S read from the state tile in accumulator layout)
    {
      float part = 0.f;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const __nv_bfloat162 s0 = *reinterpret_cast<const __nv_bfloat162*>(St + r * LDS + 8 * nt + c0);
        const __nv_bfloat162 s1 = *reinterpret_cast<const __nv_bfloat162*>(St + (r + 8) * LDS + 8 * nt + c0);
        part += dS[nt][0] * __low2float(s0) + dS[nt][1] * __high2float(s0) + dS[nt][2] * __low2float(s1) + dS[nt][3] * __high2float(s1);
      }
      part = warp_sum(part);
      if (lane == 0) red[warp] = part;
    }
    // dqg = dO S^T ;  dkg = v_new dS'^T ;  dP = tril(dO v_new^T)
    zero_acc(acc);
    mma64h<false, true>(Dt, St, acc, warp, lane);
    acc_to_global_h(acc, dqg + off, 64, warp, lane);
    zero_acc(acc);
    mma64h<false, true>(Vt, dSb, acc, warp, lane);
    acc_to_global_h(acc, dkg + off, 64, warp, lane);
    zero_acc(acc);
    mma64h<false, true>(Dt, Vt, acc, warp, lane);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int col = 8 * nt + c0;
      if (col > r) acc[nt][0] = 0.f;
      if (col + 1 > r) acc[nt][1] = 0.f;
      if (col > r + 8) acc[nt][2] = 0.f;
      if (col + 1 > r + 8) acc[nt][3] = 0.f;
    }
    acc_to_global_h(acc, dP + off, 64, warp, lane);
    __syncthreads();                                    // dVn and red[] complete
    if (tid == 0) dd[(long long)bh * NT + c] = red[0] + red[1] + red[2] + red[3] + red[4] + red[5] + red[6] + red[7];
    // dw = -dv_new S^T
    zero_acc(acc);
    mma64h<false, true>(dVn, St, acc, warp, lane);
    acc_to_global_h(acc, dw + off, 64, warp, lane, -1.f);
    // dS = d dS' + qg^T dO - w^T dv_new
    const float d = dch[(long long)bh * NT + c];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) { dS[nt][0] *= d; dS[nt][1] *= d; dS[nt][2] *= d; dS[nt][3] *= d; }
    mma64h<true, false>(Qt, Dt, dS, warp, lane);
    zero_acc(acc);
    mma64h<true, false>(Wt, dVn, acc, warp, lane);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) { dS[nt][0] -= acc[nt][0]; dS[nt][1] -= acc[nt][1]; dS[nt][2] -= acc[nt][2]; dS[nt][3] -= acc[nt][3]; }
    __syncthreads();
  }
}

// ---- host ----------------------------------------------------------------------------------------------------------------
static void check_tiles(const at::Tensor& t, int64_t BH, int64_t NT, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.is_contiguous() && t.numel() == BH * NT * 64 * 64, name, ": contiguous bf16 [BH,NT,64,64] required");
}

// Returns {o [B,S,H,64], vnew [BH,NT,64,64], states [BH,NT,64,64]}
std::vector<at::Tensor> gdn_scan_fwd(const at::Tensor& w, const at::Tensor& u, const at::Tensor& P, const at::Tensor& qg, const at::Tensor& kg,
                                     const at::Tensor& dch, int64_t B, int64_t H) {
  const c10::cuda::CUDAGuard guard(w.device());
  const int64_t BH = B * H, NT = w.numel() / (BH * 64 * 64);
  check_tiles(w, BH, NT, "w"); check_tiles(u, BH, NT, "u"); check_tiles(P, BH, NT, "P"); check_tiles(qg, BH, NT, "qg"); check_tiles(kg, BH, NT, "kg");
  TORCH_CHECK(dch.scalar_type() == at::kFloat && dch.is_contiguous() && dch.numel() == BH * NT, "gdn_scan_fwd: dch must be fp32 [BH,NT]");
  auto o = at::empty({B, NT * 64, H, 64}, w.options());
  auto vnew = at::empty({BH, NT, 64, 64}, w.options()), states = at::empty({BH, NT, 64, 64}, w.options());
  const int smem = 12 * TILE_ELEMS * 2;
  static bool configured = false;
  if (!configured) { C10_CUDA_CHECK(cudaFuncSetAttribute(gdn_scan_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); configured = true; }
  gdn_scan_fwd_kernel<<<(int)BH, 256, smem, at::cuda::getCurrentCUDAStream()>>>(
      (const bf16*)w.data_ptr(), (const bf16*)u.data_ptr(), (const bf16*)P.data_ptr(), (const bf16*)qg.data_ptr(), (const bf16*)kg.data_ptr(),
      dch.data_ptr<float>(), (bf16*)o.data_ptr(), (bf16*)vnew.data_ptr(), (bf16*)states.data_ptr(), (int)NT, (int)H);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {o, vnew, states};
}

// Returns {dw, du, dP, dqg, dkg (bf16 tiles), dd [BH,NT] fp32}
std::vector<at::Tensor> gdn_scan_bwd(const at::Tensor& w, const at::Tensor& P, const at::Tensor& qg, const at::Tensor& kg, const at::Tensor& dch,
                                     const at::Tensor& vnew, const at::Tensor& states, const at::Tensor& dout, int64_t B, int64_t H) {
  const c10::cuda::CUDAGuard guard(w.device());
  const int64_t BH = B * H, NT = w.numel() / (BH * 64 * 64);
  check_tiles(w, BH, NT, "w"); check_tiles(P, BH, NT, "P"); check_tiles(qg, BH, NT, "qg"); check_tiles(kg, BH, NT, "kg");
  check_tiles(vnew, BH, NT, "vnew"); check_tiles(states, BH, NT, "states");
  TORCH_CHECK(dout.scalar_type() == at::kBFloat16 && dout.is_contiguous() && dout.numel() == BH * NT * 64 * 64, "gdn_scan_bwd: do must be contiguous bf16 [B,S,H,64]");
  auto opts = w.options();
  auto dw = at::empty({BH, NT, 64, 64}, opts), du = at::empty({BH, NT, 64, 64}, opts), dP = at::empty({BH, NT, 64, 64}, opts);
  auto dqg = at::empty({BH, NT, 64, 64}, opts), dkg = at::empty({BH, NT, 64, 64}, opts);
  auto dd = at::empty({BH, NT}, opts.dtype(at::kFloat));
  const int smem = 16 * TILE_ELEMS * 2;
  static bool configured = false;
  if (!configured) { C10_CUDA_CHECK(cudaFuncSetAttribute(gdn_scan_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); configured = true; }
  gdn_scan_bwd_kernel<<<(int)BH, 256, smem, at::cuda::getCurrentCUDAStream()>>>(
      (const bf16*)w.data_ptr(), (const bf16*)P.data_ptr(), (const bf16*)qg.data_ptr(), (const bf16*)kg.data_ptr(), dch.data_ptr<float>(),
      (const bf16*)vnew.data_ptr(), (const bf16*)states.data_ptr(), (const bf16*)dout.data_ptr(), (bf16*)dw.data_ptr(), (bf16*)du.data_ptr(),
      (bf16*)dP.data_ptr(), (bf16*)dqg.data_ptr(), (bf16*)dkg.data_ptr(), dd.data_ptr<float>(), (int)NT, (int)H);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {dw, du, dP, dqg, dkg, dd};
}

}  // namespace q38

// =====================================================================================================================
// Chunk preparation (everything that does not depend on the running state), forward and backward.
// =====================================================================================================================
namespace q38 {

#define FRAG_LOOP(nt, e, row, col)                                             \
  _Pragma("unroll") for (int nt = 0; nt < 8; ++nt)                              \
  _Pragma("unroll") for (int e = 0; e < 4; ++e)                                 \
    if (const int row = 16 * warp + (lane >> 2) + 8 * (e >> 1); true)           \
      if (const int col = 8 * nt + 2 * (lane & 3) + (e & 1); true)

// Loads 64 tokens x 64 dims of one head (token stride `ld` elements) and returns, per token row, the reciprocal norm.
// Thread layout: token = tid / 2, half = tid % 2 (32 dims each).
__device__ __forceinline__ void load_half_row(const bf16* __restrict__ src, long long ld, int tid, float (&vals)[32]) {
  const int tok = tid >> 1, half = tid & 1;
  const uint4* p = reinterpret_cast<const uint4*>(src + (long long)tok * ld + half * 32);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4 raw = p[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) { vals[i * 8 + 2 * j] = __low2float(h[j]); vals[i * 8 + 2 * j + 1] = __high2float(h[j]); }
  }
}

__device__ __forceinline__ void store_half_row_smem(bf16* __restrict__ tile, int tid, const float (&vals)[32], float scale) {
  const int tok = tid >> 1, half = tid & 1;
#pragma unroll
  for (int i = 0; i < 16; ++i)
    *reinterpret_cast<__nv_bfloat162*>(tile + tok * LDS + half * 32 + 2 * i) = __floats2bfloat162_rn(vals[2 * i] * scale, vals[2 * i + 1] * scale);
}

__device__ __forceinline__ void store_half_row_global(bf16* __restrict__ dst, int tid, const float (&vals)[32], float scale) {
  const int tok = tid >> 1, half = tid & 1;
  uint4* p = reinterpret_cast<uint4*>(dst + tok * 64 + half * 32);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t wds[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __nv_bfloat162 h = __floats2bfloat162_rn(vals[i * 8 + 2 * j] * scale, vals[i * 8 + 2 * j + 1] * scale);
      wds[j] = *reinterpret_cast<uint32_t*>(&h);
    }
    p[i] = make_uint4(wds[0], wds[1], wds[2], wds[3]);
  }
}

// Shared prologue of the preparation kernels: normalised q/k tiles, gc, beta, reciprocal norms in shared memory.
struct PrepSmem {
  bf16 *Qn, *Kn, *KBG, *VB, *Tm;
  float *gc, *beta, *rq, *rk;
};

__device__ __forceinline__ void prep_load_qk(const PrepSmem& s, const bf16* __restrict__ q, const bf16* __restrict__ k, long long ld_qk, int tid) {
  float qv[32], kv[32];
  load_half_row(q, ld_qk, tid, qv);
  load_half_row(k, ld_qk, tid, kv);
  float sq = 0.f, sk = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) { sq += qv[i] * qv[i]; sk += kv[i] * kv[i]; }
  sq += __shfl_xor_sync(0xffffffffu, sq, 1);
  sk += __shfl_xor_sync(0xffffffffu, sk, 1);
  const float rq = rsqrtf(sq + 1e-6f), rk = rsqrtf(sk + 1e-6f);
  if ((tid & 1) == 0) { s.rq[tid >> 1] = rq; s.rk[tid >> 1] = rk; }
  store_half_row_smem(s.Qn, tid, qv, rq * 0.125f);
  store_half_row_smem(s.Kn, tid, kv, rk);
}

// gc = inclusive cumsum of g over the chunk (warp 0, two tokens per lane); beta copied to shared memory.
__device__ __forceinline__ void prep_load_gates(const PrepSmem& s, const float* __restrict__ g, const bf16* __restrict__ beta, long long ld, int tid) {
  if (tid < 32) {
    const float g0 = g[(long long)(2 * tid) * ld], g1 = g[(long long)(2 * tid + 1) * ld];
    float run = g0 + g1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const float up = __shfl_up_sync(0xffffffffu, run, o); if (tid >= o) run += up; }
    s.gc[2 * tid] = run - g1;
    s.gc[2 * tid + 1] = run;
  } else if (tid < 96) {
    s.beta[tid - 32] = __bfloat162float(beta[(long long)(tid - 32) * ld]);
  }
}

// q,k: [B,S,Hk,64]; v: [B,S,Hv,64]; g fp32 / beta bf16: [B,S,Hv].  Tiles out: [B*Hv, NT, 64, 64] bf16.
__global__ void __launch_bounds__(128) gdn_prep_fwd_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                                                           const float* __restrict__ g, const bf16* __restrict__ beta, bf16* __restrict__ w_out,
                                                           bf16* __restrict__ u_out, bf16* __restrict__ P_out, bf16* __restrict__ qg_out,
                                                           bf16* __restrict__ kg_out, bf16* __restrict__ Tm_out, float* __restrict__ carry,
                                                           float* __restrict__ gc_out, int S, int Hk, int Hv, long long qk_ld, long long v_ld) {
  extern __shared__ __align__(16) uint8_t smem_bytes[];
  bf16* sm = reinterpret_cast<bf16*>(smem_bytes);
  PrepSmem s;
  s.Qn = sm; s.Kn = sm + TILE_ELEMS; s.KBG = sm + 2 * TILE_ELEMS; s.VB = sm + 3 * TILE_ELEMS; s.Tm = sm + 4 * TILE_ELEMS;
  constexpr int LSTRIDE = 68;                                        // rows 16-byte aligned for float4 reads
  float* L = reinterpret_cast<float*>(sm + 5 * TILE_ELEMS);          // [64][68]
  s.gc = L + 64 * LSTRIDE; s.beta = s.gc + 64; s.rq = s.beta + 64; s.rk = s.rq + 64;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, bh = blockIdx.y, b = bh / Hv, hv = bh % Hv, hk = hv / (Hv / Hk);
  const int NT = gridDim.x;
  const long long tok0 = (long long)b * S + (long long)c * 64;
  const long long tile_off = ((long long)bh * NT + c) * 4096;
  prep_load_qk(s, q + tok0 * qk_ld + hk * 64, k + tok0 * qk_ld + hk * 64, qk_ld, tid);
  prep_load_gates(s, g + tok0 * Hv + hv, beta + tok0 * Hv + hv, Hv, tid);
  __syncthreads();
  {
    // qg, kg to global; KBG and VB to shared memory (thread = token half-row)
    const int tok = tid >> 1, half = tid & 1;
    const float gct = s.gc[tok], gl = s.gc[63], bt = s.beta[tok];
    float row[32];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(s.Qn + tok * LDS + half * 32 + 2 * i);
      row[2 * i] = __low2float(h); row[2 * i + 1] = __high2float(h);
    }
    store_half_row_global(qg_out + tile_off, tid, row, __expf(gct));
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(s.Kn + tok * LDS + half * 32 + 2 * i);
      row[2 * i] = __low2float(h); row[2 * i + 1] = __high2float(h);
    }
    store_half_row_global(kg_out + tile_off, tid, row, __expf(gl - gct));
    store_half_row_smem(s.KBG, tid, row, bt * __expf(gct));
    load_half_row(v + tok0 * v_ld + hv * 64, v_ld, tid, row);
    store_half_row_smem(s.VB, tid, row, bt);
    if (tid == 0) carry[(long long)bh * NT + c] = __expf(gl);
    if (tid < 64) gc_out[((long long)bh * NT + c) * 64 + tid] = s.gc[tid];
  }
  float acc[8][4];
  zero_acc(acc);
  mma64<false, true>(s.Kn, s.Kn, acc, warp, lane);                    // k_i . k_j
  FRAG_LOOP(nt, e, row, col) { L[row * LSTRIDE + col] = col < row ? s.beta[row] * acc[nt][e] * __expf(s.gc[row] - s.gc[col]) : 0.f; }
  zero_acc(acc);
  mma64<false, true>(s.Qn, s.Kn, acc, warp, lane);                    // q_i . k_j
  FRAG_LOOP(nt, e, row, col) { acc[nt][e] = col <= row ? acc[nt][e] * __expf(s.gc[row] - s.gc[col]) : 0.f; }
  acc_to_global(acc, P_out + tile_off, 64, warp, lane);
  __syncthreads();
  if (tid < 64) {
    // column `tid` of (I + L)^-1 by forward substitution; L[i][j] reads are warp broadcasts, four at a time.  The dot product of
    // row i runs as four independent chains so that its length, not the FMA latency times i, bounds the step.
    float x[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) {
      float a0 = (i == tid) ? 1.f : 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
      const float4* Lrow = reinterpret_cast<const float4*>(L + i * LSTRIDE);
#pragma unroll
      for (int j4 = 0; j4 < (i + 3) / 4; ++j4) {
        const float4 l = Lrow[j4];                      // entries at or right of the diagonal are zero
        a0 -= l.x * x[4 * j4];
        if (4 * j4 + 1 < i) a1 -= l.y * x[4 * j4 + 1];
        if (4 * j4 + 2 < i) a2 -= l.z * x[4 * j4 + 2];
        if (4 * j4 + 3 < i) a3 -= l.w * x[4 * j4 + 3];
      }
      x[i] = (a0 + a1) + (a2 + a3);
    }
#pragma unroll
    for (int i = 0; i < 64; ++i) s.Tm[i * LDS + tid] = __float2bfloat16_rn(x[i]);
  }
  __syncthreads();
  {
    // Tm tile to global for the backward pass
    const int tok = tid >> 1, half = tid & 1;
    float row[32];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(s.Tm + tok * LDS + half * 32 + 2 * i);
      row[2 * i] = __low2float(h); row[2 * i + 1] = __high2float(h);
    }
    store_half_row_global(Tm_out + tile_off, tid, row, 1.f);
  }
  zero_acc(acc);
  mma64<false, false>(s.Tm, s.KBG, acc, warp, lane);
  acc_to_global(acc, w_out + tile_off, 64, warp, lane);
  zero_acc(acc);
  mma64<false, false>(s.Tm, s.VB, acc, warp, lane);
  acc_to_global(acc, u_out + tile_off, 64, warp, lane);
}

// Row sums of a fragment-distributed 64x64 quantity into a shared [64] array (all four warps contribute distinct rows).
__device__ __forceinline__ void frag_row_add(const float (&val)[8][4], float* __restrict__ dst, int warp, int lane, float sign = 1.f) {
  float lo = 0.f, hi = 0.f;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) { lo += val[nt][0] + val[nt][1]; hi += val[nt][2] + val[nt][3]; }
  lo += __shfl_xor_sync(0xffffffffu, lo, 1); lo += __shfl_xor_sync(0xffffffffu, lo, 2);
  hi += __shfl_xor_sync(0xffffffffu, hi, 1); hi += __shfl_xor_sync(0xffffffffu, hi, 2);
  if ((lane & 3) == 0) {
    const int r = 16 * warp + (lane >> 2);
    atomicAdd(&dst[r], sign * lo);
    atomicAdd(&dst[r + 8], sign * hi);
  }
}
// Column sums (over all 64 rows: across lanes of a warp, then across warps through shared atomics).
__device__ __forceinline__ void frag_col_add(const float (&val)[8][4], float* __restrict__ dst, int lane, float sign = 1.f) {
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    float c0 = val[nt][0] + val[nt][2], c1 = val[nt][1] + val[nt][3];
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) { c0 += __shfl_xor_sync(0xffffffffu, c0, o); c1 += __shfl_xor_sync(0xffffffffu, c1, o); }
    if ((lane >> 2) == 0) {
      atomicAdd(&dst[8 * nt + 2 * (lane & 3)], sign * c0);
      atomicAdd(&dst[8 * nt + 2 * (lane & 3) + 1], sign * c1);
    }
  }
}
// One CTA per (chunk, batch, key head); loops over the value heads that share the key head so dq/dk need no atomics.
__global__ void __launch_bounds__(128) gdn_prep_bwd_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                                                           const float* __restrict__ g, const bf16* __restrict__ beta, const bf16* __restrict__ Tm_in,
                                                           const bf16* __restrict__ dw, const bf16* __restrict__ du, const bf16* __restrict__ dP,
                                                           const bf16* __restrict__ dqg, const bf16* __restrict__ dkg, const float* __restrict__ dd,
                                                           bf16* __restrict__ dq, bf16* __restrict__ dk, bf16* __restrict__ dv,
                                                           float* __restrict__ dg, float* __restrict__ dbeta, int S, int Hk, int Hv,
                                                           long long qk_ld, long long v_ld, long long dqk_ld, long long dv_ld) {
  extern __shared__ __align__(16) uint8_t smem_bytes[];
  bf16* sm = reinterpret_cast<bf16*>(smem_bytes);
  PrepSmem s;
  s.Qn = sm; s.Kn = sm + TILE_ELEMS; s.KBG = sm + 2 * TILE_ELEMS; s.VB = sm + 3 * TILE_ELEMS; s.Tm = sm + 4 * TILE_ELEMS;
  bf16* dWs = sm + 5 * TILE_ELEMS;
  bf16* dUs = sm + 6 * TILE_ELEMS;
  bf16* T1 = sm + 7 * TILE_ELEMS;
  bf16* T2 = sm + 8 * TILE_ELEMS;
  float* fl = reinterpret_cast<float*>(sm + 9 * TILE_ELEMS);
  s.gc = fl; s.beta = fl + 64; s.rq = fl + 128; s.rk = fl + 192;
  float* dgc = fl + 256;      // [64]
  float* dbt = fl + 320;      // [64]
  float* dgl = fl + 384;      // [1] gradient of gc_last from kg and the carry
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, NT = gridDim.x, rep = Hv / Hk;
  const int b = blockIdx.y / Hk, hk = blockIdx.y % Hk;
  const long long tok0 = (long long)b * S + (long long)c * 64;
  prep_load_qk(s, q + tok0 * qk_ld + hk * 64, k + tok0 * qk_ld + hk * 64, qk_ld, tid);
  float dQn[8][4], dKn[8][4];
  zero_acc(dQn);
  zero_acc(dKn);
  for (int r = 0; r < rep; ++r) {
    const int hv = hk * rep + r, bh = b * Hv + hv;
    const long long tile_off = ((long long)bh * NT + c) * 4096;
    __syncthreads();                                        // previous head is done with every shared buffer
    prep_load_gates(s, g + tok0 * Hv + hv, beta + tok0 * Hv + hv, Hv, tid);
    if (tid < 64) { dgc[tid] = 0.f; dbt[tid] = 0.f; }
    if (tid == 0) dgl[0] = 0.f;
    load_tile_async(s.Tm, Tm_in + tile_off, 64, tid);
    load_tile_async(dWs, dw + tile_off, 64, tid);
    load_tile_async(dUs, du + tile_off, 64, tid);
    cp_async_commit();
    __syncthreads();
    {
      const int tok = tid >> 1, half = tid & 1;
      const float gct = s.gc[tok], bt = s.beta[tok];
      float row[32];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(s.Kn + tok * LDS + half * 32 + 2 * i);
        row[2 * i] = __low2float(h); row[2 * i + 1] = __high2float(h);
      }
      store_half_row_smem(s.KBG, tid, row, bt * __expf(gct));
      load_half_row(v + tok0 * v_ld + hv * 64, v_ld, tid, row);
      store_half_row_smem(s.VB, tid, row, bt);
    }
    cp_async_wait<0>();
    __syncthreads();
    const float gl = s.gc[63];
    float acc[8][4], t[8][4];
    // ---- d(KBG) = Tm^T dW: contributes to dk, dbeta, dgc ----
    zero_acc(acc);
    mma64<true, false>(s.Tm, dWs, acc, warp, lane);
    frag_from_smem(s.Kn, t, warp, lane);
    {
      float tb[8][4], tg[8][4];
      FRAG_LOOP(nt, e, row, col) {
        const float E = __expf(s.gc[row]);
        tb[nt][e] = acc[nt][e] * E * t[nt][e];                       // d beta_i
        tg[nt][e] = tb[nt][e] * s.beta[row];                          // d gc_i  (= dKBG . kbg)
        dKn[nt][e] += acc[nt][e] * s.beta[row] * E;
      }
      frag_row_add(tb, dbt, warp, lane);
      frag_row_add(tg, dgc, warp, lane);
    }
    // ---- d(VB) = Tm^T dU: dv and dbeta ----
    zero_acc(acc);
    mma64<true, false>(s.Tm, dUs, acc, warp, lane);
    {
      float tb[8][4];
      const bf16* vsrc = v + tok0 * v_ld + hv * 64;
      bf16* dvdst = dv + tok0 * dv_ld + hv * 64;
      const int r0 = 16 * warp + (lane >> 2), cq = 2 * (lane & 3);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
          const int row = r0 + 8 * hrow;
          const __nv_bfloat162 vv = *reinterpret_cast<const __nv_bfloat162*>(vsrc + (long long)row * v_ld + 8 * nt + cq);
          const float a0 = acc[nt][2 * hrow], a1 = acc[nt][2 * hrow + 1];
          tb[nt][2 * hrow] = a0 * __low2float(vv);
          tb[nt][2 * hrow + 1] = a1 * __high2float(vv);
          *reinterpret_cast<__nv_bfloat162*>(dvdst + (long long)row * dv_ld + 8 * nt + cq) = __floats2bfloat162_rn(a0 * s.beta[row], a1 * s.beta[row]);
        }
      }
      frag_row_add(tb, dbt, warp, lane);
    }
    // ---- dTm = dW KBG^T + dU VB^T ;  dM = -Tm^T dTm Tm^T ----
    zero_acc(acc);
    mma64<false, true>(dWs, s.KBG, acc, warp, lane);
    mma64<false, true>(dUs, s.VB, acc, warp, lane);
    acc_to_smem(acc, T1, warp, lane);
    __syncthreads();
    zero_acc(acc);
    mma64<false, true>(T1, s.Tm, acc, warp, lane);           // dTm Tm^T
    acc_to_smem(acc, T2, warp, lane);
    __syncthreads();
    zero_acc(acc);
    mma64<true, false>(s.Tm, T2, acc, warp, lane);           // Tm^T (dTm Tm^T)  = -dM
    // ---- L_ij = beta_i A1_ij Gamma_ij (j < i) ----
    zero_acc(t);
    mma64<false, true>(s.Kn, s.Kn, t, warp, lane);           // A1
    {
      float tb[8][4], tg[8][4], da[8][4];
      FRAG_LOOP(nt, e, row, col) {
        const bool low = col < row;
        const float G = low ? -acc[nt][e] * __expf(s.gc[row] - s.gc[col]) : 0.f;      // dL_ij Gamma_ij
        tb[nt][e] = G * t[nt][e];                                                    // d beta_i
        tg[nt][e] = tb[nt][e] * s.beta[row];                                         // dL_ij L_ij
        da[nt][e] = G * s.beta[row];                                                 // dA1_ij
      }
      frag_row_add(tb, dbt, warp, lane);
      frag_row_add(tg, dgc, warp, lane);
      frag_col_add(tg, dgc, lane, -1.f);
      __syncthreads();                                        // T1 no longer read
      acc_to_smem(da, T1, warp, lane);
    }
    __syncthreads();
    mma64<false, false>(T1, s.Kn, dKn, warp, lane);          // dA1 Kn
    mma64<true, false>(T1, s.Kn, dKn, warp, lane);           // dA1^T Kn
    // ---- P_ij = (q_i.k_j) Gamma_ij (j <= i) ----
    zero_acc(t);
    mma64<false, true>(s.Qn, s.Kn, t, warp, lane);
    frag_from_global(dP + tile_off, acc, warp, lane);
    {
      float tg[8][4], hh[8][4];
      FRAG_LOOP(nt, e, row, col) {
        const float gam = col <= row ? __expf(s.gc[row] - s.gc[col]) : 0.f;
        hh[nt][e] = acc[nt][e] * gam;                                                  // dP_ij Gamma_ij
        tg[nt][e] = hh[nt][e] * t[nt][e];                                              // dP_ij P_ij
      }
      frag_row_add(tg, dgc, warp, lane);
      frag_col_add(tg, dgc, lane, -1.f);
      __syncthreads();                                        // T2 no longer read
      acc_to_smem(hh, T2, warp, lane);
    }
    __syncthreads();
    mma64<false, false>(T2, s.Kn, dQn, warp, lane);          // H Kn
    mma64<true, false>(T2, s.Qn, dKn, warp, lane);           // H^T Qn
    // ---- qg = qn e^gc ;  kg = kn e^(gl - gc) ;  carry = e^gl ----
    frag_from_global(dqg + tile_off, acc, warp, lane);
    frag_from_smem(s.Qn, t, warp, lane);
    {
      float tg[8][4];
      FRAG_LOOP(nt, e, row, col) {
        const float E = __expf(s.gc[row]);
        tg[nt][e] = acc[nt][e] * t[nt][e] * E;
        dQn[nt][e] += acc[nt][e] * E;
      }
      frag_row_add(tg, dgc, warp, lane);
    }
    frag_from_global(dkg + tile_off, acc, warp, lane);
    frag_from_smem(s.Kn, t, warp, lane);
    {
      float tg[8][4];
      float total = 0.f;
      FRAG_LOOP(nt, e, row, col) {
        const float E = __expf(gl - s.gc[row]);
        tg[nt][e] = acc[nt][e] * t[nt][e] * E;
        total += tg[nt][e];
        dKn[nt][e] += acc[nt][e] * E;
      }
      frag_row_add(tg, dgc, warp, lane, -1.f);
      total = warp_sum(total);
      if (lane == 0) atomicAdd(dgl, total);
    }
    __syncthreads();
    // ---- gates out: dg = reverse cumsum of dgc (gc_last also collects dgl and the carry term) ----
    if (tid < 32) {
      float d0 = dgc[2 * tid], d1 = dgc[2 * tid + 1];
      if (tid == 31) d1 += dgl[0] + dd[(long long)bh * NT + c] * __expf(gl);
      float run = d0 + d1;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) { const float dn = __shfl_down_sync(0xffffffffu, run, o); if (tid + o < 32) run += dn; }
      dg[(tok0 + 2 * tid) * Hv + hv] = run;
      dg[(tok0 + 2 * tid + 1) * Hv + hv] = run - d0;
    } else if (tid < 96) {
      dbeta[(tok0 + tid - 32) * Hv + hv] = dbt[tid - 32];
    }
  }
  // ---- L2-norm backward: qn = 0.125 rq q, kn = rk k ----
  {
    const bf16* qsrc = q + tok0 * qk_ld + hk * 64;
    const bf16* ksrc = k + tok0 * qk_ld + hk * 64;
    bf16* dqdst = dq + tok0 * dqk_ld + hk * 64;
    bf16* dkdst = dk + tok0 * dqk_ld + hk * 64;
    const long long ld = qk_ld, dld = dqk_ld;
    const int r0 = 16 * warp + (lane >> 2), cq = 2 * (lane & 3);
#pragma unroll
    for (int hrow = 0; hrow < 2; ++hrow) {
      const int row = r0 + 8 * hrow;
      const float rq = s.rq[row], rk = s.rk[row];
      float qh[16], kh[16], dotq = 0.f, dotk = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const __nv_bfloat162 qq = *reinterpret_cast<const __nv_bfloat162*>(qsrc + row * ld + 8 * nt + cq);
        const __nv_bfloat162 kk = *reinterpret_cast<const __nv_bfloat162*>(ksrc + row * ld + 8 * nt + cq);
        qh[2 * nt] = __low2float(qq) * rq; qh[2 * nt + 1] = __high2float(qq) * rq;
        kh[2 * nt] = __low2float(kk) * rk; kh[2 * nt + 1] = __high2float(kk) * rk;
        dotq += 0.125f * (dQn[nt][2 * hrow] * qh[2 * nt] + dQn[nt][2 * hrow + 1] * qh[2 * nt + 1]);
        dotk += dKn[nt][2 * hrow] * kh[2 * nt] + dKn[nt][2 * hrow + 1] * kh[2 * nt + 1];
      }
      dotq += __shfl_xor_sync(0xffffffffu, dotq, 1); dotq += __shfl_xor_sync(0xffffffffu, dotq, 2);
      dotk += __shfl_xor_sync(0xffffffffu, dotk, 1); dotk += __shfl_xor_sync(0xffffffffu, dotk, 2);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        *reinterpret_cast<__nv_bfloat162*>(dqdst + row * dld + 8 * nt + cq) =
            __floats2bfloat162_rn(rq * (0.125f * dQn[nt][2 * hrow] - qh[2 * nt] * dotq), rq * (0.125f * dQn[nt][2 * hrow + 1] - qh[2 * nt + 1] * dotq));
        *reinterpret_cast<__nv_bfloat162*>(dkdst + row * dld + 8 * nt + cq) =
            __floats2bfloat162_rn(rk * (dKn[nt][2 * hrow] - kh[2 * nt] * dotk), rk * (dKn[nt][2 * hrow + 1] - kh[2 * nt + 1] * dotk));
      }
    }
  }
}

// ---- host ----------------------------------------------------------------------------------------------------------------
// Returns {w, u, P, qg, kg, Tm (bf16 tiles [B*Hv,NT,64,64]), carry [B*Hv,NT] fp32, gc [B*Hv,NT,64] fp32}
std::vector<at::Tensor> gdn_prep_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& g, const at::Tensor& beta) {
  auto token_major = [](const at::Tensor& t) {
    return t.dim() == 4 && t.size(3) == 64 && t.stride(3) == 1 && t.stride(2) == 64 && t.stride(0) == t.size(1) * t.stride(1) && t.stride(1) % 8 == 0 &&
           (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0;
  };
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && token_major(q) && token_major(k) && token_major(v) && q.stride(1) == k.stride(1),
              "gdn_prep_fwd: bf16 [B,S,H,64] tensors with contiguous heads and a common token stride required (views of a packed qkv tensor are fine)");
  TORCH_CHECK(g.scalar_type() == at::kFloat && g.is_contiguous() && beta.scalar_type() == at::kBFloat16 && beta.is_contiguous(), "gdn_prep_fwd: g fp32 / beta bf16 [B,S,Hv]");
  const c10::cuda::CUDAGuard guard(q.device());
  const int64_t B = q.size(0), S = q.size(1), Hk = q.size(2), Hv = v.size(2);
  TORCH_CHECK(S % 64 == 0 && Hv % Hk == 0, "gdn_prep_fwd: sequence must be a multiple of 64 and value heads a multiple of key heads");
  const int64_t NT = S / 64, BH = B * Hv;
  auto opts = q.options();
  std::vector<at::Tensor> out;
  for (int i = 0; i < 6; ++i) out.push_back(at::empty({BH, NT, 64, 64}, opts));
  out.push_back(at::empty({BH, NT}, opts.dtype(at::kFloat)));
  out.push_back(at::empty({BH, NT, 64}, opts.dtype(at::kFloat)));
  const int smem = 5 * TILE_ELEMS * 2 + (64 * 68 + 256) * 4;
  static bool configured = false;
  if (!configured) { C10_CUDA_CHECK(cudaFuncSetAttribute(gdn_prep_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); configured = true; }
  gdn_prep_fwd_kernel<<<dim3((int)NT, (int)BH), 128, smem, at::cuda::getCurrentCUDAStream()>>>(
      (const bf16*)q.data_ptr(), (const bf16*)k.data_ptr(), (const bf16*)v.data_ptr(), g.data_ptr<float>(), (const bf16*)beta.data_ptr(),
      (bf16*)out[0].data_ptr(), (bf16*)out[1].data_ptr(), (bf16*)out[2].data_ptr(), (bf16*)out[3].data_ptr(), (bf16*)out[4].data_ptr(),
      (bf16*)out[5].data_ptr(), out[6].data_ptr<float>(), out[7].data_ptr<float>(), (int)S, (int)Hk, (int)Hv, (long long)q.stride(1), (long long)v.stride(1));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return out;
}

// Returns {dqkv packed bf16 [B,S,(2 Hk + Hv) 64] holding dq | dk | dv per token, dg, dbeta (fp32 [B,S,Hv])}
std::vector<at::Tensor> gdn_prep_bwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& g, const at::Tensor& beta,
                                     const at::Tensor& Tm, const at::Tensor& dw, const at::Tensor& du, const at::Tensor& dP, const at::Tensor& dqg,
                                     const at::Tensor& dkg, const at::Tensor& dd) {
  const c10::cuda::CUDAGuard guard(q.device());
  const int64_t B = q.size(0), S = q.size(1), Hk = q.size(2), Hv = v.size(2), NT = S / 64, BH = B * Hv;
  check_tiles(Tm, BH, NT, "Tm"); check_tiles(dw, BH, NT, "dw"); check_tiles(du, BH, NT, "du"); check_tiles(dP, BH, NT, "dP");
  check_tiles(dqg, BH, NT, "dqg"); check_tiles(dkg, BH, NT, "dkg");
  TORCH_CHECK(dd.scalar_type() == at::kFloat && dd.is_contiguous() && dd.numel() == BH * NT, "gdn_prep_bwd: dd must be fp32 [BH,NT]");
  const int64_t packed = (2 * Hk + Hv) * 64;
  auto dqkv = at::empty({B, S, packed}, q.options());
  bf16* dq_ptr = (bf16*)dqkv.data_ptr();
  bf16* dk_ptr = dq_ptr + Hk * 64;
  bf16* dv_ptr = dq_ptr + 2 * Hk * 64;
  auto dg = at::empty({B, S, Hv}, q.options().dtype(at::kFloat)), dbeta = at::empty({B, S, Hv}, q.options().dtype(at::kFloat));
  const int smem = 9 * TILE_ELEMS * 2 + 400 * 4;
  static bool configured = false;
  if (!configured) { C10_CUDA_CHECK(cudaFuncSetAttribute(gdn_prep_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); configured = true; }
  gdn_prep_bwd_kernel<<<dim3((int)NT, (int)(B * Hk)), 128, smem, at::cuda::getCurrentCUDAStream()>>>(
      (const bf16*)q.data_ptr(), (const bf16*)k.data_ptr(), (const bf16*)v.data_ptr(), g.data_ptr<float>(), (const bf16*)beta.data_ptr(),
      (const bf16*)Tm.data_ptr(), (const bf16*)dw.data_ptr(), (const bf16*)du.data_ptr(), (const bf16*)dP.data_ptr(), (const bf16*)dqg.data_ptr(),
      (const bf16*)dkg.data_ptr(), dd.data_ptr<float>(), dq_ptr, dk_ptr, dv_ptr, dg.data_ptr<float>(),
      dbeta.data_ptr<float>(), (int)S, (int)Hk, (int)Hv, (long long)q.stride(1), (long long)v.stride(1), (long long)packed, (long long)packed);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {dqkv, dg, dbeta};
}

}  // namespace q38
