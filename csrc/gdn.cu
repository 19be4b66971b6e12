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
//                  accumulator registers of four warps (warp w owns k-rows 16w..16w+15); every product is a 64x64x64
//                  bf16 mma.sync with fp32 accumulation; chunk operands are prefetched with cp.async one chunk ahead.
//                  The chain per chunk is latency bound (three dependent products), which is why this pass uses
//                  register-resident warp MMAs instead of the TMEM round trips of tcgen05.
//   gdn_scan_bwd   the reverse pass: dS' -> (dw, du, dP, dqg, dkg, dd) per chunk and dS.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"
#include "host.h"

namespace q38 {

constexpr int C64 = 64, LDS = 72;                 // 64x64 bf16 tiles padded to 72 columns (bank-conflict-free fragment loads)
constexpr int TILE_ELEMS = C64 * LDS;
using bf16 = __nv_bfloat16;

__device__ __forceinline__ uint32_t pack2(bf16 a, bf16 b) {
  return (uint32_t)__bfloat16_as_ushort(a) | ((uint32_t)__bfloat16_as_ushort(b) << 16);
}

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// acc[64x64] += A * B with four warps; warp w owns rows 16w..16w+15.
//   A(i,k) = TA ? As[k*LDS + i] : As[i*LDS + k]          B(k,n) = TB ? Bs[n*LDS + k] : Bs[k*LDS + n]
// Accumulator element acc[nt][e]: row = 16w + lane/4 + 8*(e>>1), col = 8nt + 2*(lane%4) + (e&1).
template <bool TA, bool TB>
__device__ __forceinline__ void mma64(const bf16* __restrict__ As, const bf16* __restrict__ Bs, float (&acc)[8][4], int warp, int lane) {
  const int r = 16 * warp + (lane >> 2), cq = 2 * (lane & 3);
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    const int k0 = 16 * ks + cq;
    uint32_t a[4];
    if (!TA) {
      a[0] = *reinterpret_cast<const uint32_t*>(As + r * LDS + k0);
      a[1] = *reinterpret_cast<const uint32_t*>(As + (r + 8) * LDS + k0);
      a[2] = *reinterpret_cast<const uint32_t*>(As + r * LDS + k0 + 8);
      a[3] = *reinterpret_cast<const uint32_t*>(As + (r + 8) * LDS + k0 + 8);
    } else {
      a[0] = pack2(As[k0 * LDS + r], As[(k0 + 1) * LDS + r]);
      a[1] = pack2(As[k0 * LDS + r + 8], As[(k0 + 1) * LDS + r + 8]);
      a[2] = pack2(As[(k0 + 8) * LDS + r], As[(k0 + 9) * LDS + r]);
      a[3] = pack2(As[(k0 + 8) * LDS + r + 8], As[(k0 + 9) * LDS + r + 8]);
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const int n = 8 * nt + (lane >> 2);
      uint32_t b0, b1;
      if (TB) {
        b0 = *reinterpret_cast<const uint32_t*>(Bs + n * LDS + k0);
        b1 = *reinterpret_cast<const uint32_t*>(Bs + n * LDS + k0 + 8);
      } else {
        b0 = pack2(Bs[k0 * LDS + n], Bs[(k0 + 1) * LDS + n]);
        b1 = pack2(Bs[(k0 + 8) * LDS + n], Bs[(k0 + 9) * LDS + n]);
      }
      mma16816(acc[nt], a, b0, b1);
    }
  }
}

__device__ __forceinline__ void zero_acc(float (&acc)[8][4]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
}

// Accumulator fragment -> padded bf16 tile in shared memory (row-major).
__device__ __forceinline__ void acc_to_smem(const float (&acc)[8][4], bf16* __restrict__ dst, int warp, int lane) {
  const int r = 16 * warp + (lane >> 2), cq = 2 * (lane & 3);
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    *reinterpret_cast<__nv_bfloat162*>(dst + r * LDS + 8 * nt + cq) = __floats2bfloat162_rn(acc[nt][0], acc[nt][1]);
    *reinterpret_cast<__nv_bfloat162*>(dst + (r + 8) * LDS + 8 * nt + cq) = __floats2bfloat162_rn(acc[nt][2], acc[nt][3]);
  }
}

// Accumulator fragment -> dense [64,64] bf16 tile in global memory with row stride `ld` elements.
__device__ __forceinline__ void acc_to_global(const float (&acc)[8][4], bf16* __restrict__ dst, long long ld, int warp, int lane, float scale = 1.f) {
  const int r = 16 * warp + (lane >> 2), cq = 2 * (lane & 3);
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    *reinterpret_cast<__nv_bfloat162*>(dst + (long long)r * ld + 8 * nt + cq) = __floats2bfloat162_rn(acc[nt][0] * scale, acc[nt][1] * scale);
    *reinterpret_cast<__nv_bfloat162*>(dst + (long long)(r + 8) * ld + 8 * nt + cq) = __floats2bfloat162_rn(acc[nt][2] * scale, acc[nt][3] * scale);
  }
}

// cp.async of a dense [64,64] bf16 tile (row stride `ld` elements, 16-byte aligned rows) into a padded shared tile.
__device__ __forceinline__ void load_tile_async(bf16* __restrict__ dst, const bf16* __restrict__ src, long long ld, int tid) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int chunk = tid + 128 * i;                 // 512 chunks of 16 bytes
    const int row = chunk >> 3, col = (chunk & 7) * 8;
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst + row * LDS + col));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src + (long long)row * ld + col) : "memory");
  }
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// ---------------------------------------------------------------------------------------------------------------------
// Forward scan.  Chunk operands w,u,P,qg,kg: [BH, NT, 64, 64] bf16; dch: [BH, NT] fp32.
// Outputs: o [B, S, H, 64] bf16 (token-major), vnew [BH, NT, 64, 64] bf16, states [BH, NT, 64, 64] bf16 (chunk-start S).
// ---------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) gdn_scan_fwd_kernel(const bf16* __restrict__ w, const bf16* __restrict__ u, const bf16* __restrict__ P,
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
    for (int t = 0; t < 5; ++t) load_tile_async(sm + (buf * 5 + t) * TILE_ELEMS, srcs[t] + (long long)c * tile, 64, tid);
    cp_async_commit();
  };
  float S[8][4];
  zero_acc(S);
  prefetch(0, 0);
  for (int c = 0; c < NT; ++c) {
    const int buf = c & 1;
    if (c + 1 < NT) { prefetch(c + 1, buf ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    acc_to_smem(S, Sb, warp, lane);
    acc_to_global(S, states + ((long long)bh * NT + c) * tile, 64, warp, lane);
    __syncthreads();                                   // operand tiles of chunk c and Sb are visible
    const bf16* Wt = sm + (buf * 5 + 0) * TILE_ELEMS;
    const bf16* Ut = Wt + TILE_ELEMS;
    const bf16* Pt = Ut + TILE_ELEMS;
    const bf16* Qt = Pt + TILE_ELEMS;
    const bf16* Kt = Qt + TILE_ELEMS;
    float acc[8][4];
    zero_acc(acc);
    mma64<false, false>(Wt, Sb, acc, warp, lane);      // w S
    {
      const int r = 16 * warp + (lane >> 2), cq = 2 * (lane & 3);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const __nv_bfloat162 u0 = *reinterpret_cast<const __nv_bfloat162*>(Ut + r * LDS + 8 * nt + cq);
        const __nv_bfloat162 u1 = *reinterpret_cast<const __nv_bfloat162*>(Ut + (r + 8) * LDS + 8 * nt + cq);
        acc[nt][0] = __low2float(u0) - acc[nt][0]; acc[nt][1] = __high2float(u0) - acc[nt][1];
        acc[nt][2] = __low2float(u1) - acc[nt][2]; acc[nt][3] = __high2float(u1) - acc[nt][3];
      }
    }
    acc_to_smem(acc, Vn, warp, lane);                  // v_new (bf16) for the two products below
    acc_to_global(acc, vnew + ((long long)bh * NT + c) * tile, 64, warp, lane);
    float out[8][4];
    zero_acc(out);
    mma64<false, false>(Qt, Sb, out, warp, lane);      // qg S
    __syncthreads();                                   // Vn complete
    mma64<false, false>(Pt, Vn, out, warp, lane);      // + P v_new
    acc_to_global(out, o + (((long long)b * NT * 64 + (long long)c * 64) * H + hv) * 64, (long long)H * 64, warp, lane);
    const float d = dch[(long long)bh * NT + c];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) { S[nt][0] *= d; S[nt][1] *= d; S[nt][2] *= d; S[nt][3] *= d; }
    mma64<true, false>(Kt, Vn, S, warp, lane);         // + kg^T v_new
    __syncthreads();                                   // everyone is done with Sb, Vn and this buffer
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Backward scan (reverse over chunks).  Inputs: the forward operands, vnew, states, and do [B,S,H,64].
// Outputs per chunk: dw, du, dP, dqg, dkg [BH,NT,64,64] bf16 and dd [BH,NT] fp32.
// ---------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) gdn_scan_bwd_kernel(const bf16* __restrict__ w, const bf16* __restrict__ P, const bf16* __restrict__ qg,
                                                           const bf16* __restrict__ kg, const float* __restrict__ dch, const bf16* __restrict__ vnew,
                                                           const bf16* __restrict__ states, const bf16* __restrict__ dout, bf16* __restrict__ dw,
                                                           bf16* __restrict__ du, bf16* __restrict__ dP, bf16* __restrict__ dqg, bf16* __restrict__ dkg,
                                                           float* __restrict__ dd, int NT, int H) {
  extern __shared__ __align__(16) uint8_t smem_bytes[];
  bf16* sm = reinterpret_cast<bf16*>(smem_bytes);
  // two buffers of seven tiles: w, P, qg, kg, vnew, state, do ; then dS (bf16) and dv_new (bf16)
  bf16* dSb = sm + 14 * TILE_ELEMS;
  bf16* dVn = dSb + TILE_ELEMS;
  __shared__ float red[4];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x, b = bh / H, hv = bh % H;
  const long long tile = 64 * 64, base = (long long)bh * NT * tile;
  auto prefetch = [&](int c, int buf) {
    bf16* dst = sm + buf * 7 * TILE_ELEMS;
    load_tile_async(dst + 0 * TILE_ELEMS, w + base + (long long)c * tile, 64, tid);
    load_tile_async(dst + 1 * TILE_ELEMS, P + base + (long long)c * tile, 64, tid);
    load_tile_async(dst + 2 * TILE_ELEMS, qg + base + (long long)c * tile, 64, tid);
    load_tile_async(dst + 3 * TILE_ELEMS, kg + base + (long long)c * tile, 64, tid);
    load_tile_async(dst + 4 * TILE_ELEMS, vnew + base + (long long)c * tile, 64, tid);
    load_tile_async(dst + 5 * TILE_ELEMS, states + base + (long long)c * tile, 64, tid);
    load_tile_async(dst + 6 * TILE_ELEMS, dout + (((long long)b * NT * 64 + (long long)c * 64) * H + hv) * 64, (long long)H * 64, tid);
    cp_async_commit();
  };
  float dS[8][4];
  zero_acc(dS);
  prefetch(NT - 1, (NT - 1) & 1);
  for (int c = NT - 1; c >= 0; --c) {
    const int buf = c & 1;
    if (c > 0) { prefetch(c - 1, buf ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    acc_to_smem(dS, dSb, warp, lane);
    __syncthreads();
    const bf16* Wt = sm + buf * 7 * TILE_ELEMS;
    const bf16* Pt = Wt + TILE_ELEMS;
    const bf16* Qt = Pt + TILE_ELEMS;
    const bf16* Kt = Qt + TILE_ELEMS;
    const bf16* Vt = Kt + TILE_ELEMS;
    const bf16* St = Vt + TILE_ELEMS;
    const bf16* Dt = St + TILE_ELEMS;
    const long long off = base + (long long)c * tile;
    float acc[8][4];
    // dv_new = P^T dO + kg dS'
    zero_acc(acc);
    mma64<true, false>(Pt, Dt, acc, warp, lane);
    mma64<false, false>(Kt, dSb, acc, warp, lane);
    acc_to_smem(acc, dVn, warp, lane);
    acc_to_global(acc, du + off, 64, warp, lane);
    // dd = <dS', S>   (fragment of S read from the state tile in accumulator layout)
    {
      const int r = 16 * warp + (lane >> 2), cq = 2 * (lane & 3);
      float part = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const __nv_bfloat162 s0 = *reinterpret_cast<const __nv_bfloat162*>(St + r * LDS + 8 * nt + cq);
        const __nv_bfloat162 s1 = *reinterpret_cast<const __nv_bfloat162*>(St + (r + 8) * LDS + 8 * nt + cq);
        part += dS[nt][0] * __low2float(s0) + dS[nt][1] * __high2float(s0) + dS[nt][2] * __low2float(s1) + dS[nt][3] * __high2float(s1);
      }
      part = warp_sum(part);
      if (lane == 0) red[warp] = part;
    }
    // dqg = dO S^T ;  dkg = v_new dS'^T ;  dP = tril(dO v_new^T)
    zero_acc(acc);
    mma64<false, true>(Dt, St, acc, warp, lane);
    acc_to_global(acc, dqg + off, 64, warp, lane);
    zero_acc(acc);
    mma64<false, true>(Vt, dSb, acc, warp, lane);
    acc_to_global(acc, dkg + off, 64, warp, lane);
    zero_acc(acc);
    mma64<false, true>(Dt, Vt, acc, warp, lane);
    {
      const int r = 16 * warp + (lane >> 2), cq = 2 * (lane & 3);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int col = 8 * nt + cq;
        if (col > r) acc[nt][0] = 0.f;
        if (col + 1 > r) acc[nt][1] = 0.f;
        if (col > r + 8) acc[nt][2] = 0.f;
        if (col + 1 > r + 8) acc[nt][3] = 0.f;
      }
    }
    acc_to_global(acc, dP + off, 64, warp, lane);
    __syncthreads();                                    // dVn and red[] complete
    if (tid == 0) dd[(long long)bh * NT + c] = red[0] + red[1] + red[2] + red[3];
    // dw = -dv_new S^T
    zero_acc(acc);
    mma64<false, true>(dVn, St, acc, warp, lane);
    acc_to_global(acc, dw + off, 64, warp, lane, -1.f);
    // dS = d dS' + qg^T dO - w^T dv_new
    const float d = dch[(long long)bh * NT + c];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) { dS[nt][0] *= d; dS[nt][1] *= d; dS[nt][2] *= d; dS[nt][3] *= d; }
    mma64<true, false>(Qt, Dt, dS, warp, lane);
    zero_acc(acc);
    mma64<true, false>(Wt, dVn, acc, warp, lane);
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) { dS[nt][0] -= acc[nt][0]; dS[nt][1] -= acc[nt][1]; dS[nt][2] -= acc[nt][2]; dS[nt][3] -= acc[nt][3]; }
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
  gdn_scan_fwd_kernel<<<(int)BH, 128, smem, at::cuda::getCurrentCUDAStream()>>>(
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
  gdn_scan_bwd_kernel<<<(int)BH, 128, smem, at::cuda::getCurrentCUDAStream()>>>(
      (const bf16*)w.data_ptr(), (const bf16*)P.data_ptr(), (const bf16*)qg.data_ptr(), (const bf16*)kg.data_ptr(), dch.data_ptr<float>(),
      (const bf16*)vnew.data_ptr(), (const bf16*)states.data_ptr(), (const bf16*)dout.data_ptr(), (bf16*)dw.data_ptr(), (bf16*)du.data_ptr(),
      (bf16*)dP.data_ptr(), (bf16*)dqg.data_ptr(), (bf16*)dkg.data_ptr(), dd.data_ptr<float>(), (int)NT, (int)H);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {dw, du, dP, dqg, dkg, dd};
}

}  // namespace q38
