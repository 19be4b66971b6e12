// Mixture-of-experts kernels: routing, deterministic counting sort by expert, row gather / weighted combine, and the
// grouped tcgen05 GEMMs over the expert-sorted rows (no padding, no host synchronisation).
//
// Sorted order = by expert, then by pair index (pair = token * k + slot): what a stable sort gives, so results do not
// depend on scheduling.  A tile schedule (expert, first row, valid rows per 128-row tile) is produced on the device; the
// grouped GEMM launches an upper bound of tiles and surplus CTAs exit.
//
// Grouped GEMM epilogues:
//   EPI_STORE    C[row, n]  = A[row,:] . B_e[n,:]                       bf16 out         (down projection, dgrad)
//   EPI_SWIGLU   two accumulators (gate, up) -> gu[row, 2f] and hmid[row, f] = silu(g) * u with eager bf16 rounding points
//   EPI_DSWIGLU  accumulator = d(hmid); reads gu, writes d(gu)[row, 2f]  (SwiGLU backward fused into the dgrad GEMM)
//   EPI_WGRAD    C_e[m, n] += sum over the expert's rows of A[row, m] B[row, n]   fp32 accumulate; the ragged last K block
//                is zero-masked in shared memory before the MMA reads it
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "ptx.cuh"
#include "host.h"
#include "q38_noalloc.h"

namespace q38 {

// =====================================================================================================================
// Routing
// =====================================================================================================================
constexpr int MAX_TOPK = 8;

// One warp per token, E <= 64 (two logits per lane).  probs = softmax(logits) in fp32, top-k, renormalise, round the
// weights to bf16 (the logits' dtype).  Also accumulates assignment counts and probability sums for the balancing loss.
__global__ void __launch_bounds__(256) moe_route_fwd_kernel(const __nv_bfloat16* __restrict__ logits, int T, int E, int K,
                                                            float* __restrict__ top_w, int* __restrict__ top_idx,
                                                            float* __restrict__ probs_out, float* __restrict__ counts,
                                                            float* __restrict__ prob_sum) {
  __shared__ float s_cnt[64], s_ps[64];
  if (threadIdx.x < 64) { s_cnt[threadIdx.x] = 0.f; s_ps[threadIdx.x] = 0.f; }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + warp;
  if (t < T) {
    const int e0 = lane, e1 = lane + 32;
    const float l0 = e0 < E ? __bfloat162float(logits[(size_t)t * E + e0]) : -INFINITY;
    const float l1 = e1 < E ? __bfloat162float(logits[(size_t)t * E + e1]) : -INFINITY;
    const float mx = warp_max(fmaxf(l0, l1));
    float p0 = e0 < E ? __expf(l0 - mx) : 0.f, p1 = e1 < E ? __expf(l1 - mx) : 0.f;
    const float denom = warp_sum(p0 + p1);
    p0 /= denom; p1 /= denom;
    if (e0 < E) { probs_out[(size_t)t * E + e0] = p0; atomicAdd(&s_ps[e0], p0); }
    if (e1 < E) { probs_out[(size_t)t * E + e1] = p1; atomicAdd(&s_ps[e1], p1); }
    float a0 = e0 < E ? p0 : -1.f, a1 = e1 < E ? p1 : -1.f;
    float sel_p[MAX_TOPK]; int sel_e[MAX_TOPK];
    float total = 0.f;
    for (int j = 0; j < K; ++j) {
      // arg-max over 64 candidates; ties resolve to the lowest expert index
      float best = a0; int be = e0;
      if (a1 > best) { best = a1; be = e1; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, be, o);
        if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
      }
      sel_p[j] = best; sel_e[j] = be; total += best;
      if (be == e0) a0 = -1.f;
      if (be == e1) a1 = -1.f;
    }
    if (lane == 0) {
      for (int j = 0; j < K; ++j) {
        top_w[(size_t)t * K + j] = bf16_round(sel_p[j] / total);
        top_idx[(size_t)t * K + j] = sel_e[j];
        atomicAdd(&s_cnt[sel_e[j]], 1.f);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x < E) { atomicAdd(&counts[threadIdx.x], s_cnt[threadIdx.x]); atomicAdd(&prob_sum[threadIdx.x], s_ps[threadIdx.x]); }
}

// dlogits = probs * (dp - <dp, probs>),  dp_e = dprob_sum_e + [e selected as slot j] (dw_j - <dw, w>) / s
__global__ void __launch_bounds__(256) moe_route_bwd_kernel(const float* __restrict__ probs, const int* __restrict__ top_idx,
                                                            const float* __restrict__ top_w, const float* __restrict__ d_top_w,
                                                            const float* __restrict__ d_prob_sum, int T, int E, int K,
                                                            __nv_bfloat16* __restrict__ dlogits) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + warp;
  if (t >= T) return;
  const int e0 = lane, e1 = lane + 32;
  const float p0 = e0 < E ? probs[(size_t)t * E + e0] : 0.f, p1 = e1 < E ? probs[(size_t)t * E + e1] : 0.f;
  float dp0 = (d_prob_sum && e0 < E) ? d_prob_sum[e0] : 0.f, dp1 = (d_prob_sum && e1 < E) ? d_prob_sum[e1] : 0.f;
  // lane j < K holds slot j (expert id and incoming gradient), read once; the three passes below take them by shuffle instead
  // of re-reading global memory in every iteration (the dependent loads were what this kernel waited for)
  const int my_e = lane < K ? top_idx[(size_t)t * K + lane] : 0;
  const float my_dw = lane < K ? d_top_w[(size_t)t * K + lane] : 0.f;
  float s = 0.f, dot = 0.f;
  for (int j = 0; j < K; ++j) {
    const int e = __shfl_sync(0xffffffffu, my_e, j);
    s += __shfl_sync(0xffffffffu, e < 32 ? p0 : p1, e & 31);
  }
  for (int j = 0; j < K; ++j) {
    const int e = __shfl_sync(0xffffffffu, my_e, j);
    const float pe = __shfl_sync(0xffffffffu, e < 32 ? p0 : p1, e & 31);
    dot += __shfl_sync(0xffffffffu, my_dw, j) * (pe / s);          // unrounded weight for the derivative
  }
  for (int j = 0; j < K; ++j) {
    const int e = __shfl_sync(0xffffffffu, my_e, j);
    const float g = (__shfl_sync(0xffffffffu, my_dw, j) - dot) / s;
    if (e == e0) dp0 += g;
    if (e == e1) dp1 += g;
  }
  const float inner = warp_sum(dp0 * p0 + dp1 * p1);
  if (e0 < E) dlogits[(size_t)t * E + e0] = __float2bfloat16_rn(p0 * (dp0 - inner));
  if (e1 < E) dlogits[(size_t)t * E + e1] = __float2bfloat16_rn(p1 * (dp1 - inner));
}

// =====================================================================================================================
// Deterministic counting sort of the P = T*k (token, slot) pairs by expert
// =====================================================================================================================
constexpr int SORT_THREADS = 256, SORT_ITERS = 4, SORT_CHUNK = SORT_THREADS * SORT_ITERS;

// A pair whose expert id lies outside [0, E) is skipped by the histogram and the scatter (it is counted nowhere, its
// inv_perm entry becomes -1 and the tail of perm stays unwritten) and ERR_BOUNDS is recorded when an error word is given.
__global__ void __launch_bounds__(SORT_THREADS) moe_hist_kernel(const int* __restrict__ expert_of_pair, int P, int E, int* __restrict__ block_counts,
                                                                int* __restrict__ err) {
  __shared__ int cnt[64];
  if (threadIdx.x < 64) cnt[threadIdx.x] = 0;
  __syncthreads();
  for (int it = 0; it < SORT_ITERS; ++it) {
    const int i = blockIdx.x * SORT_CHUNK + it * SORT_THREADS + threadIdx.x;
    if (i < P) {
      const int e = expert_of_pair[i];
      if ((unsigned)e < (unsigned)E) atomicAdd(&cnt[e], 1);
      else report_error(err, ERR_BOUNDS);
    }
  }
  __syncthreads();
  if (threadIdx.x < E) block_counts[blockIdx.x * E + threadIdx.x] = cnt[threadIdx.x];
}

// Single CTA: per-expert totals, expert offsets, per-block bases, and the 128-row tile schedule.
// sched layout: [0] = number of tiles; then per tile (expert, row0, rows).  offsets has E+1 entries.
__global__ void __launch_bounds__(64) moe_scan_kernel(int* __restrict__ block_counts, int nblocks, int E, int* __restrict__ offsets,
                                                      int* __restrict__ sched, int max_tiles, int tile_rows) {
  __shared__ int tot[64], off[65], tstart[65];
  const int e = threadIdx.x;
  int total = 0;
  if (e < E) {
    for (int b = 0; b < nblocks; ++b) { const int c = block_counts[b * E + e]; block_counts[b * E + e] = total; total += c; }
    tot[e] = total;
  }
  __syncthreads();
  if (e == 0) {
    int acc = 0, tacc = 0;
    for (int i = 0; i < E; ++i) { off[i] = acc; tstart[i] = tacc; acc += tot[i]; tacc += (tot[i] + tile_rows - 1) / tile_rows; }
    off[E] = acc; tstart[E] = tacc;
    sched[0] = tacc;
  }
  __syncthreads();
  if (e < E) {
    offsets[e] = off[e];
    if (e == E - 1) offsets[E] = off[E];
    for (int b = 0; b < nblocks; ++b) block_counts[b * E + e] += off[e];          // base position of (block, expert)
    const int ntile = (tot[e] + tile_rows - 1) / tile_rows;
    for (int i = 0; i < ntile; ++i) {
      const int tile = tstart[e] + i;
      if (tile < max_tiles) {
        sched[1 + 3 * tile] = e;
        sched[2 + 3 * tile] = off[e] + i * tile_rows;
        sched[3 + 3 * tile] = min(tile_rows, tot[e] - i * tile_rows);
      }
    }
  }
  // tiles past the end carry zero rows
  for (int tile = tstart[E] + threadIdx.x; tile < max_tiles; tile += blockDim.x) { sched[1 + 3 * tile] = 0; sched[2 + 3 * tile] = 0; sched[3 + 3 * tile] = 0; }
}

__global__ void __launch_bounds__(SORT_THREADS) moe_scatter_kernel(const int* __restrict__ expert_of_pair, int P, int E,
                                                                   const int* __restrict__ block_base, int* __restrict__ perm, int* __restrict__ inv_perm) {
  __shared__ int cursor[64];
  __shared__ int warp_cnt[SORT_THREADS / 32][64];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x < 64) cursor[threadIdx.x] = threadIdx.x < E ? block_base[blockIdx.x * E + threadIdx.x] : 0;
  for (int it = 0; it < SORT_ITERS; ++it) {
    for (int i = threadIdx.x; i < (SORT_THREADS / 32) * 64; i += SORT_THREADS) (&warp_cnt[0][0])[i] = 0;
    __syncthreads();
    const int i = blockIdx.x * SORT_CHUNK + it * SORT_THREADS + threadIdx.x;
    int e = i < P ? expert_of_pair[i] : -1;
    const bool valid = (unsigned)e < (unsigned)E;
    if (!valid) {
      if (i < P) inv_perm[i] = -1;
      e = -1;
    }
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(same & ((1u << lane) - 1));
    if (valid && rank == 0) warp_cnt[warp][e] = __popc(same);
    __syncthreads();
    if (valid) {
      int before = cursor[e];
      for (int w = 0; w < warp; ++w) before += warp_cnt[w][e];
      const int pos = before + rank;
      perm[pos] = i;
      inv_perm[i] = pos;
    }
    __syncthreads();
    if (threadIdx.x < E) {
      int add = 0;
      for (int w = 0; w < SORT_THREADS / 32; ++w) add += warp_cnt[w][threadIdx.x];
      cursor[threadIdx.x] += add;
    }
    __syncthreads();
  }
}

// x_sorted[pos, :] = x[perm[pos] / k, :]   (one warp per sorted row, 16-byte copies; h % 8 == 0)
__global__ void __launch_bounds__(256) moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ perm, int P, int K, int h,
                                                         __nv_bfloat16* __restrict__ out) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= P) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(perm[row] / K) * h);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)row * h);
  for (int i = lane; i < h / 8; i += 32) dst[i] = src[i];
}

// out[t,:] = sum_j w[t,j] * bf16(y_sorted[inv_perm[t*k+j], :])  (+ extra[t,:] * extra_scale[t])   fixed slot order, no atomics
__global__ void __launch_bounds__(256) moe_combine_fwd_kernel(const __nv_bfloat16* __restrict__ y_sorted, const int* __restrict__ inv_perm,
                                                              const float* __restrict__ top_w, int T, int K, int h,
                                                              __nv_bfloat16* __restrict__ out) {
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= T) return;
  for (int i = lane; i < h / 2; i += 32) {
    float a0 = 0.f, a1 = 0.f;
    for (int j = 0; j < K; ++j) {
      const __nv_bfloat162 v = reinterpret_cast<const __nv_bfloat162*>(y_sorted + (size_t)inv_perm[(size_t)t * K + j] * h)[i];
      const float w = top_w[(size_t)t * K + j];
      // the eager path rounds each weighted row to bf16 before summing over slots
      a0 += bf16_round(__low2float(v) * w);
      a1 += bf16_round(__high2float(v) * w);
    }
    reinterpret_cast<__nv_bfloat162*>(out + (size_t)t * h)[i] = __floats2bfloat162_rn(a0, a1);
  }
}

// dy_sorted[pos,:] = w[pair] * dout[token,:];  dw[pair] = <dout[token,:], y_sorted[pos,:]>      (one warp per pair)
__global__ void __launch_bounds__(256) moe_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ y_sorted,
                                                              const int* __restrict__ inv_perm, const float* __restrict__ top_w, int T, int K, int h,
                                                              __nv_bfloat16* __restrict__ dy_sorted, float* __restrict__ d_top_w) {
  const int pair = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (pair >= T * K) return;
  const int t = pair / K, pos = inv_perm[pair];
  const float w = top_w[pair];
  float dot = 0.f;
  for (int i = lane; i < h / 2; i += 32) {
    const __nv_bfloat162 d = reinterpret_cast<const __nv_bfloat162*>(dout + (size_t)t * h)[i];
    const __nv_bfloat162 y = reinterpret_cast<const __nv_bfloat162*>(y_sorted + (size_t)pos * h)[i];
    dot += __low2float(d) * __low2float(y) + __high2float(d) * __high2float(y);
    reinterpret_cast<__nv_bfloat162*>(dy_sorted + (size_t)pos * h)[i] = __floats2bfloat162_rn(__low2float(d) * w, __high2float(d) * w);
  }
  dot = warp_sum(dot);
  if (lane == 0) d_top_w[pair] = dot;
}

// dx[t,:] = sum_j dx_sorted[inv_perm[t*k+j], :]
__global__ void __launch_bounds__(256) moe_unpermute_sum_kernel(const __nv_bfloat16* __restrict__ dx_sorted, const int* __restrict__ inv_perm,
                                                                int T, int K, int h, __nv_bfloat16* __restrict__ dx) {
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= T) return;
  for (int i = lane; i < h / 2; i += 32) {
    float a0 = 0.f, a1 = 0.f;
    for (int j = 0; j < K; ++j) {
      const __nv_bfloat162 v = reinterpret_cast<const __nv_bfloat162*>(dx_sorted + (size_t)inv_perm[(size_t)t * K + j] * h)[i];
      a0 += __low2float(v); a1 += __high2float(v);
    }
    reinterpret_cast<__nv_bfloat162*>(dx + (size_t)t * h)[i] = __floats2bfloat162_rn(a0, a1);
  }
}

// =====================================================================================================================
// Grouped tcgen05 GEMM
// =====================================================================================================================
enum { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_DSWIGLU = 2, EPI_WGRAD = 3 };

// 16 consecutive bf16 values to a 32-byte aligned address as two 16-byte stores
__device__ __forceinline__ void store16_bf16(__nv_bfloat16* dst, const float (&v)[16]) {
  uint32_t w[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
    w[e] = *reinterpret_cast<uint32_t*>(&h);
  }
  reinterpret_cast<uint4*>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
  reinterpret_cast<uint4*>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
}
constexpr int G_BM = 128, G_BK = 64, G_THREADS = 192;

struct GroupedArgs {
  const int* sched;        // tile schedule (EPI_STORE / SWIGLU / DSWIGLU)
  const int* offsets;      // expert row offsets [E+1] (EPI_WGRAD)
  int bn;                  // UMMA N (multiple of 16, <= 256); for SWIGLU the expert width f
  int bn_alloc;            // rows of the B tile in shared memory: bn, rounded up to whole 64-wide boxes when B is MN-major
  int stages;
  int K;                   // reduction length (not used by WGRAD)
  int N;                   // valid output columns per expert
  int b_rows_per_expert;   // rows of the B tensor map per expert
  void* out0; long long ld0;        // main output
  void* out1; long long ld1;        // SWIGLU: gu [P, 2f];  DSWIGLU: gu input
  long long c_expert_stride;        // WGRAD: elements between experts in C
  int M;                            // WGRAD: rows of C per expert
  int* err;
  // Expert parallelism (EPI_STORE only): output row `row` is stored into rank ret_rank[row]'s buffer at row ret_row[row].
  const int* ret_rank; const int* ret_row;
  void* peer_out[16];
};

template <int EPI, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(G_THREADS) grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                                                                 GroupedArgs p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  const int nacc = EPI == EPI_SWIGLU ? 2 : 1;
  const int A_BYTES = G_BM * G_BK * 2, B_BYTES = nacc * p.bn_alloc * G_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.stages * STAGE_BYTES);
  uint64_t* empty = full + p.stages;
  uint64_t* acc_ready = empty + p.stages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ---- which problem is this CTA? ----
  int expert, a_row0, rows_valid, k_begin, num_kb, m0 = 0;
  const int n0 = blockIdx.y * p.bn;
  if (EPI == EPI_WGRAD) {
    expert = blockIdx.z;
    k_begin = p.offsets[expert];
    const int cnt = p.offsets[expert + 1] - k_begin;
    if (cnt <= 0) return;
    num_kb = (cnt + G_BK - 1) / G_BK;
    m0 = blockIdx.x * G_BM;
    a_row0 = 0; rows_valid = cnt;
  } else {
    const int tile = blockIdx.x;
    if (tile >= p.sched[0]) return;
    expert = p.sched[1 + 3 * tile]; a_row0 = p.sched[2 + 3 * tile]; rows_valid = p.sched[3 + 3 * tile];
    if (rows_valid <= 0) return;
    k_begin = 0;
    num_kb = (p.K + G_BK - 1) / G_BK;
  }
  const uint32_t tmem_cols = (nacc * p.bn <= 32) ? 32 : (nacc * p.bn <= 64) ? 64 : (nacc * p.bn <= 128) ? 128 : (nacc * p.bn <= 256) ? 256 : 512;

  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&tmA);
    ptx::prefetch_tensormap(&tmB);
    for (int s = 0; s < p.stages; ++s) { ptx::mbar_init(&full[s], 1); ptx::mbar_init(&empty[s], 1); }
    ptx::mbar_init(acc_ready, 1);
    ptx::fence_barrier_init();
  }
  if (warp == 1) { ptx::tmem_alloc(tmem_slot, tmem_cols); ptx::tmem_relinquish(); }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int b_row_base = expert * p.b_rows_per_expert;

  if (warp == 0) {
    if (ptx::elect_one()) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % p.stages, round = kb / p.stages;
        if (!ptx::mbar_wait(&empty[s], (round & 1) ^ 1, 1u << 20)) { report_error(p.err, ERR_MMA_WAIT); break; }
        uint8_t* a_dst = smem + s * STAGE_BYTES;
        uint8_t* b_dst = a_dst + A_BYTES;
        ptx::mbar_expect_tx(&full[s], STAGE_BYTES);
        const int k0 = k_begin + kb * G_BK;
        if (A_MN) {
#pragma unroll
          for (int i = 0; i < G_BM / 64; ++i) ptx::tma_load_3d(a_dst + i * 8192, &tmA, &full[s], m0 + 64 * i, k0, 0);
        } else {
          ptx::tma_load_3d(a_dst, &tmA, &full[s], k0, a_row0, 0);
        }
        if (EPI == EPI_WGRAD) {            // B MN-major, rows = the same sorted rows as A
          for (int i = 0; i < p.bn_alloc / 64; ++i) ptx::tma_load_3d(b_dst + i * 8192, &tmB, &full[s], n0 + 64 * i, k0, 0);
        } else if (B_MN) {                 // B_e stored [K, N]: row = expert * K_total + k
          for (int i = 0; i < p.bn_alloc / 64; ++i) ptx::tma_load_3d(b_dst + i * 8192, &tmB, &full[s], n0 + 64 * i, b_row_base + k0, 0);
        } else if (EPI == EPI_SWIGLU) {    // gate rows [0,f) and up rows [f,2f) of expert e
          ptx::tma_load_3d(b_dst, &tmB, &full[s], k0, b_row_base, 0);
          ptx::tma_load_3d(b_dst + p.bn * G_BK * 2, &tmB, &full[s], k0, b_row_base + p.bn, 0);
        } else {
          ptx::tma_load_3d(b_dst, &tmB, &full[s], k0, b_row_base + n0, 0);
        }
      }
    }
  } else if (warp == 1) {
    const uint32_t idesc = ptx::umma_idesc_bf16(G_BM, p.bn, A_MN, B_MN);
    bool ok = true;
    for (int kb = 0; kb < num_kb && ok; ++kb) {
      const int s = kb % p.stages, round = kb / p.stages;
      if (!ptx::mbar_wait(&full[s], round & 1, 1u << 20)) { if (lane == 0) report_error(p.err, ERR_TMA_WAIT); ok = false; break; }
      uint8_t* a_tile = smem + s * STAGE_BYTES;
      if (EPI == EPI_WGRAD) {
        const int valid = rows_valid - kb * G_BK;          // rows of this K block that belong to the expert
        if (valid < G_BK) {
          // MN-major box = 64 K-rows of 128 bytes: rows >= valid hold another expert's data and are cleared
          // both operands: rows past the expert's range may be another expert's rows or never-written buffer space
          const int boxes = G_BM / 64 + p.bn_alloc / 64;         // the B boxes follow the A boxes in the stage
          for (int i = lane; i < (G_BK - valid) * 8 * boxes; i += 32) {
            const int box = i / ((G_BK - valid) * 8), rem = i % ((G_BK - valid) * 8);
            *reinterpret_cast<uint4*>(a_tile + box * 8192 + (valid + rem / 8) * 128 + (rem % 8) * 16) = make_uint4(0, 0, 0, 0);
          }
          ptx::fence_proxy_async();
        }
        __syncwarp();
      }
      ptx::tc_fence_after();
      if (ptx::elect_one()) {
        const uint32_t a_base = ptx::smem_u32(a_tile), b_base = a_base + A_BYTES;
#pragma unroll
        for (int j = 0; j < G_BK / 16; ++j) {
          const uint64_t a_desc = A_MN ? ptx::umma_smem_desc_sw128(a_base + j * 2048, 8192, 1024) : ptx::umma_smem_desc_sw128(a_base + j * 32, 0, 1024);
          const uint64_t b_desc = B_MN ? ptx::umma_smem_desc_sw128(b_base + j * 2048, 8192, 1024) : ptx::umma_smem_desc_sw128(b_base + j * 32, 0, 1024);
          ptx::umma_f16(tmem_base, a_desc, b_desc, idesc, (kb | j) != 0);
          if (EPI == EPI_SWIGLU) {
            const uint64_t u_desc = ptx::umma_smem_desc_sw128(b_base + p.bn * G_BK * 2 + j * 32, 0, 1024);
            ptx::umma_f16(tmem_base + p.bn, a_desc, u_desc, idesc, (kb | j) != 0);
          }
        }
        ptx::umma_commit(&empty[s]);
      }
      __syncwarp();
    }
    if (ptx::elect_one()) ptx::umma_commit(acc_ready);
  } else {
    const int quarter = warp & 3;
    const int r_local = quarter * 32 + lane;
    bool ok = ptx::mbar_wait(acc_ready, 0, 1u << 22);
    if (!ok) report_error(p.err, ERR_EPILOGUE_WAIT);
    ptx::tc_fence_after();
    if (ok) {
      const uint32_t lane_addr = tmem_base + (uint32_t(quarter * 32) << 16);
      if (EPI == EPI_WGRAD) {
        const int row = m0 + r_local;
        float* c_row = reinterpret_cast<float*>(p.out0) + expert * p.c_expert_stride + (long long)row * p.ld0;
        for (int c0 = 0; c0 < p.bn; c0 += 16) {
          uint32_t r[16];
          ptx::tmem_ld_32x32b_x16(lane_addr + c0, r);
          ptx::tmem_ld_wait();
          if (row < p.M) {
            if (n0 + c0 + 16 <= p.N && p.ld0 % 4 == 0) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                float4* dst = reinterpret_cast<float4*>(c_row + n0 + c0 + 4 * v);
                float4 cur = *dst;
                cur.x += __uint_as_float(r[4 * v]); cur.y += __uint_as_float(r[4 * v + 1]);
                cur.z += __uint_as_float(r[4 * v + 2]); cur.w += __uint_as_float(r[4 * v + 3]);
                *dst = cur;
              }
            } else {
#pragma unroll
              for (int e = 0; e < 16; ++e) if (n0 + c0 + e < p.N) c_row[n0 + c0 + e] += __uint_as_float(r[e]);
            }
          }
        }
      } else {
        const bool live = r_local < rows_valid;
        const long long row = a_row0 + r_local;
        for (int c0 = 0; c0 < p.bn; c0 += 16) {
          uint32_t r[16];
          ptx::tmem_ld_32x32b_x16(lane_addr + c0, r);
          if (EPI == EPI_SWIGLU) {
            uint32_t u[16];
            ptx::tmem_ld_32x32b_x16(lane_addr + p.bn + c0, u);
            ptx::tmem_ld_wait();
            if (live) {
              __nv_bfloat16* gu = reinterpret_cast<__nv_bfloat16*>(p.out1) + row * p.ld1;
              __nv_bfloat16* hm = reinterpret_cast<__nv_bfloat16*>(p.out0) + row * p.ld0;
              float gv[16], uv[16], hv[16];
#pragma unroll
              for (int e = 0; e < 16; ++e) {
                gv[e] = bf16_round(__uint_as_float(r[e]));
                uv[e] = bf16_round(__uint_as_float(u[e]));
                hv[e] = bf16_round(siluf_(gv[e])) * uv[e];
              }
              store16_bf16(gu + c0, gv);              // f % 16 == 0: every 16-column group is 32-byte aligned
              store16_bf16(gu + p.bn + c0, uv);
              store16_bf16(hm + c0, hv);
            }
          } else {
            ptx::tmem_ld_wait();
            if (live) {
              if (EPI == EPI_STORE) {
                __nv_bfloat16* o = p.ret_rank ? reinterpret_cast<__nv_bfloat16*>(p.peer_out[p.ret_rank[row]]) + (long long)p.ret_row[row] * p.ld0
                                              : reinterpret_cast<__nv_bfloat16*>(p.out0) + row * p.ld0;
                if (n0 + c0 + 16 <= p.N && p.ld0 % 8 == 0) {
                  float v[16];
#pragma unroll
                  for (int e = 0; e < 16; ++e) v[e] = __uint_as_float(r[e]);
                  store16_bf16(o + n0 + c0, v);
                } else {
#pragma unroll
                  for (int e = 0; e < 16; ++e) if (n0 + c0 + e < p.N) o[n0 + c0 + e] = __float2bfloat16_rn(__uint_as_float(r[e]));
                }
              } else {   // EPI_DSWIGLU: accumulator = d(hmid) for columns n0+c0.. of f = p.N
                const __nv_bfloat16* gu = reinterpret_cast<const __nv_bfloat16*>(p.out1) + row * p.ld1;
                __nv_bfloat16* dgu = reinterpret_cast<__nv_bfloat16*>(p.out0) + row * p.ld0;
                const int c = n0 + c0;
                if (c + 16 <= p.N && p.N % 8 == 0) {
                  // 16 gate and 16 up values as four 16-byte loads
                  uint4 graw[2], uraw[2];
                  graw[0] = reinterpret_cast<const uint4*>(gu + c)[0]; graw[1] = reinterpret_cast<const uint4*>(gu + c)[1];
                  uraw[0] = reinterpret_cast<const uint4*>(gu + p.N + c)[0]; uraw[1] = reinterpret_cast<const uint4*>(gu + p.N + c)[1];
                  const __nv_bfloat16* gp = reinterpret_cast<const __nv_bfloat16*>(graw);
                  const __nv_bfloat16* up = reinterpret_cast<const __nv_bfloat16*>(uraw);
                  float dg[16], du_[16];
#pragma unroll
                  for (int e = 0; e < 16; ++e) {
                    const float dh = bf16_round(__uint_as_float(r[e]));
                    const float g = __bfloat162float(gp[e]), uu = __bfloat162float(up[e]);
                    const float sg = sigmoidf_(g);
                    dg[e] = dh * uu * sg * (1.f + g * (1.f - sg));
                    du_[e] = dh * g * sg;
                  }
                  store16_bf16(dgu + c, dg);
                  store16_bf16(dgu + p.N + c, du_);
                } else {
#pragma unroll
                  for (int e = 0; e < 16; ++e) {
                    const int cc = c + e;
                    if (cc < p.N) {
                      const float dh = bf16_round(__uint_as_float(r[e]));
                      const float g = __bfloat162float(gu[cc]), uu = __bfloat162float(gu[p.N + cc]);
                      const float sg = sigmoidf_(g);
                      dgu[cc] = __float2bfloat16_rn(dh * uu * sg * (1.f + g * (1.f - sg)));
                      dgu[p.N + cc] = __float2bfloat16_rn(dh * g * sg);
                    }
                  }
                }
              }
            }
          }
        }
      }
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) ptx::tmem_dealloc(tmem_base, tmem_cols);
}

// ---- host ----------------------------------------------------------------------------------------------------------------
static int pick_stages(int bn_alloc, int nacc) {
  const int stage = G_BM * G_BK * 2 + nacc * bn_alloc * G_BK * 2;
  if (nacc == 1) {                              // two single-accumulator CTAs share an SM: one runs its epilogue while the other multiplies
    const int s = (110 * 1024) / stage;
    return s > 3 ? 3 : (s < 2 ? 2 : s);
  }
  const int s = (200 * 1024) / stage;
  return s > 4 ? 4 : (s < 2 ? 2 : s);
}

// Width of the N tile of a grouped product: a multiple of 16 up to 192 (two CTAs x 256 TMEM columns per SM) that covers N with the
// least tile time, a tile costing its width plus a fixed part worth about 32 columns.  144 -> 144, 576 -> 192.
static int pick_group_bn(int N) {
  if (N <= 64) return 64;
  int best = 128;
  double best_cost = 1e30;
  for (int bn = 192; bn >= 64; bn -= 16) {
    const int tiles = (N + bn - 1) / bn;
    const double cost = tiles * (bn + 32.0);
    if (cost < best_cost - 1e-9) { best = bn; best_cost = cost; }
  }
  return best;
}

template <int EPI, bool A_MN, bool B_MN>
static void launch_grouped(const CUtensorMap& ta, const CUtensorMap& tb, GroupedArgs p, dim3 grid, int nacc, cudaStream_t stream) {
  auto kernel = grouped_gemm_kernel<EPI, A_MN, B_MN>;
  p.bn_alloc = (B_MN || EPI == EPI_WGRAD) ? (p.bn + 63) / 64 * 64 : p.bn;
  p.stages = pick_stages(p.bn_alloc, nacc);
  const int smem = p.stages * (G_BM * G_BK * 2 + nacc * p.bn_alloc * G_BK * 2) + 1024 + 256;
  static int configured = 0;
  if (configured < smem) { C10_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024)); configured = 227 * 1024; }
  kernel<<<grid, G_THREADS, smem, stream>>>(ta, tb, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

static void check_bf16_2d(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 2 && t.is_contiguous(), name, ": contiguous 2-D bf16 CUDA tensor required");
}

// rows: sorted activations [P, K]; weight: [E, N, K] (K-major) or [E, K, N] (b_mn_major) bf16; out [P, N] bf16
void moe_grouped_gemm_impl(const at::Tensor& rows, const at::Tensor& weight, at::Tensor& out, const at::Tensor& sched, bool b_mn_major, at::Tensor& err,
                           const int* ret_rank, const int* ret_row, const std::vector<int64_t>& peer_out);

void moe_grouped_gemm(const at::Tensor& rows, const at::Tensor& weight, at::Tensor& out, const at::Tensor& sched, bool b_mn_major, at::Tensor& err) {
  if (moe_persistent_enabled()) return moe_grouped_gemm_p(rows, weight, out, sched, b_mn_major, err);      // persistent kernel (moe_persistent.cu)
  moe_grouped_gemm_impl(rows, weight, out, sched, b_mn_major, err, nullptr, nullptr, {});
}

// Same product, but every output row is stored into the buffer of the rank it came from (peer_out[ret_rank[row]] at row
// ret_row[row]); `out` only provides the row width and dtype of those buffers.
void moe_grouped_gemm_return(const at::Tensor& rows, const at::Tensor& weight, at::Tensor& out, const at::Tensor& sched, bool b_mn_major, at::Tensor& err,
                             const at::Tensor& ret_rank, const at::Tensor& ret_row, std::vector<int64_t> peer_out) {
  TORCH_CHECK(ret_rank.scalar_type() == at::kInt && ret_row.scalar_type() == at::kInt && peer_out.size() <= 16, "moe_grouped_gemm_return: bad return map");
  moe_grouped_gemm_impl(rows, weight, out, sched, b_mn_major, err, ret_rank.data_ptr<int>(), ret_row.data_ptr<int>(), peer_out);
}

void moe_grouped_gemm_impl(const at::Tensor& rows, const at::Tensor& weight, at::Tensor& out, const at::Tensor& sched, bool b_mn_major, at::Tensor& err,
                           const int* ret_rank, const int* ret_row, const std::vector<int64_t>& peer_out) {
  check_bf16_2d(rows, "moe_grouped_gemm rows"); check_bf16_2d(out, "moe_grouped_gemm out");
  TORCH_CHECK(weight.dim() == 3 && weight.is_contiguous() && weight.scalar_type() == at::kBFloat16, "moe_grouped_gemm: weight must be contiguous bf16 [E,*,*]");
  const c10::cuda::CUDAGuard guard(rows.device());
  const int P = rows.size(0), K = rows.size(1), E = weight.size(0);
  const int N = b_mn_major ? weight.size(2) : weight.size(1);
  TORCH_CHECK((b_mn_major ? weight.size(1) : weight.size(2)) == K && (ret_rank || out.size(0) == P) && out.size(1) == N, "moe_grouped_gemm: shape mismatch");
  const int bn = pick_group_bn(N);
  const int max_tiles = (sched.numel() - 1) / 3;
  CUtensorMap ta = make_tmap_bf16(rows.data_ptr(), K, P, 1, K, 0, G_BM);
  CUtensorMap tb = b_mn_major ? make_tmap_bf16(weight.data_ptr(), N, (int64_t)E * K, 1, N, 0, 64)
                              : make_tmap_bf16(weight.data_ptr(), K, (int64_t)E * N, 1, K, 0, bn);
  GroupedArgs p{};
  p.sched = sched.data_ptr<int>(); p.bn = bn; p.K = K; p.N = N; p.b_rows_per_expert = b_mn_major ? K : N;
  p.out0 = out.data_ptr(); p.ld0 = N; p.err = err.data_ptr<int>();
  p.ret_rank = ret_rank; p.ret_row = ret_row;
  for (size_t i = 0; i < peer_out.size(); ++i) p.peer_out[i] = reinterpret_cast<void*>(peer_out[i]);
  dim3 grid(max_tiles, (N + bn - 1) / bn, 1);
  auto stream = at::cuda::getCurrentCUDAStream();
  if (b_mn_major) launch_grouped<EPI_STORE, false, true>(ta, tb, p, grid, 1, stream);
  else launch_grouped<EPI_STORE, false, false>(ta, tb, p, grid, 1, stream);
}

// rows [P, h], gate_up weight [E, 2f, h] -> hmid [P, f], gu [P, 2f]
void moe_grouped_swiglu(const at::Tensor& rows, const at::Tensor& weight, at::Tensor& hmid, at::Tensor& gu, const at::Tensor& sched, at::Tensor& err) {
  if (moe_persistent_enabled()) return moe_grouped_swiglu_p(rows, weight, hmid, gu, sched, err);
  check_bf16_2d(rows, "moe_grouped_swiglu rows"); check_bf16_2d(hmid, "hmid"); check_bf16_2d(gu, "gu");
  const c10::cuda::CUDAGuard guard(rows.device());
  const int P = rows.size(0), K = rows.size(1), E = weight.size(0), f = weight.size(1) / 2;
  TORCH_CHECK(weight.size(2) == K && f % 16 == 0 && f <= 256 && hmid.size(1) == f && gu.size(1) == 2 * f, "moe_grouped_swiglu: expert width must be a multiple of 16, at most 256");
  const int max_tiles = (sched.numel() - 1) / 3;
  CUtensorMap ta = make_tmap_bf16(rows.data_ptr(), K, P, 1, K, 0, G_BM);
  CUtensorMap tb = make_tmap_bf16(weight.data_ptr(), K, (int64_t)E * 2 * f, 1, K, 0, f);
  GroupedArgs p{};
  p.sched = sched.data_ptr<int>(); p.bn = f; p.K = K; p.N = f; p.b_rows_per_expert = 2 * f;
  p.out0 = hmid.data_ptr(); p.ld0 = f; p.out1 = gu.data_ptr(); p.ld1 = 2 * f; p.err = err.data_ptr<int>();
  launch_grouped<EPI_SWIGLU, false, false>(ta, tb, p, dim3(max_tiles, 1, 1), 2, at::cuda::getCurrentCUDAStream());
}

// d(hmid) = dy_sorted [P, h] . W_down[e] ([h, f], MN-major B), fused SwiGLU backward -> dgu [P, 2f]
void moe_grouped_dswiglu(const at::Tensor& dy, const at::Tensor& w_down, const at::Tensor& gu, at::Tensor& dgu, const at::Tensor& sched, at::Tensor& err) {
  if (moe_persistent_enabled()) return moe_grouped_dswiglu_p(dy, w_down, gu, dgu, sched, err);
  check_bf16_2d(dy, "dy"); check_bf16_2d(gu, "gu"); check_bf16_2d(dgu, "dgu");
  const c10::cuda::CUDAGuard guard(dy.device());
  const int P = dy.size(0), K = dy.size(1), E = w_down.size(0), f = w_down.size(2);
  TORCH_CHECK(w_down.size(1) == K && gu.size(1) == 2 * f && dgu.size(1) == 2 * f && f % 8 == 0, "moe_grouped_dswiglu: shape mismatch");
  const int bn = pick_group_bn(f);
  const int max_tiles = (sched.numel() - 1) / 3;
  CUtensorMap ta = make_tmap_bf16(dy.data_ptr(), K, P, 1, K, 0, G_BM);
  CUtensorMap tb = make_tmap_bf16(w_down.data_ptr(), f, (int64_t)E * K, 1, f, 0, 64);
  GroupedArgs p{};
  p.sched = sched.data_ptr<int>(); p.bn = bn; p.K = K; p.N = f; p.b_rows_per_expert = K;
  p.out0 = dgu.data_ptr(); p.ld0 = 2 * f; p.out1 = const_cast<void*>(gu.data_ptr()); p.ld1 = 2 * f; p.err = err.data_ptr<int>();
  launch_grouped<EPI_DSWIGLU, false, true>(ta, tb, p, dim3(max_tiles, (f + bn - 1) / bn, 1), 1, at::cuda::getCurrentCUDAStream());
}

// grad[e][m, n] += sum_{rows of expert e} a[row, m] * b[row, n]      a [P, M], b [P, N] bf16, grad [E, M, N] fp32
void moe_grouped_wgrad_p(const at::Tensor& a, const at::Tensor& b, at::Tensor& grad, const at::Tensor& offsets, at::Tensor& err);   // moe_persistent.cu

void moe_grouped_wgrad(const at::Tensor& a, const at::Tensor& b, at::Tensor& grad, const at::Tensor& offsets, at::Tensor& err) {
  if (moe_persistent_enabled()) return moe_grouped_wgrad_p(a, b, grad, offsets, err);
  check_bf16_2d(a, "wgrad a"); check_bf16_2d(b, "wgrad b");
  TORCH_CHECK(grad.is_cuda() && grad.scalar_type() == at::kFloat && grad.dim() == 3 && grad.is_contiguous(), "moe_grouped_wgrad: grad must be contiguous fp32 [E,M,N]");
  const c10::cuda::CUDAGuard guard(a.device());
  const int P = a.size(0), M = a.size(1), N = b.size(1), E = grad.size(0);
  TORCH_CHECK(b.size(0) == P && grad.size(1) == M && grad.size(2) == N && M % 8 == 0 && N % 8 == 0, "moe_grouped_wgrad: shape mismatch");
  const int bn = pick_group_bn(N);
  CUtensorMap ta = make_tmap_bf16(a.data_ptr(), M, P, 1, M, 0, 64);
  CUtensorMap tb = make_tmap_bf16(b.data_ptr(), N, P, 1, N, 0, 64);
  GroupedArgs p{};
  p.offsets = offsets.data_ptr<int>(); p.bn = bn; p.N = N; p.M = M; p.out0 = grad.data_ptr(); p.ld0 = N; p.c_expert_stride = (long long)M * N;
  p.err = err.data_ptr<int>();
  launch_grouped<EPI_WGRAD, true, true>(ta, tb, p, dim3((M + G_BM - 1) / G_BM, (N + bn - 1) / bn, E), 1, at::cuda::getCurrentCUDAStream());
}

// ---- routing / sort host wrappers ------------------------------------------------------------------------------------------
// logits [T, E] bf16 -> {top_w [T,k] fp32 (bf16-rounded), top_idx [T,k] int32, probs [T,E] fp32, counts [E], prob_sum [E]}
std::vector<at::Tensor> moe_route_fwd(const at::Tensor& logits, int64_t k) {
  check_bf16_2d(logits, "moe_route_fwd logits");
  const c10::cuda::CUDAGuard guard(logits.device());
  const int T = logits.size(0), E = logits.size(1);
  TORCH_CHECK(E <= 64 && k <= MAX_TOPK && k <= E, "moe_route_fwd: at most 64 experts and top-8");
  auto f32 = logits.options().dtype(at::kFloat);
  auto top_w = at::empty({T, k}, f32), probs = at::empty({T, E}, f32), counts = at::zeros({E}, f32), psum = at::zeros({E}, f32);
  auto top_idx = at::empty({T, k}, logits.options().dtype(at::kInt));
  if (T) moe_route_fwd_kernel<<<(T + 7) / 8, 256, 0, at::cuda::getCurrentCUDAStream()>>>((const __nv_bfloat16*)logits.data_ptr(), T, E, (int)k, top_w.data_ptr<float>(),
      top_idx.data_ptr<int>(), probs.data_ptr<float>(), counts.data_ptr<float>(), psum.data_ptr<float>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {top_w, top_idx, probs, counts, psum};
}

at::Tensor moe_route_bwd(const at::Tensor& probs, const at::Tensor& top_idx, const at::Tensor& top_w, const at::Tensor& d_top_w,
                         const c10::optional<at::Tensor>& d_prob_sum) {
  const c10::cuda::CUDAGuard guard(probs.device());
  const int T = probs.size(0), E = probs.size(1), k = top_idx.size(1);
  auto dlogits = at::empty({T, E}, probs.options().dtype(at::kBFloat16));
  if (T) moe_route_bwd_kernel<<<(T + 7) / 8, 256, 0, at::cuda::getCurrentCUDAStream()>>>(probs.data_ptr<float>(), top_idx.data_ptr<int>(), top_w.data_ptr<float>(),
      d_top_w.data_ptr<float>(), d_prob_sum.has_value() ? d_prob_sum->data_ptr<float>() : nullptr, T, E, k, (__nv_bfloat16*)dlogits.data_ptr());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return dlogits;
}

// top_idx [T,k] int32 -> {perm [P], inv_perm [P], offsets [E+1], sched [1 + 3 * max_tiles]}
std::vector<at::Tensor> moe_sort(const at::Tensor& top_idx, int64_t E, const c10::optional<at::Tensor>& err) {
  TORCH_CHECK(top_idx.is_cuda() && top_idx.scalar_type() == at::kInt && top_idx.is_contiguous() && E <= 64, "moe_sort: int32 [T,k], at most 64 experts");
  const c10::cuda::CUDAGuard guard(top_idx.device());
  const int P = top_idx.numel();
  const int nblocks = (P + SORT_CHUNK - 1) / SORT_CHUNK;
  const int max_tiles = (P + G_BM - 1) / G_BM + (int)E;
  auto i32 = top_idx.options();
  auto block_counts = at::empty({std::max(nblocks, 1) * (int)E}, i32), perm = at::empty({P}, i32), inv = at::empty({P}, i32);
  auto offsets = at::empty({(int)E + 1}, i32), sched = at::empty({1 + 3 * max_tiles}, i32);
  auto stream = at::cuda::getCurrentCUDAStream();
  if (nblocks) moe_hist_kernel<<<nblocks, SORT_THREADS, 0, stream>>>(top_idx.data_ptr<int>(), P, (int)E, block_counts.data_ptr<int>(),
                                                                     err.has_value() ? err->data_ptr<int>() : nullptr);
  moe_scan_kernel<<<1, 64, 0, stream>>>(block_counts.data_ptr<int>(), nblocks, (int)E, offsets.data_ptr<int>(), sched.data_ptr<int>(), max_tiles, G_BM);
  if (nblocks) moe_scatter_kernel<<<nblocks, SORT_THREADS, 0, stream>>>(top_idx.data_ptr<int>(), P, (int)E, block_counts.data_ptr<int>(), perm.data_ptr<int>(), inv.data_ptr<int>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch(3);
  return {perm, inv, offsets, sched};
}

at::Tensor moe_gather(const at::Tensor& x, const at::Tensor& perm, int64_t k) {
  check_bf16_2d(x, "moe_gather x");
  const c10::cuda::CUDAGuard guard(x.device());
  const int P = perm.numel(), h = x.size(1);
  TORCH_CHECK(h % 8 == 0, "moe_gather: hidden size must be a multiple of 8");
  auto out = at::empty({P, h}, x.options());
  if (P) moe_gather_kernel<<<(P + 7) / 8, 256, 0, at::cuda::getCurrentCUDAStream()>>>((const __nv_bfloat16*)x.data_ptr(), perm.data_ptr<int>(), P, (int)k, h, (__nv_bfloat16*)out.data_ptr());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return out;
}

at::Tensor moe_combine_fwd(const at::Tensor& y_sorted, const at::Tensor& inv_perm, const at::Tensor& top_w) {
  check_bf16_2d(y_sorted, "moe_combine_fwd y");
  const c10::cuda::CUDAGuard guard(y_sorted.device());
  const int T = top_w.size(0), k = top_w.size(1), h = y_sorted.size(1);
  auto out = at::empty({T, h}, y_sorted.options());
  if (T) moe_combine_fwd_kernel<<<(T + 7) / 8, 256, 0, at::cuda::getCurrentCUDAStream()>>>((const __nv_bfloat16*)y_sorted.data_ptr(), inv_perm.data_ptr<int>(),
      top_w.data_ptr<float>(), T, k, h, (__nv_bfloat16*)out.data_ptr());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return out;
}

std::vector<at::Tensor> moe_combine_bwd(const at::Tensor& dout, const at::Tensor& y_sorted, const at::Tensor& inv_perm, const at::Tensor& top_w) {
  check_bf16_2d(dout, "moe_combine_bwd dout");
  const c10::cuda::CUDAGuard guard(dout.device());
  const int T = top_w.size(0), k = top_w.size(1), h = y_sorted.size(1);
  auto dy = at::empty_like(y_sorted);
  auto dw = at::empty({T, k}, top_w.options());
  if (T) moe_combine_bwd_kernel<<<(T * k + 7) / 8, 256, 0, at::cuda::getCurrentCUDAStream()>>>((const __nv_bfloat16*)dout.data_ptr(), (const __nv_bfloat16*)y_sorted.data_ptr(),
      inv_perm.data_ptr<int>(), top_w.data_ptr<float>(), T, k, h, (__nv_bfloat16*)dy.data_ptr(), dw.data_ptr<float>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {dy, dw};
}

at::Tensor moe_unpermute_sum(const at::Tensor& dx_sorted, const at::Tensor& inv_perm, int64_t T, int64_t k) {
  check_bf16_2d(dx_sorted, "moe_unpermute_sum");
  const c10::cuda::CUDAGuard guard(dx_sorted.device());
  const int h = dx_sorted.size(1);
  auto dx = at::empty({T, h}, dx_sorted.options());
  if (T) moe_unpermute_sum_kernel<<<((int)T + 7) / 8, 256, 0, at::cuda::getCurrentCUDAStream()>>>((const __nv_bfloat16*)dx_sorted.data_ptr(), inv_perm.data_ptr<int>(), (int)T, (int)k, h,
      (__nv_bfloat16*)dx.data_ptr());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return dx;
}

}  // namespace q38

// =====================================================================================================================
// Allocation-free entry point (see q38_noalloc.h): same kernels as moe_sort, scratch in a static device array.
// =====================================================================================================================
static __device__ __align__(256) int g_sort_static_scratch[Q38_SORT_STATIC_MAX_BLOCKS * 64];

namespace {
constexpr int kMaxDevices = 64;
int* g_sort_static_ptr[kMaxDevices] = {nullptr};

// The array's name is only a host-side handle; kernels need its device address, which differs per GPU.
int* sort_static_scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (g_sort_static_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_sort_static_scratch) != cudaSuccess) return nullptr;
    g_sort_static_ptr[dev] = static_cast<int*>(ptr);
  }
  return g_sort_static_ptr[dev];
}
}  // namespace

extern "C" int q38_moe_sort_static(const int* expert_of_pair, int P, int experts, int* perm, int* inv_perm, int* offsets, int* sched,
                                   int max_tiles, cudaStream_t stream) {
  using namespace q38;
  if (!expert_of_pair || !perm || !inv_perm || !offsets || !sched || P <= 0 || experts <= 0) return Q38_NOALLOC_BAD_ARGUMENT;
  if (experts > 64 || P > Q38_SORT_STATIC_MAX_PAIRS) return Q38_NOALLOC_TOO_LARGE;
  if (max_tiles < (P + G_BM - 1) / G_BM + experts) return Q38_NOALLOC_BAD_ARGUMENT;
  const int nblocks = (P + SORT_CHUNK - 1) / SORT_CHUNK;
  if (nblocks > Q38_SORT_STATIC_MAX_BLOCKS) return Q38_NOALLOC_TOO_LARGE;
  int* scratch = sort_static_scratch_for_current_device();
  if (scratch == nullptr) return Q38_NOALLOC_CUDA_ERROR;
  // Every word of the scratch that the scan and scatter kernels read is written by the histogram kernel first.
  moe_hist_kernel<<<nblocks, SORT_THREADS, 0, stream>>>(expert_of_pair, P, experts, scratch, nullptr);
  moe_scan_kernel<<<1, 64, 0, stream>>>(scratch, nblocks, experts, offsets, sched, max_tiles, G_BM);
  moe_scatter_kernel<<<nblocks, SORT_THREADS, 0, stream>>>(expert_of_pair, P, experts, scratch, perm, inv_perm);
  if (cudaGetLastError() != cudaSuccess) return Q38_NOALLOC_CUDA_ERROR;
  count_launch(3);
  return Q38_NOALLOC_OK;
}

