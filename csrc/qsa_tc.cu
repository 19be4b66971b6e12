// QSA block statistics on the tcgen05 tensor cores.
//
//   stats[b, h, t, j] = (max_s x, sum_s exp(x - max)),  x = scale * q_h(t) . k(s),  s in key block j (64 keys), s <= t
//
// the raw material of the distillation target of the indexer (same contract as qsa_main_block_stats in qsa_index.cu, which
// remains the path for sequence lengths that are not a multiple of 128).
//
// One CTA per (128 query rows = two 64-token query blocks of one head, batch).  The query tile is loaded once; key tiles of 256
// keys stream through a TMA ring; each group is one 128 x 256 x 64 product (four K = 16 instructions) into one of two 256-column
// TMEM accumulators, so the row statistics of group g (four epilogue warps, one query row per thread: tcgen05.ld, running max,
// exp2, sum) overlap the MMAs of group g + 1.  The kernel is bound by the exponentials, not by the products: S^2 / 2 of them per
// head.  Every mbarrier wait is bounded and reports through the error word.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "ptx.cuh"
#include "host.h"

namespace q38 {

constexpr int QT_ROWS = 128, QT_KEYS = 256, QT_STAGES = 2, QT_THREADS = 320;     // TMA warp, MMA warp, two epilogue warpgroups

struct QsaTcArgs {
  float2* stats;
  int S, nq, nkv, nb;
  float scale;
  int* err;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(QT_THREADS) qsa_block_stats_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, QsaTcArgs p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  constexpr int Q_BYTES = QT_ROWS * 128, K_BYTES = QT_KEYS * 128;
  uint8_t* q_tile = smem;
  uint8_t* k_ring = smem + Q_BYTES;
  uint64_t* q_full = reinterpret_cast<uint64_t*>(k_ring + QT_STAGES * K_BYTES);
  uint64_t* k_full = q_full + 1;
  uint64_t* k_empty = k_full + QT_STAGES;
  uint64_t* acc_full = k_empty + QT_STAGES;      // [2]
  uint64_t* acc_empty = acc_full + 2;            // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles = p.S / QT_ROWS;
  const int tile = tiles - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;        // the longest key loops first
  const int row0 = tile * QT_ROWS;
  const int groups = (row0 + QT_ROWS + QT_KEYS - 1) / QT_KEYS;
  const int q_batch = b * p.nq + h, k_batch = b * p.nkv + h / (p.nq / p.nkv);

  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&tmQ);
    ptx::prefetch_tensormap(&tmK);
    ptx::mbar_init(q_full, 1);
    for (int s = 0; s < QT_STAGES; ++s) { ptx::mbar_init(&k_full[s], 1); ptx::mbar_init(&k_empty[s], 1); }
    for (int a = 0; a < 2; ++a) { ptx::mbar_init(&acc_full[a], 1); ptx::mbar_init(&acc_empty[a], 4); }
    ptx::fence_barrier_init();
  }
  if (warp == 1) { ptx::tmem_alloc(tmem_slot, 512); ptx::tmem_relinquish(); }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (ptx::elect_one()) {
      ptx::mbar_expect_tx(q_full, Q_BYTES);
      ptx::tma_load_3d(q_tile, &tmQ, q_full, 0, row0, q_batch);
      for (int g = 0; g < groups; ++g) {
        const int s = g % QT_STAGES, round = g / QT_STAGES;
        if (!ptx::mbar_wait(&k_empty[s], (round & 1) ^ 1, 1u << 20)) { report_error(p.err, ERR_MMA_WAIT); break; }
        ptx::mbar_expect_tx(&k_full[s], K_BYTES);
        ptx::tma_load_3d(k_ring + s * K_BYTES, &tmK, &k_full[s], 0, g * QT_KEYS, k_batch);     // rows past S are zero-filled
      }
    }
  } else if (warp == 1) {
    if (ptx::elect_one()) {
      const uint32_t idesc = ptx::umma_idesc_bf16(QT_ROWS, QT_KEYS, false, false);
      bool ok = ptx::mbar_wait(q_full, 0, 1u << 20);
      if (!ok) report_error(p.err, ERR_TMA_WAIT);
      const uint32_t a_base = ptx::smem_u32(q_tile);
      for (int g = 0; g < groups && ok; ++g) {
        const int s = g % QT_STAGES, acc = g & 1;
        if (!ptx::mbar_wait(&acc_empty[acc], ((g >> 1) & 1) ^ 1, 1u << 22)) { report_error(p.err, ERR_EPILOGUE_WAIT); ok = false; break; }
        if (!ptx::mbar_wait(&k_full[s], (g / QT_STAGES) & 1, 1u << 20)) { report_error(p.err, ERR_TMA_WAIT); ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t b_base = ptx::smem_u32(k_ring + s * K_BYTES), d_tmem = tmem_base + acc * QT_KEYS;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          ptx::umma_f16(d_tmem, ptx::umma_smem_desc_sw128(a_base + j * 32, 0, 1024), ptx::umma_smem_desc_sw128(b_base + j * 32, 0, 1024), idesc, j != 0);
        ptx::umma_commit(&k_empty[s]);
        ptx::umma_commit(&acc_full[acc]);
      }
    }
  } else {
    // Two epilogue warpgroups (warps 2-5 and 6-9): group g is read out by warpgroup g & 1, which owns accumulator g & 1, so two
    // groups' exponentials are in flight per SM.  A warp may read the TMEM lanes 32 (warp % 4) .. + 31.
    const int wg = (warp - 2) >> 2, quarter = warp & 3, r = quarter * 32 + lane;
    const int t = row0 + r, own = t >> 6, tin = t & 63;
    float2* out_row = p.stats + ((long long)q_batch * p.S + t) * p.nb;
    const float c = p.scale * 1.4426950408889634f;            // scores to log2 units
    bool ok = true;
    for (int g = wg; g < groups && ok; g += 2) {
      const int acc = g & 1;
      if (!ptx::mbar_wait(&acc_full[acc], (g >> 1) & 1, 1u << 22)) { report_error(p.err, ERR_EPILOGUE_WAIT); ok = false; break; }
      ptx::tc_fence_after();
      const uint32_t t_addr = tmem_base + acc * QT_KEYS + (uint32_t(quarter * 32) << 16);
      uint32_t nxt_lo[32], nxt_hi[32];
      ptx::tmem_ld_32x32b_x32(t_addr, nxt_lo);
      ptx::tmem_ld_32x32b_x32(t_addr + 32, nxt_hi);
#pragma unroll 1
      for (int jb4 = 0; jb4 < 4; ++jb4) {
        const int jb = g * 4 + jb4;
        float v[64];
        ptx::tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) { v[e] = __uint_as_float(nxt_lo[e]); v[32 + e] = __uint_as_float(nxt_hi[e]); }
        if (jb4 < 3) {                                       // the next block's columns load while this block is reduced
          ptx::tmem_ld_32x32b_x32(t_addr + (jb4 + 1) * 64, nxt_lo);
          ptx::tmem_ld_32x32b_x32(t_addr + (jb4 + 1) * 64 + 32, nxt_hi);
        }
        if (jb > own) continue;                              // a key block after the query's own block: not causal, never read
        float m, sum = 0.f;
        if (jb < own) {                                      // every key of the block is visible
          float m0 = v[0], m1 = v[1], m2 = v[2], m3 = v[3];
#pragma unroll
          for (int e = 4; e < 64; e += 4) { m0 = fmaxf(m0, v[e]); m1 = fmaxf(m1, v[e + 1]); m2 = fmaxf(m2, v[e + 2]); m3 = fmaxf(m3, v[e + 3]); }
          m = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
          const float mc = m * c;
          float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
          for (int e = 0; e < 64; e += 4) {
            s0 += fast_exp2(v[e] * c - mc); s1 += fast_exp2(v[e + 1] * c - mc); s2 += fast_exp2(v[e + 2] * c - mc); s3 += fast_exp2(v[e + 3] * c - mc);
          }
          sum = (s0 + s1) + (s2 + s3);
        } else {                                             // the diagonal block: keys up to the query's own position
          m = -INFINITY;
#pragma unroll
          for (int e = 0; e < 64; ++e) if (e <= tin) m = fmaxf(m, v[e]);
          const float mc = m * c;
#pragma unroll
          for (int e = 0; e < 64; ++e) if (e <= tin) sum += fast_exp2(v[e] * c - mc);
        }
        out_row[jb] = make_float2(m * p.scale, sum);
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&acc_empty[acc]);
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) ptx::tmem_dealloc(tmem_base, 512);
}

// q [B, nq, S, 64], k [B, nkv, S, 64] bf16 contiguous, S a multiple of 128 -> stats [B, nq, S, S / 64] float2 (as a [.., 2] fp32 tensor).
at::Tensor qsa_block_stats_tc(const at::Tensor& q, const at::Tensor& k, double scale, at::Tensor& err) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && q.is_contiguous() && k.is_contiguous() && k.scalar_type() == at::kBFloat16 && q.dim() == 4 &&
              q.size(3) == 64 && k.size(3) == 64, "qsa_block_stats_tc: contiguous bf16 [B, heads, S, 64] tensors required");
  const int B = (int)q.size(0), nq = (int)q.size(1), S = (int)q.size(2), nkv = (int)k.size(1);
  TORCH_CHECK(S % QT_ROWS == 0 && nq % nkv == 0 && k.size(2) == S && k.size(0) == B, "qsa_block_stats_tc: S must be a multiple of 128 and the shapes consistent");
  const c10::cuda::CUDAGuard guard(q.device());
  const int nb = S / 64;
  auto stats = at::empty({B, nq, S, nb, 2}, q.options().dtype(at::kFloat));
  CUtensorMap tq = make_tmap_box(q.data_ptr(), 2, 64, S, (int64_t)B * nq, 64, (int64_t)S * 64, QT_ROWS, 128);
  CUtensorMap tk = make_tmap_box(k.data_ptr(), 2, 64, S, (int64_t)B * nkv, 64, (int64_t)S * 64, QT_KEYS, 128);
  QsaTcArgs p{};
  p.stats = reinterpret_cast<float2*>(stats.data_ptr<float>()); p.S = S; p.nq = nq; p.nkv = nkv; p.nb = nb; p.scale = (float)scale; p.err = err.data_ptr<int>();
  const int smem = QT_ROWS * 128 + QT_STAGES * QT_KEYS * 128 + 1024 + 256;
  static bool configured = false;
  if (!configured) { C10_CUDA_CHECK(cudaFuncSetAttribute(qsa_block_stats_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); configured = true; }
  qsa_block_stats_tc_kernel<<<dim3(S / QT_ROWS, nq, B), QT_THREADS, smem, at::cuda::getCurrentCUDAStream()>>>(tq, tk, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return stats;
}

}  // namespace q38
