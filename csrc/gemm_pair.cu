// Dense bf16 GEMM on pairs of SMs: C[M,N] = alpha * A[M,K] * B[N,K]^T, both operands K-major, with tcgen05.mma.cta_group::2.
//
// A cluster of two CTAs (one SM pair) owns a 256 x bn tile.  Each CTA loads its own 128 rows of A and HALF of the B tile
// (bn/2 rows) - the tensor core of each SM reads the other half from its peer's shared memory - so a K block costs
// 16 KB + bn/2 x 128 B of shared memory per SM instead of 16 KB + bn x 128 B.  That halves the B traffic from L2 per SM and
// makes room for six pipeline stages where the one-CTA kernel (gemm_persistent.cu) has four.  Roles per CTA:
//
//   warp 0     TMA producer (both CTAs): loads its A tile and its half of B; the bytes are counted on the LEADER's `full` barrier
//   warp 1     MMA issuer (leader CTA only): tcgen05.mma.cta_group::2 into one of two 256-column accumulators; each commit is
//              sent to the barrier of both CTAs (two plain commits, one of them to the peer's cluster address)
//   warps 2-9  epilogue (both CTAs, two warpgroups on alternate 32-column chunks): each CTA drains its own 128 accumulator rows
//              from its own TMEM, stages 32 x 32 boxes in swizzled shared memory and hands them to the TMA unit; the accumulator
//              is released on the leader's barrier
//
// Every load is an ordinary tiled TMA load into the issuing CTA's own shared memory.  Every wait is bounded and reports through the error word; both CTAs reach the
// cluster barrier at the end on every path, so neither exits while its peer can still touch its shared memory.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "ptx.cuh"
#include "host.h"

namespace q38 {

constexpr int G2_BM = 128, G2_BK = 64, G2_THREADS = 320, G2_ACC_COLS = 256, G2_MAX_STAGES = 8;

struct PairArgs {
  int M, N, K, batch, bn, stages;
  int tiles_m, tiles_n, total_kb, work_items;
  float alpha;
  int* err;
};

namespace ptx2 {
__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `p` (a location in this CTA's shared memory) as seen in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_rank(const void* p, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(ptx::smem_u32(p)), "r"(rank));
  return out;
}
// Counts this CTA's arrival and its expected bytes on a barrier of the pair.  Relaxed: the arrival orders nothing of this thread's
// own memory traffic (the data arrives through the TMA unit's complete_tx), and a cluster-scope release costs the producer
// several hundred cycles per K block.
__device__ __forceinline__ void arrive_expect_tx_cluster(uint32_t bar_cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.relaxed.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(bar_cluster_addr), "r"(bytes) : "memory");
}
__device__ __forceinline__ void arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
// Tiled load into this CTA's shared memory whose completion bytes are counted on a barrier of either CTA of the pair.
__device__ __forceinline__ void tma_load_3d_pair(void* dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      : : "r"(ptx::smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ptx::smem_u32(slot)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A[smem of both CTAs] * B[smem halves of both CTAs]; issued by ONE thread of the leader CTA.
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      : : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// `bar` (a shared::cluster address, in either CTA) completes once all pair MMAs issued so far by this thread have finished.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}
}  // namespace ptx2

template <typename OutT, bool ACCUM>
__global__ void __launch_bounds__(G2_THREADS) gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                                                               const __grid_constant__ CUtensorMap tmC, PairArgs p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);            // the same offset in both CTAs (same kernel, same layout)
  const int half_n = p.bn / 2;
  const int A_BYTES = G2_BM * 128, B_BYTES = half_n * 128, STAGE_BYTES = A_BYTES + B_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.stages * STAGE_BYTES);
  uint64_t* empty = full + G2_MAX_STAGES;
  uint64_t* acc_full = empty + G2_MAX_STAGES;       // [2]
  uint64_t* acc_empty = acc_full + 2;               // [2], used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  uint8_t* stage_out = smem + p.stages * STAGE_BYTES + 1024;               // [8 warps][2 buffers][4096 bytes]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx2::cluster_rank();                              // 0 = leader
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&tmA);
    ptx::prefetch_tensormap(&tmB);
    ptx::prefetch_tensormap(&tmC);
    for (int s = 0; s < p.stages; ++s) { ptx::mbar_init(&full[s], 2); ptx::mbar_init(&empty[s], 1); }     // full: one arrival (with its bytes) per CTA
    for (int a = 0; a < 2; ++a) { ptx::mbar_init(&acc_full[a], 1); ptx::mbar_init(&acc_empty[a], 16); }   // acc_empty: eight epilogue warps of each CTA
    ptx::fence_barrier_init();
  }
  if (warp == 1) { ptx2::tmem_alloc_pair(tmem_slot, 512); ptx2::tmem_relinquish_pair(); }
  ptx::tc_fence_before();
  __syncthreads();
  ptx2::cluster_sync();                              // the peer's barriers are initialised before anything of ours can reach them
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto decode = [&](int w, int& bz, int& m0, int& n0) {
    const int tn = w % p.tiles_n; w /= p.tiles_n;
    const int tm = w % p.tiles_m; bz = w / p.tiles_m;
    m0 = tm * 2 * G2_BM; n0 = tn * p.bn;
  };

  if (warp == 0) {
    if (ptx::elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int w = cluster_id; w < p.work_items && ok; w += num_clusters) {
        int bz, m0, n0;
        decode(w, bz, m0, n0);
        for (int kb = 0; kb < p.total_kb; ++kb, ++it) {
          const int s = it % p.stages;
          if (!ptx::mbar_wait(&empty[s], ((it / p.stages) & 1) ^ 1, 1u << 20)) { report_error(p.err, ERR_MMA_WAIT); ok = false; break; }
          uint8_t* a_dst = smem + s * STAGE_BYTES;
          uint8_t* b_dst = a_dst + A_BYTES;
          const uint32_t leader_full = ptx2::map_to_rank(&full[s], 0);
          if (rank == 0) ptx::mbar_expect_tx(&full[s], STAGE_BYTES);
          else ptx2::arrive_expect_tx_cluster(leader_full, STAGE_BYTES);
          const int k0 = kb * G2_BK;
          ptx2::tma_load_3d_pair(a_dst, &tmA, leader_full, k0, m0 + (int)rank * G2_BM, bz);
          ptx2::tma_load_3d_pair(b_dst, &tmB, leader_full, k0, n0 + (int)rank * half_n, bz);
        }
      }
    }
  } else if (warp == 1) {
    if (rank == 0 && ptx::elect_one()) {
      const uint32_t idesc = ptx::umma_idesc_bf16(2 * G2_BM, p.bn, false, false);
      uint32_t it = 0, tile = 0;
      bool ok = true;
      for (int w = cluster_id; w < p.work_items && ok; w += num_clusters, ++tile) {
        const int acc = tile & 1;
        if (!ptx::mbar_wait(&acc_empty[acc], ((tile >> 1) & 1) ^ 1, 1u << 22)) { report_error(p.err, ERR_EPILOGUE_WAIT); ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * G2_ACC_COLS;
        for (int kb = 0; kb < p.total_kb; ++kb, ++it) {
          const int s = it % p.stages;
          if (!ptx::mbar_wait(&full[s], (it / p.stages) & 1, 1u << 20)) { report_error(p.err, ERR_TMA_WAIT); ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t a_base = ptx::smem_u32(smem + s * STAGE_BYTES), b_base = a_base + A_BYTES;
#pragma unroll
          for (int j = 0; j < G2_BK / 16; ++j)
            ptx2::umma_f16_pair(d_tmem, ptx::umma_smem_desc_sw128(a_base + j * 32, 0, 1024), ptx::umma_smem_desc_sw128(b_base + j * 32, 0, 1024), idesc,
                                (kb | j) != 0);
          ptx2::umma_commit_pair(ptx2::map_to_rank(&empty[s], 0));          // the stage is free again in both CTAs
          ptx2::umma_commit_pair(ptx2::map_to_rank(&empty[s], 1));
        }
        if (ok) {
          ptx2::umma_commit_pair(ptx2::map_to_rank(&acc_full[acc], 0));     // the accumulator is complete in both CTAs
          ptx2::umma_commit_pair(ptx2::map_to_rank(&acc_full[acc], 1));
        }
      }
    }
  } else {
    // Two warpgroups (warps 2-5 and 6-9) drain alternate 32-column chunks of the accumulator; inside a warp the TMEM read of its
    // next chunk is in flight while the current one is converted, staged and handed to the TMA unit.
    const int quarter = warp & 3, ew = warp - 2, group = ew >> 2;
    uint32_t tile = 0, chunk = 0;
    bool ok = true;
    for (int w = cluster_id; w < p.work_items && ok; w += num_clusters, ++tile) {
      int bz, m0, n0;
      decode(w, bz, m0, n0);
      const int acc = tile & 1;
      if (!ptx::mbar_wait(&acc_full[acc], (tile >> 1) & 1, 1u << 22)) { report_error(p.err, ERR_EPILOGUE_WAIT); ok = false; break; }
      ptx::tc_fence_after();
      const int row0 = m0 + (int)rank * G2_BM + quarter * 32;
      const uint32_t t_addr = tmem_base + acc * G2_ACC_COLS + (uint32_t(quarter * 32) << 16);
      auto emit = [&](const uint32_t (&r)[32], int c0) {
        uint8_t* buf = stage_out + (ew * 2 + (chunk & 1)) * 4096;
        if (lane == 0) ptx::bulk_wait_read<1>();               // the store issued two chunks ago has read this buffer
        __syncwarp();
        if constexpr (sizeof(OutT) == 2) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t wd[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * e]) * p.alpha, __uint_as_float(r[v * 8 + 2 * e + 1]) * p.alpha);
              wd[e] = *reinterpret_cast<uint32_t*>(&h2);
            }
            *reinterpret_cast<uint4*>(buf + lane * 64 + ((v ^ ((lane >> 1) & 3)) << 4)) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
          }
        } else {
#pragma unroll
          for (int v = 0; v < 8; ++v)
            *reinterpret_cast<float4*>(buf + lane * 128 + ((v ^ (lane & 7)) << 4)) =
                make_float4(__uint_as_float(r[v * 4]) * p.alpha, __uint_as_float(r[v * 4 + 1]) * p.alpha, __uint_as_float(r[v * 4 + 2]) * p.alpha,
                            __uint_as_float(r[v * 4 + 3]) * p.alpha);
        }
        ptx::fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          if (n0 + c0 < p.N && row0 < p.M) {
            if constexpr (ACCUM) ptx::tma_reduce_add_3d(&tmC, buf, n0 + c0, row0, bz);
            else ptx::tma_store_3d(&tmC, buf, n0 + c0, row0, bz);
          }
          ptx::bulk_commit();                                  // possibly empty: keeps the buffer accounting uniform
        }
        ++chunk;
      };
      uint32_t ra[32], rb[32];
      int c0 = 32 * group;
      if (c0 < p.bn) ptx::tmem_ld_32x32b_x32(t_addr + c0, ra);
      for (; c0 < p.bn; c0 += 128) {                           // two chunks of this warpgroup per trip: ra, then rb
        ptx::tmem_ld_wait();
        if (c0 + 64 < p.bn) ptx::tmem_ld_32x32b_x32(t_addr + c0 + 64, rb);
        emit(ra, c0);
        if (c0 + 64 < p.bn) {
          ptx::tmem_ld_wait();
          if (c0 + 128 < p.bn) ptx::tmem_ld_32x32b_x32(t_addr + c0 + 128, ra);
          emit(rb, c0 + 64);
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx2::arrive_cluster(ptx2::map_to_rank(&acc_empty[acc], 0));      // released on the leader's barrier
    }
    if (lane == 0) ptx::bulk_wait<0>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx2::cluster_sync();                              // neither CTA leaves while its peer may still signal its barriers or read its tiles
  if (warp == 1) ptx2::tmem_dealloc_pair(tmem_base, 512);
}

static bool g_pair_failed = false;            // a cluster launch was refused once: stay on the one-CTA kernel
bool gemm_pair_enabled() {
  static const bool on = [] { const char* v = std::getenv("Q38_GEMM_PAIR"); return v == nullptr || v[0] != '0'; }();
  return on && !g_pair_failed;
}

// C = alpha * A B^T (+ C) for K-major bf16 A [batch, M, K] and B [batch, N, K]; C bf16 or fp32, storable by TMA.  Returns false when
// the shape is not taken (the caller then runs the one-CTA kernel).
bool gemm_bf16_pair(const at::Tensor& a, const at::Tensor& b, at::Tensor& c, double alpha, bool accumulate, at::Tensor& err) {
  const int batch = a.size(0), M = a.size(1), K = a.size(2), N = b.size(1);
  const bool out_fp32 = c.scalar_type() == at::kFloat;
  const int c_eb = out_fp32 ? 4 : 2;
  if (M < 2 * G2_BM || N < 64 || K % 8 != 0) return false;
  // N tile: a multiple of 32 (store boxes) whose half is a multiple of 8 rows; as in the one-CTA kernel, the most useful columns per tile time
  int bn = 256;
  if (N <= 256) bn = (N + 31) / 32 * 32;
  else {
    double best = 0.0;
    for (int cand = 256; cand >= 128; cand -= 32) {
      const int tiles = (N + cand - 1) / cand;
      const double eff = double(N) / double(tiles * (cand + 32));
      if (eff > best + 1e-9) { bn = cand; best = eff; }
    }
  }
  PairArgs p{};
  p.M = M; p.N = N; p.K = K; p.batch = batch; p.bn = bn;
  p.tiles_m = (M + 2 * G2_BM - 1) / (2 * G2_BM); p.tiles_n = (N + bn - 1) / bn;
  p.total_kb = (K + G2_BK - 1) / G2_BK;
  p.work_items = p.tiles_m * p.tiles_n * batch;
  p.alpha = (float)alpha; p.err = err.data_ptr<int>();
  const int stage_bytes = G2_BM * 128 + bn / 2 * 128, fixed = 1024 + 1024 + 8 * 2 * 4096;
  p.stages = std::min(G2_MAX_STAGES, (227 * 1024 - fixed) / stage_bytes);
  if (p.stages < 3) return false;
  const int smem = p.stages * stage_bytes + fixed;
  CUtensorMap ta = make_tmap_box(a.data_ptr(), 2, K, M, batch, a.stride(1), a.stride(0), G2_BM, 128);
  CUtensorMap tb = make_tmap_box(b.data_ptr(), 2, K, N, batch, b.stride(1), b.stride(0), bn / 2, 128);
  CUtensorMap tc = make_tmap_box(c.data_ptr(), c_eb, N, M, batch, c.stride(1), c.stride(0), 32, 32 * c_eb);
  const int clusters = std::max(1, std::min(p.work_items, kNumSMs / 2));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters); cfg.blockDim = dim3(G2_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = at::cuda::getCurrentCUDAStream();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  // The number of clusters that can be resident at once (pairs must sit in one TPC) bounds the grid: with a static walk over the
  // tiles, clusters beyond it would run as a second wave.
#define Q38_PAIR(OutT, ACC) { auto k = gemm_pair_kernel<OutT, ACC>; static int resident = 0; \
    if (!resident) { C10_CUDA_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024)); \
      cudaLaunchConfig_t probe = cfg; probe.gridDim = dim3(kNumSMs); probe.dynamicSmemBytes = 227 * 1024 - 1024; int n = 0; \
      if (cudaOccupancyMaxActiveClusters(&n, k, &probe) != cudaSuccess || n < 1) { (void)cudaGetLastError(); n = kNumSMs / 2; } \
      resident = n; if (std::getenv("Q38_GEMM_TRACE")) std::fprintf(stderr, "[gemm_pair] resident clusters %d\n", n); } \
    cfg.gridDim = dim3(2 * std::max(1, std::min(p.work_items, resident))); \
    { const cudaError_t st = cudaLaunchKernelEx(&cfg, k, ta, tb, tc, p); \
      if (st != cudaSuccess) { (void)cudaGetLastError(); g_pair_failed = true; \
        std::fprintf(stderr, "[q38] SM-pair GEMM launch refused (%s; grid %u, %d bytes of shared memory): using the one-CTA kernel from here on\n", \
                     cudaGetErrorString(st), cfg.gridDim.x, smem); return false; } } }
  if (out_fp32) { if (accumulate) Q38_PAIR(float, true) else Q38_PAIR(float, false) }
  else { if (accumulate) Q38_PAIR(__nv_bfloat16, true) else Q38_PAIR(__nv_bfloat16, false) }
#undef Q38_PAIR
  count_launch();
  return true;
}

}  // namespace q38
