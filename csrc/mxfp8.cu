// Block-scaled MXFP8 path of the routed experts: quantisation kernels and a grouped tcgen05 GEMM of kind mxf8f6f4.block_scale.
//
// Format (OCP MX): elements are E4M3, every 32 consecutive elements along the reduction dimension K share one E8M0 scale
// (a power of two, stored as the biased exponent).  A product is  D[m,n] = sum_k  sA[m,k/32] a[m,k] * sB[n,k/32] b[n,k].
//
// Scale-factor storage.  The tensor core reads scales from tensor memory in a fixed arrangement; the global arrays use the
// matching one so that a 512-byte block can be copied to shared memory as is and from there into tensor memory with one
// `tcgen05.cp ... 32x128b.warpx4`.  A block covers 128 rows and 4 K-blocks (128 elements of K):
//     byte offset inside the block = (row % 32) * 16 + (row / 32) * 4 + kblock % 4
// Blocks are stored tile-major: [tile][128-row block inside the tile][K chunk][512].  For the activations a tile is one entry
// of the expert tile schedule (at most 128 sorted rows of one expert, starting at an arbitrary sorted row); for the weights a
// tile is one N tile of one expert.  Rows of a tile that do not exist get the scale 2^0.
//
// Kernels
//   mxfp8_quantize_rows     bf16 rows (optionally gathered through the expert sort permutation) -> e4m3 rows [P, K] in sorted
//                           order + tile-major scales, driven by the tile schedule
//   mxfp8_quantize_weight   bf16/fp32 [E, N, K] (any strides, so a transposed view quantises along the other axis) -> e4m3
//                           [E, N, K] contiguous + tile-major scales for N tiles of `bn` rows
//   mxfp8_grouped_gemm      out[sorted row, n] = sum_k A[row, k] W[expert(row), n, k]  (bf16 out), one CTA per (tile, N tile):
//                           TMA -> shared memory (128-byte swizzle) -> tcgen05.mma.kind::mxf8f6f4.block_scale -> TMEM -> bf16 rows
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "ptx.cuh"
#include "host.h"

namespace q38 {

constexpr int MX_BLOCK = 32;          // elements per scale
constexpr int MX_CHUNK = 128;         // elements of K per scale-factor block (4 scales per row)
constexpr int MX_SF_BYTES = 512;      // one 128-row x 4-scale block

// Shared exponent e of a 32-element block with absolute maximum `amax`: the smallest power of two with amax / 2^e <= 448
// (the largest finite E4M3 value), so nothing saturates.  Returned as the biased E8M0 byte; *inv receives 2^-e.
__device__ __forceinline__ uint32_t mx_scale_byte(float amax, float* inv) {
  if (!(amax > 0.f)) { *inv = 1.f; return 127u; }
  const float t = amax * (1.f / 448.f);
  const uint32_t bits = __float_as_uint(t);
  int e = int((bits >> 23) & 0xFF) - 127;
  if (bits & 0x7FFFFFu) e += 1;                          // ceil(log2(t))
  e = max(-127, min(127, e));
  *inv = __uint_as_float(uint32_t(127 - e) << 23);       // 2^-e (e = 127 gives a denormal-free 2^-127? no: clamp below)
  if (e >= 127) *inv = __uint_as_float(1u << 22);        // 2^-127 as a subnormal
  return uint32_t(e + 127);
}

// four floats -> four E4M3 bytes (round to nearest even, saturating)
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(lo) : "f"(a), "f"(b));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(hi) : "f"(c), "f"(d));
  return uint32_t(lo) | (uint32_t(hi) << 16);
}

__device__ __forceinline__ long long mx_sf_offset(long long block_index, int row_in_block, int kblock) {
  return block_index * MX_SF_BYTES + (row_in_block & 31) * 16 + (row_in_block >> 5) * 4 + (kblock & 3);
}

// Quantise one 32-element block held as floats; `count` (<= 32) elements are real, the rest are treated as zero.
__device__ __forceinline__ void mx_quantize_block(const float (&v)[32], int count, uint8_t* __restrict__ q_dst, uint8_t* __restrict__ sf_dst) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) if (i < count) amax = fmaxf(amax, fabsf(v[i]));
  float inv;
  const uint32_t byte = mx_scale_byte(amax, &inv);
  *sf_dst = uint8_t(byte);
  if (count == 32) {
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = pack_e4m3x4(v[4 * i] * inv, v[4 * i + 1] * inv, v[4 * i + 2] * inv, v[4 * i + 3] * inv);
    reinterpret_cast<uint4*>(q_dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<uint4*>(q_dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
  } else {
    for (int i = 0; i < count; i += 4) {
      const uint32_t w = pack_e4m3x4(v[i] * inv, i + 1 < count ? v[i + 1] * inv : 0.f, i + 2 < count ? v[i + 2] * inv : 0.f, i + 3 < count ? v[i + 3] * inv : 0.f);
      for (int j = 0; j < 4 && i + j < count; ++j) q_dst[i + j] = uint8_t(w >> (8 * j));
    }
  }
}

// ---- activations: one CTA per schedule tile, one warp per row, one lane per 32-element block -------------------------------------
// src bf16 [*, K] row stride ld.  perm != nullptr: sorted row p reads source row perm[p] / topk (gather), else source row p.
// q [P, K] e4m3 (sorted rows), sf tile-major [max_tiles][chunks][512].
__global__ void __launch_bounds__(256) mxfp8_quantize_rows_kernel(const __nv_bfloat16* __restrict__ src, long long ld, const int* __restrict__ perm, int topk,
                                                                  const int* __restrict__ sched, int K, uint8_t* __restrict__ q, uint8_t* __restrict__ sf) {
  const int tile = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ntiles = sched[0];
  const int row0 = tile < ntiles ? sched[2 + 3 * tile] : 0, rows = tile < ntiles ? sched[3 + 3 * tile] : 0;
  const int nblocks = (K + MX_BLOCK - 1) / MX_BLOCK, chunks = (K + MX_CHUNK - 1) / MX_CHUNK;
  for (int r = warp; r < 128; r += 8) {
    for (int kb = lane; kb < chunks * 4; kb += 32) {
      uint8_t* sf_dst = sf + mx_sf_offset((long long)tile * chunks + kb / 4, r, kb);
      if (r >= rows || kb >= nblocks) { *sf_dst = 127; continue; }
      const long long p = row0 + r;
      const long long s_row = perm ? perm[p] / topk : p;
      const __nv_bfloat16* s = src + s_row * ld + kb * MX_BLOCK;
      const int count = min(MX_BLOCK, K - kb * MX_BLOCK);
      float v[32];
      if (count == 32 && (ld % 8 == 0)) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 raw = reinterpret_cast<const uint4*>(s)[i];
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
          for (int j = 0; j < 4; ++j) { v[8 * i + 2 * j] = __low2float(h[j]); v[8 * i + 2 * j + 1] = __high2float(h[j]); }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = i < count ? __bfloat162float(s[i]) : 0.f;
      }
      mx_quantize_block(v, count, q + p * K + kb * MX_BLOCK, sf_dst);
    }
  }
}

// ---- weights: W[e, n, k] read through strides (elements), T = float or bf16 ---------------------------------------------------
// q [E, N, K] contiguous e4m3; sf tile-major: tile = e * tiles_n + n / bn, 128-row blocks inside the tile.
template <typename T>
__global__ void __launch_bounds__(256) mxfp8_quantize_weight_kernel(const T* __restrict__ w, long long se, long long sn, long long sk, int N, int K, int bn,
                                                                    uint8_t* __restrict__ q, uint8_t* __restrict__ sf) {
  const int tiles_n = (N + bn - 1) / bn, blocks_per_tile = (bn + 127) / 128;
  const int tile = blockIdx.x, e = tile / tiles_n, n0 = (tile % tiles_n) * bn;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblocks = (K + MX_BLOCK - 1) / MX_BLOCK, chunks = (K + MX_CHUNK - 1) / MX_CHUNK;
  for (int r = warp; r < blocks_per_tile * 128; r += 8) {
    const int n = n0 + r;
    const bool live = r < bn && n < N;
    for (int kb = lane; kb < chunks * 4; kb += 32) {
      uint8_t* sf_dst = sf + mx_sf_offset(((long long)tile * blocks_per_tile + r / 128) * chunks + kb / 4, r % 128, kb);
      if (!live || kb >= nblocks) { *sf_dst = 127; continue; }
      const int count = min(MX_BLOCK, K - kb * MX_BLOCK);
      const T* s = w + e * se + n * sn + (long long)kb * MX_BLOCK * sk;
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = i < count ? to_float<T>(s[i * sk]) : 0.f;
      mx_quantize_block(v, count, q + ((long long)e * N + n) * K + kb * MX_BLOCK, sf_dst);
    }
  }
}


// =====================================================================================================================
// Grouped block-scaled GEMM
// =====================================================================================================================
namespace mx {

// Shared-memory descriptor without swizzle: 8-row x 16-byte core matrices, `sbo` bytes between core matrices along rows.
__device__ __forceinline__ uint64_t smem_desc_plain(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return uint64_t((smem_addr & 0x3FFFFu) >> 4) | (uint64_t(lbo_bytes >> 4) << 16) | (uint64_t(sbo_bytes >> 4) << 32) | (uint64_t(1) << 46);
}
// 32 rows x 16 bytes of shared memory -> 4 TMEM columns, replicated into the four 32-lane quarters (the scale-factor copy).
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t src_desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(src_desc) : "memory");
}
// Instruction descriptor of kind::mxf8f6f4.block_scale: E4M3 x E4M3, E8M0 scales, K-major operands.
// [4,6) B scale id, [7,10) A format (0 = E4M3), [10,13) B format, [17,23) N >> 3, 23 scale format (1 = E8M0), [24,29) M >> 4, [29,31) A scale id.
__device__ __forceinline__ uint32_t idesc(int M, int N, uint32_t a_sf_id, uint32_t b_sf_id) {
  return (b_sf_id << 4) | (uint32_t(N >> 3) << 17) | (1u << 23) | (uint32_t(M >> 4) << 24) | (a_sf_id << 29);
}
__device__ __forceinline__ void umma_mxf8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc_, uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n"
      : : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc_), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}
// Plain (non-tensor) bulk copy global -> shared memory, completion on an mbarrier; 16-byte aligned addresses and size.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               : : "r"(ptx::smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(ptx::smem_u32(bar)) : "memory");
}

}  // namespace mx

constexpr int MX_BM = 128, MX_STAGES = 4, MX_THREADS = 192;

struct MxArgs {
  const int* sched;
  const uint8_t* sfa;        // [max_tiles][chunks][512]
  const uint8_t* sfb;        // [E * tiles_n][chunks][512]   (bn <= 128: one 128-row block per N tile)
  int bn, K, N, chunks, tiles_n, b_rows_per_expert;
  __nv_bfloat16* out; long long ldo;
  int* err;
};

// One CTA per (schedule tile, N tile).  Stage = {A 128 x 128 B, B bn x 128 B (both 128-byte swizzled), SFA 512 B, SFB 512 B}.
// TMEM: accumulator in columns [0, bn), scale factors of stage s in columns 128 + 8 s (A) and 132 + 8 s (B).
__global__ void __launch_bounds__(MX_THREADS) mxfp8_grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, MxArgs p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  const int A_BYTES = MX_BM * 128, B_BYTES = ((p.bn * 128 + 1023) / 1024) * 1024, STAGE_BYTES = A_BYTES + B_BYTES + 2 * MX_SF_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + MX_STAGES * STAGE_BYTES);
  uint64_t* empty = full + MX_STAGES;
  uint64_t* acc_ready = empty + MX_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, ntile = blockIdx.y;
  if (tile >= p.sched[0]) return;
  const int expert = p.sched[1 + 3 * tile], a_row0 = p.sched[2 + 3 * tile], rows_valid = p.sched[3 + 3 * tile];
  if (rows_valid <= 0) return;
  const int n0 = ntile * p.bn, num_kb = p.chunks;

  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&tmA);
    ptx::prefetch_tensormap(&tmB);
    for (int s = 0; s < MX_STAGES; ++s) { ptx::mbar_init(&full[s], 1); ptx::mbar_init(&empty[s], 1); }
    ptx::mbar_init(acc_ready, 1);
    ptx::fence_barrier_init();
  }
  if (warp == 1) { ptx::tmem_alloc(tmem_slot, 256); ptx::tmem_relinquish(); }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (ptx::elect_one()) {
      const uint8_t* sfa_src = p.sfa + (long long)tile * p.chunks * MX_SF_BYTES;
      const uint8_t* sfb_src = p.sfb + ((long long)expert * p.tiles_n + ntile) * p.chunks * MX_SF_BYTES;
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % MX_STAGES, round = kb / MX_STAGES;
        if (!ptx::mbar_wait(&empty[s], (round & 1) ^ 1, 1u << 20)) { report_error(p.err, ERR_MMA_WAIT); break; }
        uint8_t* a_dst = smem + s * STAGE_BYTES;
        uint8_t* b_dst = a_dst + A_BYTES;
        uint8_t* sf_dst = b_dst + B_BYTES;
        ptx::mbar_expect_tx(&full[s], A_BYTES + p.bn * 128 + 2 * MX_SF_BYTES);
        ptx::tma_load_3d(a_dst, &tmA, &full[s], kb * MX_CHUNK, a_row0, 0);
        ptx::tma_load_3d(b_dst, &tmB, &full[s], kb * MX_CHUNK, expert * p.b_rows_per_expert + n0, 0);
        mx::bulk_load(sf_dst, sfa_src + (long long)kb * MX_SF_BYTES, MX_SF_BYTES, &full[s]);
        mx::bulk_load(sf_dst + MX_SF_BYTES, sfb_src + (long long)kb * MX_SF_BYTES, MX_SF_BYTES, &full[s]);
      }
    }
  } else if (warp == 1) {
    if (ptx::elect_one()) {
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % MX_STAGES, round = kb / MX_STAGES;
        if (!ptx::mbar_wait(&full[s], round & 1, 1u << 20)) { report_error(p.err, ERR_TMA_WAIT); ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t a_base = ptx::smem_u32(smem + s * STAGE_BYTES), b_base = a_base + A_BYTES, sf_base = b_base + B_BYTES;
        const uint32_t sfa_t = tmem_base + 128 + 8 * s, sfb_t = sfa_t + 4;
        mx::tmem_cp_sf(sfa_t, mx::smem_desc_plain(sf_base, 128, 128));
        mx::tmem_cp_sf(sfb_t, mx::smem_desc_plain(sf_base + MX_SF_BYTES, 128, 128));
#pragma unroll
        for (int j = 0; j < 4; ++j) {                                  // four K = 32 steps per 128-byte row
          const uint64_t a_desc = ptx::umma_smem_desc_sw128(a_base + j * 32, 0, 1024);
          const uint64_t b_desc = ptx::umma_smem_desc_sw128(b_base + j * 32, 0, 1024);
          mx::umma_mxf8(tmem_base, a_desc, b_desc, mx::idesc(MX_BM, p.bn, j, j), sfa_t, sfb_t, (kb | j) != 0);
        }
        ptx::umma_commit(&empty[s]);
      }
      if (ok) ptx::umma_commit(acc_ready);
    }
  } else {
    const int quarter = warp & 3, r_local = quarter * 32 + lane;
    const bool ok = ptx::mbar_wait(acc_ready, 0, 1u << 22);
    if (!ok) report_error(p.err, ERR_EPILOGUE_WAIT);
    ptx::tc_fence_after();
    if (ok) {
      const uint32_t lane_addr = tmem_base + (uint32_t(quarter * 32) << 16);
      const bool live = r_local < rows_valid;
      __nv_bfloat16* o_row = p.out + (long long)(a_row0 + r_local) * p.ldo;
      for (int c0 = 0; c0 < p.bn; c0 += 16) {
        uint32_t r[16];
        ptx::tmem_ld_32x32b_x16(lane_addr + c0, r);
        ptx::tmem_ld_wait();
        if (!live) continue;
        const int col = n0 + c0;
        if (col + 16 <= p.N && (p.ldo % 8 == 0)) {
          uint32_t w[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[2 * e]), __uint_as_float(r[2 * e + 1]));
            w[e] = *reinterpret_cast<uint32_t*>(&h);
          }
          reinterpret_cast<uint4*>(o_row + col)[0] = make_uint4(w[0], w[1], w[2], w[3]);
          reinterpret_cast<uint4*>(o_row + col)[1] = make_uint4(w[4], w[5], w[6], w[7]);
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) if (col + e < p.N) o_row[col + e] = __float2bfloat16_rn(__uint_as_float(r[e]));
        }
      }
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) ptx::tmem_dealloc(tmem_base, 256);
}


// ---- host ----------------------------------------------------------------------------------------------------------------------
// N tile of the block-scaled kernel: a multiple of 16, at most 128 (one 128-row scale block per tile).
int64_t mxfp8_pick_bn(int64_t N) {
  int best = 128;
  double best_cost = 1e30;
  for (int bn = 128; bn >= 64; bn -= 16) {
    const int tiles = (int)((N + bn - 1) / bn);
    const double cost = tiles * (bn + 32.0);
    if (cost < best_cost - 1e-9) { best = bn; best_cost = cost; }
  }
  return best;
}

// src bf16 [R, K]; perm (optional) + topk: gather through the expert sort; sched from moe_sort.  Returns {q uint8 [P, K], sf uint8}.
std::vector<at::Tensor> mxfp8_quantize_rows(const at::Tensor& src, const c10::optional<at::Tensor>& perm, int64_t topk, const at::Tensor& sched, int64_t P) {
  TORCH_CHECK(src.is_cuda() && src.scalar_type() == at::kBFloat16 && src.dim() == 2 && src.stride(1) == 1, "mxfp8_quantize_rows: bf16 [R, K] rows required");
  const int K = (int)src.size(1);
  TORCH_CHECK(K % 16 == 0, "mxfp8_quantize_rows: K must be a multiple of 16");
  const c10::cuda::CUDAGuard guard(src.device());
  const int max_tiles = (int)((sched.numel() - 1) / 3), chunks = (K + MX_CHUNK - 1) / MX_CHUNK;
  auto u8 = src.options().dtype(at::kByte);
  auto q = at::empty({P, K}, u8), sf = at::empty({(int64_t)max_tiles * chunks * MX_SF_BYTES}, u8);
  if (max_tiles)
    mxfp8_quantize_rows_kernel<<<max_tiles, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
        (const __nv_bfloat16*)src.data_ptr(), (long long)src.stride(0), perm.has_value() ? perm->data_ptr<int>() : nullptr, (int)topk, sched.data_ptr<int>(), K,
        q.data_ptr<uint8_t>(), sf.data_ptr<uint8_t>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {q, sf};
}

// w [E, N, K] (fp32 or bf16, any strides) -> {q uint8 [E, N, K], sf uint8 [E * tiles_n * chunks * 512]} for N tiles of `bn` rows.
std::vector<at::Tensor> mxfp8_quantize_weight(const at::Tensor& w, int64_t bn) {
  TORCH_CHECK(w.is_cuda() && w.dim() == 3 && (w.scalar_type() == at::kFloat || w.scalar_type() == at::kBFloat16), "mxfp8_quantize_weight: fp32 / bf16 [E, N, K] required");
  TORCH_CHECK(bn >= 16 && bn <= 128 && bn % 16 == 0, "mxfp8_quantize_weight: N tile must be a multiple of 16 up to 128");
  const c10::cuda::CUDAGuard guard(w.device());
  const int E = (int)w.size(0), N = (int)w.size(1), K = (int)w.size(2);
  TORCH_CHECK(K % 16 == 0, "mxfp8_quantize_weight: K must be a multiple of 16");
  const int tiles_n = (N + (int)bn - 1) / (int)bn, chunks = (K + MX_CHUNK - 1) / MX_CHUNK;
  auto u8 = w.options().dtype(at::kByte);
  auto q = at::empty({E, N, K}, u8), sf = at::empty({(int64_t)E * tiles_n * chunks * MX_SF_BYTES}, u8);
  auto stream = at::cuda::getCurrentCUDAStream();
  if (w.scalar_type() == at::kFloat)
    mxfp8_quantize_weight_kernel<float><<<E * tiles_n, 256, 0, stream>>>(w.data_ptr<float>(), w.stride(0), w.stride(1), w.stride(2), N, K, (int)bn, q.data_ptr<uint8_t>(),
                                                                           sf.data_ptr<uint8_t>());
  else
    mxfp8_quantize_weight_kernel<__nv_bfloat16><<<E * tiles_n, 256, 0, stream>>>((const __nv_bfloat16*)w.data_ptr(), w.stride(0), w.stride(1), w.stride(2), N, K, (int)bn,
                                                                                   q.data_ptr<uint8_t>(), sf.data_ptr<uint8_t>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {q, sf};
}

// out[row, :] = A[row, :] . W[expert(row)]^T for the sorted rows of the schedule.  aq [P, K], wq [E, N, K] uint8 (e4m3); bf16 out [P, N].
void mxfp8_grouped_gemm(const at::Tensor& aq, const at::Tensor& sfa, const at::Tensor& wq, const at::Tensor& sfw, at::Tensor& out, const at::Tensor& sched, int64_t bn,
                        at::Tensor& err) {
  TORCH_CHECK(aq.is_cuda() && aq.scalar_type() == at::kByte && aq.dim() == 2 && aq.is_contiguous() && wq.scalar_type() == at::kByte && wq.dim() == 3 && wq.is_contiguous(),
              "mxfp8_grouped_gemm: contiguous e4m3 (uint8) operands required");
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.dim() == 2 && out.stride(1) == 1, "mxfp8_grouped_gemm: bf16 output rows required");
  const c10::cuda::CUDAGuard guard(aq.device());
  const int P = (int)aq.size(0), K = (int)aq.size(1), E = (int)wq.size(0), N = (int)wq.size(1);
  TORCH_CHECK(wq.size(2) == K && out.size(0) == P && out.size(1) == N && K % 16 == 0, "mxfp8_grouped_gemm: shape mismatch");
  TORCH_CHECK(bn >= 16 && bn <= 128 && bn % 16 == 0, "mxfp8_grouped_gemm: N tile must be a multiple of 16 up to 128");
  const int max_tiles = (int)((sched.numel() - 1) / 3), chunks = (K + MX_CHUNK - 1) / MX_CHUNK, tiles_n = (N + (int)bn - 1) / (int)bn;
  TORCH_CHECK(sfa.numel() == (int64_t)max_tiles * chunks * MX_SF_BYTES && sfw.numel() == (int64_t)E * tiles_n * chunks * MX_SF_BYTES,
              "mxfp8_grouped_gemm: scale arrays do not match the schedule / the N tile the weights were quantised for");
  if (!max_tiles || !P) return;
  CUtensorMap ta = make_tmap_box(aq.data_ptr(), 1, K, P, 1, K, 0, MX_BM, 128);
  CUtensorMap tb = make_tmap_box(wq.data_ptr(), 1, K, (int64_t)E * N, 1, K, 0, (int)bn, 128);
  MxArgs p{};
  p.sched = sched.data_ptr<int>(); p.sfa = sfa.data_ptr<uint8_t>(); p.sfb = sfw.data_ptr<uint8_t>();
  p.bn = (int)bn; p.K = K; p.N = N; p.chunks = chunks; p.tiles_n = tiles_n; p.b_rows_per_expert = N;
  p.out = (__nv_bfloat16*)out.data_ptr(); p.ldo = out.stride(0); p.err = err.data_ptr<int>();
  const int b_bytes = (((int)bn * 128 + 1023) / 1024) * 1024;
  const int smem = MX_STAGES * (MX_BM * 128 + b_bytes + 2 * MX_SF_BYTES) + 1024 + 256;
  static bool configured = false;
  if (!configured) { C10_CUDA_CHECK(cudaFuncSetAttribute(mxfp8_grouped_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); configured = true; }
  mxfp8_grouped_gemm_kernel<<<dim3(max_tiles, tiles_n), MX_THREADS, smem, at::cuda::getCurrentCUDAStream()>>>(ta, tb, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

}  // namespace q38
