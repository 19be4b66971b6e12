// Persistent grouped expert GEMM: one CTA per SM walks the (schedule tile, N tile) work items of a grouped product, with the
// same three decoupled roles as the dense persistent GEMM (gemm_persistent.cu):
//
//   warp 0     TMA producer: a ring of {A 128 x 64, B bn x 64 (two of them for the gate/up pair)} bf16 stages filled across tiles
//   warp 1     MMA issuer: tcgen05.mma into one of two TMEM accumulator sets (256 columns each)
//   warps 2-9  epilogue (two warpgroups on alternate 16-column chunks): tcgen05.ld of the finished set, SwiGLU / SwiGLU-backward /
//              plain store, masked to the expert's rows
//
// so the read-out of tile i overlaps the loads and MMAs of tile i + 1, and the per-tile set-up (barrier init, TMEM allocation,
// descriptor prefetch) is paid once per SM instead of once per tile.  The expert products have K = 576 or 144: a tile's MMAs take
// far less time than its epilogue, which is why the one-tile-per-CTA kernel in moe.cu sits at 28-41 % of the memory roofline.
//
// Epilogues (same arithmetic and rounding points as moe.cu):
//   PE_STORE    C[row, n] = A[row, :] . B_e[n, :]                                   (down projection, input gradients)
//   PE_SWIGLU   gate and up accumulators -> gu[row, 2f] and hmid[row, f] = silu(g) * u
//   PE_DSWIGLU  accumulator = d(hmid); reads gu, writes d(gu)[row, 2f]
//   PE_WGRAD    C_e[m, n] += sum over the expert's rows of A[row, m] B[row, n]: both operands MN-major, K = the expert's rows
//               (the ragged last K block is cleared in shared memory), fp32 read-modify-write of C fetched one chunk ahead
// The expert-parallel return epilogue stays in moe.cu.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "ptx.cuh"
#include "host.h"

namespace q38 {

enum { PE_STORE = 0, PE_SWIGLU = 1, PE_DSWIGLU = 2, PE_WGRAD = 3 };
constexpr int PG_BM = 128, PG_BK = 64, PG_STAGES = 4, PG_THREADS = 320, PG_ACC_COLS = 256;

struct PGroupedArgs {
  const int* sched;        // [0] = tiles; then (expert, first row, rows) per tile
  int bn, bn_alloc, tiles_n, K, N, b_rows_per_expert;
  void* out0; long long ld0;
  void* out1; long long ld1;
  int* err;
  // PE_WGRAD: expert row offsets [E + 1], experts, M tiles and rows of C per expert, elements between experts in C
  const int* offsets; int experts, tiles_m, M; long long c_expert_stride;
};

struct PGWork { int expert, row0, rows, n0, m0, k_begin, num_kb; };

__device__ __forceinline__ void pg_store16(__nv_bfloat16* dst, const float (&v)[16]) {
  uint32_t w[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
    w[e] = *reinterpret_cast<uint32_t*>(&h);
  }
  reinterpret_cast<uint4*>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
  reinterpret_cast<uint4*>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
}

template <int EPI, bool B_MN, bool A_MN = false>
__global__ void __launch_bounds__(PG_THREADS) grouped_persistent_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                                                                        PGroupedArgs p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  constexpr int NACC = EPI == PE_SWIGLU ? 2 : 1;
  const int A_BYTES = PG_BM * PG_BK * 2, B_BYTES = NACC * p.bn_alloc * PG_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + PG_STAGES * STAGE_BYTES);
  uint64_t* empty = full + PG_STAGES;
  uint64_t* acc_full = empty + PG_STAGES;       // [2]
  uint64_t* acc_empty = acc_full + 2;           // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int work_items = EPI == PE_WGRAD ? p.experts * p.tiles_m * p.tiles_n : p.sched[0] * p.tiles_n;

  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&tmA);
    ptx::prefetch_tensormap(&tmB);
    for (int s = 0; s < PG_STAGES; ++s) { ptx::mbar_init(&full[s], 1); ptx::mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { ptx::mbar_init(&acc_full[a], 1); ptx::mbar_init(&acc_empty[a], 8); }
    ptx::fence_barrier_init();
  }
  if (warp == 1) { ptx::tmem_alloc(tmem_slot, 512); ptx::tmem_relinquish(); }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // work item -> tile.  Grouped products: (schedule tile, N tile), the N tiles of one row tile consecutive (A reuse from L2).
  // Weight gradients: (expert, M tile, N tile), the tiles of one expert consecutive; an expert without rows has num_kb = 0 and is
  // skipped by all three roles alike.
  auto decode = [&](int w) {
    PGWork k;
    if (EPI == PE_WGRAD) {
      const int per_expert = p.tiles_m * p.tiles_n, in_expert = w % per_expert;
      k.expert = w / per_expert;
      k.m0 = (in_expert / p.tiles_n) * PG_BM; k.n0 = (in_expert % p.tiles_n) * p.bn;
      k.k_begin = p.offsets[k.expert];
      k.rows = p.offsets[k.expert + 1] - k.k_begin;
      k.row0 = 0;
      k.num_kb = k.rows > 0 ? (k.rows + PG_BK - 1) / PG_BK : 0;
    } else {
      const int tile = w / p.tiles_n;
      k.n0 = (w % p.tiles_n) * p.bn; k.m0 = 0; k.k_begin = 0;
      k.expert = p.sched[1 + 3 * tile]; k.row0 = p.sched[2 + 3 * tile]; k.rows = p.sched[3 + 3 * tile];
      k.num_kb = (p.K + PG_BK - 1) / PG_BK;
    }
    return k;
  };

  if (warp == 0) {
    if (ptx::elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < work_items && ok; w += gridDim.x) {
        const PGWork k = decode(w);
        const int b_row_base = k.expert * p.b_rows_per_expert;
        for (int kb = 0; kb < k.num_kb; ++kb, ++it) {
          const int s = it % PG_STAGES;
          if (!ptx::mbar_wait(&empty[s], ((it / PG_STAGES) & 1) ^ 1, 1u << 20)) { report_error(p.err, ERR_MMA_WAIT); ok = false; break; }
          uint8_t* a_dst = smem + s * STAGE_BYTES;
          uint8_t* b_dst = a_dst + A_BYTES;
          ptx::mbar_expect_tx(&full[s], STAGE_BYTES);
          const int k0 = k.k_begin + kb * PG_BK;
          if (A_MN) {                         // A stored [rows, M]: boxes of 64 columns
#pragma unroll
            for (int i = 0; i < PG_BM / 64; ++i) ptx::tma_load_3d(a_dst + i * 8192, &tmA, &full[s], k.m0 + 64 * i, k0, 0);
          } else {
            ptx::tma_load_3d(a_dst, &tmA, &full[s], k0, k.row0, 0);
          }
          if (EPI == PE_WGRAD) {              // B stored [rows, N], the same sorted rows as A
            for (int i = 0; i < p.bn_alloc / 64; ++i) ptx::tma_load_3d(b_dst + i * 8192, &tmB, &full[s], k.n0 + 64 * i, k0, 0);
          } else if (B_MN) {                  // B_e stored [K, N]: row = expert * K + k, boxes of 64 columns
            for (int i = 0; i < p.bn_alloc / 64; ++i) ptx::tma_load_3d(b_dst + i * 8192, &tmB, &full[s], k.n0 + 64 * i, b_row_base + k0, 0);
          } else if (EPI == PE_SWIGLU) {      // gate rows [n0, n0 + bn) and up rows [f + n0, f + n0 + bn) of expert e
            ptx::tma_load_3d(b_dst, &tmB, &full[s], k0, b_row_base + k.n0, 0);
            ptx::tma_load_3d(b_dst + p.bn * PG_BK * 2, &tmB, &full[s], k0, b_row_base + p.N + k.n0, 0);
          } else {
            ptx::tma_load_3d(b_dst, &tmB, &full[s], k0, b_row_base + k.n0, 0);
          }
        }
      }
    }
  } else if (warp == 1) {
    const uint32_t idesc = ptx::umma_idesc_bf16(PG_BM, p.bn, A_MN, B_MN);
    uint32_t it = 0, item = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < work_items && ok; w += gridDim.x) {
      const PGWork k = decode(w);
      if (k.num_kb == 0) continue;
      const int acc = item & 1;
      if (!ptx::mbar_wait(&acc_empty[acc], ((item >> 1) & 1) ^ 1, 1u << 22)) { if (lane == 0) report_error(p.err, ERR_EPILOGUE_WAIT); ok = false; break; }
      ptx::tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * PG_ACC_COLS;
      for (int kb = 0; kb < k.num_kb; ++kb, ++it) {
        const int s = it % PG_STAGES;
        if (!ptx::mbar_wait(&full[s], (it / PG_STAGES) & 1, 1u << 20)) { if (lane == 0) report_error(p.err, ERR_TMA_WAIT); ok = false; break; }
        uint8_t* a_tile = smem + s * STAGE_BYTES;
        if (EPI == PE_WGRAD) {
          const int valid = k.rows - kb * PG_BK;            // K rows of this block that belong to the expert
          if (valid < PG_BK) {
            // an MN-major box is 64 K-rows of 128 bytes; rows past the expert's range hold another expert's rows or memory
            // never written, in both operands (the B boxes follow the A boxes in the stage): clear them
            const int boxes = PG_BM / 64 + p.bn_alloc / 64, per_box = (PG_BK - valid) * 8;
            for (int i = lane; i < per_box * boxes; i += 32) {
              const int box = i / per_box, rem = i % per_box;
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
          for (int j = 0; j < PG_BK / 16; ++j) {
            const uint64_t a_desc = A_MN ? ptx::umma_smem_desc_sw128(a_base + j * 2048, 8192, 1024) : ptx::umma_smem_desc_sw128(a_base + j * 32, 0, 1024);
            const uint64_t b_desc = B_MN ? ptx::umma_smem_desc_sw128(b_base + j * 2048, 8192, 1024) : ptx::umma_smem_desc_sw128(b_base + j * 32, 0, 1024);
            ptx::umma_f16(d_tmem, a_desc, b_desc, idesc, (kb | j) != 0);
            if (EPI == PE_SWIGLU) {
              const uint64_t u_desc = ptx::umma_smem_desc_sw128(b_base + p.bn * PG_BK * 2 + j * 32, 0, 1024);
              ptx::umma_f16(d_tmem + p.bn, a_desc, u_desc, idesc, (kb | j) != 0);
            }
          }
          ptx::umma_commit(&empty[s]);
        }
        __syncwarp();
      }
      if (ok && ptx::elect_one()) ptx::umma_commit(&acc_full[acc]);
      __syncwarp();
      ++item;
    }
  } else {
    const int quarter = warp & 3, r_local = quarter * 32 + lane, group = (warp - 2) >> 2;      // the two warpgroups take alternate 16-column chunks
    uint32_t item = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < work_items && ok; w += gridDim.x) {
      const PGWork k = decode(w);
      if (k.num_kb == 0) continue;
      const int rows = k.rows, n0 = k.n0;
      const int acc = item & 1;
      const uint32_t lane_addr = tmem_base + acc * PG_ACC_COLS + (uint32_t(quarter * 32) << 16);
      if (EPI == PE_WGRAD) {
        // C is read before the accumulator is awaited and one chunk ahead of its use: the row-per-thread read-modify-write is
        // latency bound otherwise
        const int crow = k.m0 + r_local;
        const bool live = crow < p.M, vec = p.ld0 % 4 == 0;
        float* c_row = reinterpret_cast<float*>(p.out0) + k.expert * p.c_expert_stride + (long long)crow * p.ld0;
        float4 cur[4], nxt[4];
        auto fetch = [&](int c, float4 (&dst)[4]) {
          if (live && vec && c + 16 <= p.N) {
#pragma unroll
            for (int v = 0; v < 4; ++v) dst[v] = reinterpret_cast<const float4*>(c_row + c)[v];
          }
        };
        fetch(n0 + 16 * group, cur);
        if (!ptx::mbar_wait(&acc_full[acc], (item >> 1) & 1, 1u << 22)) { report_error(p.err, ERR_EPILOGUE_WAIT); ok = false; break; }
        ptx::tc_fence_after();
        for (int c0 = 16 * group; c0 < p.bn; c0 += 32) {
          uint32_t r[16];
          ptx::tmem_ld_32x32b_x16(lane_addr + c0, r);
          if (c0 + 32 < p.bn) fetch(n0 + c0 + 32, nxt);
          ptx::tmem_ld_wait();
          const int c = n0 + c0;
          if (live) {
            if (vec && c + 16 <= p.N) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                float4 o = cur[v];
                o.x += __uint_as_float(r[4 * v]); o.y += __uint_as_float(r[4 * v + 1]);
                o.z += __uint_as_float(r[4 * v + 2]); o.w += __uint_as_float(r[4 * v + 3]);
                reinterpret_cast<float4*>(c_row + c)[v] = o;
              }
            } else {
#pragma unroll
              for (int e = 0; e < 16; ++e) if (c + e < p.N) c_row[c + e] += __uint_as_float(r[e]);
            }
          }
#pragma unroll
          for (int v = 0; v < 4; ++v) cur[v] = nxt[v];
        }
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&acc_empty[acc]);
        ++item;
        continue;
      }
      if (!ptx::mbar_wait(&acc_full[acc], (item >> 1) & 1, 1u << 22)) { report_error(p.err, ERR_EPILOGUE_WAIT); ok = false; break; }
      ptx::tc_fence_after();
      const bool live = r_local < rows;
      const long long row = k.row0 + r_local;
      if (EPI == PE_DSWIGLU) {
        // accumulator = d(hmid) for f = p.N columns.  The gate/up values of a chunk do not depend on the accumulator, so they are
        // fetched one chunk ahead: the global-load latency hides behind the TMEM read and the arithmetic of the chunk before.
        const __nv_bfloat16* gu = reinterpret_cast<const __nv_bfloat16*>(p.out1) + row * p.ld1;
        __nv_bfloat16* dgu = reinterpret_cast<__nv_bfloat16*>(p.out0) + row * p.ld0;
        const bool vec = p.N % 8 == 0;
        uint4 cur[4], nxt[4];
        auto fetch = [&](int c, uint4 (&dst)[4]) {
          if (live && vec && c + 16 <= p.N) {
            dst[0] = reinterpret_cast<const uint4*>(gu + c)[0]; dst[1] = reinterpret_cast<const uint4*>(gu + c)[1];
            dst[2] = reinterpret_cast<const uint4*>(gu + p.N + c)[0]; dst[3] = reinterpret_cast<const uint4*>(gu + p.N + c)[1];
          }
        };
        fetch(n0 + 16 * group, cur);
        for (int c0 = 16 * group; c0 < p.bn; c0 += 32) {
          uint32_t r[16];
          ptx::tmem_ld_32x32b_x16(lane_addr + c0, r);
          if (c0 + 32 < p.bn) fetch(n0 + c0 + 32, nxt);
          ptx::tmem_ld_wait();
          const int c = n0 + c0;
          if (live) {
            if (vec && c + 16 <= p.N) {
              const __nv_bfloat16* gp = reinterpret_cast<const __nv_bfloat16*>(cur);
              const __nv_bfloat16* up = gp + 16;
              float dg[16], du_[16];
#pragma unroll
              for (int e = 0; e < 16; ++e) {
                const float dh = bf16_round(__uint_as_float(r[e]));
                const float g = __bfloat162float(gp[e]), uu = __bfloat162float(up[e]);
                const float sg = sigmoidf_(g);
                dg[e] = dh * uu * sg * (1.f + g * (1.f - sg));
                du_[e] = dh * g * sg;
              }
              pg_store16(dgu + c, dg);
              pg_store16(dgu + p.N + c, du_);
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
#pragma unroll
          for (int i = 0; i < 4; ++i) cur[i] = nxt[i];
        }
      } else
      for (int c0 = 16 * group; c0 < p.bn; c0 += 32) {
        uint32_t r[16];
        ptx::tmem_ld_32x32b_x16(lane_addr + c0, r);
        const int c = n0 + c0;
        if (EPI == PE_SWIGLU) {
          uint32_t u[16];
          ptx::tmem_ld_32x32b_x16(lane_addr + p.bn + c0, u);
          ptx::tmem_ld_wait();
          if (live && c < p.N) {                            // f % 16 == 0: a 16-column group is valid as a whole or not at all
            __nv_bfloat16* gu = reinterpret_cast<__nv_bfloat16*>(p.out1) + row * p.ld1;
            __nv_bfloat16* hm = reinterpret_cast<__nv_bfloat16*>(p.out0) + row * p.ld0;
            float gv[16], uv[16], hv[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              gv[e] = bf16_round(__uint_as_float(r[e]));
              uv[e] = bf16_round(__uint_as_float(u[e]));
              hv[e] = bf16_round(siluf_(gv[e])) * uv[e];
            }
            pg_store16(gu + c, gv);
            pg_store16(gu + p.N + c, uv);
            pg_store16(hm + c, hv);
          }
          continue;
        }
        ptx::tmem_ld_wait();
        if (!live) continue;
        if (EPI == PE_STORE) {
          __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out0) + row * p.ld0;
          if (c + 16 <= p.N && p.ld0 % 8 == 0) {
            float v[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) v[e] = __uint_as_float(r[e]);
            pg_store16(o + c, v);
          } else {
#pragma unroll
            for (int e = 0; e < 16; ++e) if (c + e < p.N) o[c + e] = __float2bfloat16_rn(__uint_as_float(r[e]));
          }
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&acc_empty[acc]);
      ++item;
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) ptx::tmem_dealloc(tmem_base, 512);
}


// ---- host ----------------------------------------------------------------------------------------------------------------------
static int g_persistent_override = -1;          // -1: the environment decides; 0 / 1: set by moe_set_persistent (tests, A/B timing)
void moe_set_persistent(int64_t mode) { g_persistent_override = (int)mode; }
bool moe_persistent_enabled() {
  static const bool on = [] { const char* v = std::getenv("Q38_MOE_PERSISTENT"); return v == nullptr || v[0] != '0'; }();
  return g_persistent_override < 0 ? on : g_persistent_override != 0;
}

// N tile: a multiple of 16 up to `limit` columns that covers N with the least tile time (a tile costs its width plus a fixed part).
static int pg_pick_bn(int N, int limit) {
  if (N <= 64) return 64;
  int best = 128;
  double best_cost = 1e30;
  for (int bn = limit; bn >= 64; bn -= 16) {
    const int tiles = (N + bn - 1) / bn;
    const double cost = tiles * (bn + 32.0);
    if (cost < best_cost - 1e-9) { best = bn; best_cost = cost; }
  }
  return best;
}

template <int EPI, bool B_MN, bool A_MN = false>
static void pg_launch(const CUtensorMap& ta, const CUtensorMap& tb, PGroupedArgs p, int max_tiles, cudaStream_t stream) {
  auto kernel = grouped_persistent_kernel<EPI, B_MN, A_MN>;
  constexpr int nacc = EPI == PE_SWIGLU ? 2 : 1;
  p.bn_alloc = B_MN ? (p.bn + 63) / 64 * 64 : p.bn;
  const int smem = PG_STAGES * (PG_BM * PG_BK * 2 + nacc * p.bn_alloc * PG_BK * 2) + 1024 + 256;
  static bool configured = false;
  if (!configured) { C10_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024)); configured = true; }
  const int grid = std::max(1, std::min(max_tiles * p.tiles_n, kNumSMs));
  kernel<<<grid, PG_THREADS, smem, stream>>>(ta, tb, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

static void pg_check(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 2 && t.is_contiguous(), name, ": contiguous 2-D bf16 CUDA tensor required");
}

// rows [P, K] sorted; weight [E, N, K] (K-major) or [E, K, N] (b_mn_major); out [P, N]
void moe_grouped_gemm_p(const at::Tensor& rows, const at::Tensor& weight, at::Tensor& out, const at::Tensor& sched, bool b_mn_major, at::Tensor& err) {
  pg_check(rows, "moe_grouped_gemm rows"); pg_check(out, "moe_grouped_gemm out");
  TORCH_CHECK(weight.dim() == 3 && weight.is_contiguous() && weight.scalar_type() == at::kBFloat16, "moe_grouped_gemm: weight must be contiguous bf16 [E,*,*]");
  const c10::cuda::CUDAGuard guard(rows.device());
  const int P = rows.size(0), K = rows.size(1), E = weight.size(0);
  const int N = b_mn_major ? weight.size(2) : weight.size(1);
  TORCH_CHECK((b_mn_major ? weight.size(1) : weight.size(2)) == K && out.size(0) == P && out.size(1) == N, "moe_grouped_gemm: shape mismatch");
  const int bn = pg_pick_bn(N, 256), max_tiles = (sched.numel() - 1) / 3;
  CUtensorMap ta = make_tmap_bf16(rows.data_ptr(), K, P, 1, K, 0, PG_BM);
  CUtensorMap tb = b_mn_major ? make_tmap_bf16(weight.data_ptr(), N, (int64_t)E * K, 1, N, 0, 64) : make_tmap_bf16(weight.data_ptr(), K, (int64_t)E * N, 1, K, 0, bn);
  PGroupedArgs p{};
  p.sched = sched.data_ptr<int>(); p.bn = bn; p.tiles_n = (N + bn - 1) / bn; p.K = K; p.N = N; p.b_rows_per_expert = b_mn_major ? K : N;
  p.out0 = out.data_ptr(); p.ld0 = N; p.err = err.data_ptr<int>();
  auto stream = at::cuda::getCurrentCUDAStream();
  if (b_mn_major) pg_launch<PE_STORE, true>(ta, tb, p, max_tiles, stream);
  else pg_launch<PE_STORE, false>(ta, tb, p, max_tiles, stream);
}

// rows [P, h], gate_up weight [E, 2f, h] -> hmid [P, f], gu [P, 2f]
void moe_grouped_swiglu_p(const at::Tensor& rows, const at::Tensor& weight, at::Tensor& hmid, at::Tensor& gu, const at::Tensor& sched, at::Tensor& err) {
  pg_check(rows, "moe_grouped_swiglu rows"); pg_check(hmid, "hmid"); pg_check(gu, "gu");
  const c10::cuda::CUDAGuard guard(rows.device());
  const int P = rows.size(0), K = rows.size(1), E = weight.size(0), f = weight.size(1) / 2;
  TORCH_CHECK(weight.size(2) == K && f % 16 == 0 && f <= 256 && hmid.size(1) == f && gu.size(1) == 2 * f, "moe_grouped_swiglu: expert width must be a multiple of 16, at most 256");
  const int tiles_n = (f + 127) / 128, bn = ((f + tiles_n - 1) / tiles_n + 15) / 16 * 16;       // gate and up accumulators of one set share 256 columns
  const int max_tiles = (sched.numel() - 1) / 3;
  CUtensorMap ta = make_tmap_bf16(rows.data_ptr(), K, P, 1, K, 0, PG_BM);
  CUtensorMap tb = make_tmap_bf16(weight.data_ptr(), K, (int64_t)E * 2 * f, 1, K, 0, bn);
  PGroupedArgs p{};
  p.sched = sched.data_ptr<int>(); p.bn = bn; p.tiles_n = tiles_n; p.K = K; p.N = f; p.b_rows_per_expert = 2 * f;
  p.out0 = hmid.data_ptr(); p.ld0 = f; p.out1 = gu.data_ptr(); p.ld1 = 2 * f; p.err = err.data_ptr<int>();
  pg_launch<PE_SWIGLU, false>(ta, tb, p, max_tiles, at::cuda::getCurrentCUDAStream());
}

// d(hmid) = dy_sorted [P, h] . W_down[e] ([h, f], MN-major B), fused SwiGLU backward -> dgu [P, 2f]
void moe_grouped_dswiglu_p(const at::Tensor& dy, const at::Tensor& w_down, const at::Tensor& gu, at::Tensor& dgu, const at::Tensor& sched, at::Tensor& err) {
  pg_check(dy, "dy"); pg_check(gu, "gu"); pg_check(dgu, "dgu");
  const c10::cuda::CUDAGuard guard(dy.device());
  const int P = dy.size(0), K = dy.size(1), E = w_down.size(0), f = w_down.size(2);
  TORCH_CHECK(w_down.size(1) == K && gu.size(1) == 2 * f && dgu.size(1) == 2 * f && f % 8 == 0, "moe_grouped_dswiglu: shape mismatch");
  const int bn = pg_pick_bn(f, 256), max_tiles = (sched.numel() - 1) / 3;
  CUtensorMap ta = make_tmap_bf16(dy.data_ptr(), K, P, 1, K, 0, PG_BM);
  CUtensorMap tb = make_tmap_bf16(w_down.data_ptr(), f, (int64_t)E * K, 1, f, 0, 64);
  PGroupedArgs p{};
  p.sched = sched.data_ptr<int>(); p.bn = bn; p.tiles_n = (f + bn - 1) / bn; p.K = K; p.N = f; p.b_rows_per_expert = K;
  p.out0 = dgu.data_ptr(); p.ld0 = 2 * f; p.out1 = const_cast<void*>(gu.data_ptr()); p.ld1 = 2 * f; p.err = err.data_ptr<int>();
  pg_launch<PE_DSWIGLU, true>(ta, tb, p, max_tiles, at::cuda::getCurrentCUDAStream());
}

// grad[e] += a[rows of e]^T b[rows of e]:  a [P, M], b [P, N] sorted by expert, grad [E, M, N] fp32, offsets [E + 1]
void moe_grouped_wgrad_p(const at::Tensor& a, const at::Tensor& b, at::Tensor& grad, const at::Tensor& offsets, at::Tensor& err) {
  pg_check(a, "wgrad a"); pg_check(b, "wgrad b");
  TORCH_CHECK(grad.is_cuda() && grad.scalar_type() == at::kFloat && grad.dim() == 3 && grad.is_contiguous(), "moe_grouped_wgrad: grad must be contiguous fp32 [E,M,N]");
  const c10::cuda::CUDAGuard guard(a.device());
  const int P = a.size(0), M = a.size(1), N = b.size(1), E = grad.size(0);
  TORCH_CHECK(b.size(0) == P && grad.size(1) == M && grad.size(2) == N && M % 8 == 0 && N % 8 == 0 && offsets.numel() == E + 1, "moe_grouped_wgrad: shape mismatch");
  const int bn = pg_pick_bn(N, 256);
  CUtensorMap ta = make_tmap_bf16(a.data_ptr(), M, P, 1, M, 0, 64);
  CUtensorMap tb = make_tmap_bf16(b.data_ptr(), N, P, 1, N, 0, 64);
  PGroupedArgs p{};
  p.offsets = offsets.data_ptr<int>(); p.experts = E; p.tiles_m = (M + PG_BM - 1) / PG_BM; p.M = M; p.c_expert_stride = (long long)M * N;
  p.bn = bn; p.tiles_n = (N + bn - 1) / bn; p.N = N; p.K = 0; p.out0 = grad.data_ptr(); p.ld0 = N; p.err = err.data_ptr<int>();
  pg_launch<PE_WGRAD, true, true>(ta, tb, p, E * p.tiles_m, at::cuda::getCurrentCUDAStream());
}

}  // namespace q38
