// Persistent bf16 GEMM: one CTA per SM walks a list of (tile, K-split) work items.  Three roles run concurrently and are
// decoupled by mbarrier rings, so the accumulator read-out of one tile overlaps the MMAs of the next:
//
//   warp 0   TMA producer: fills a 4-stage ring of {A 128 x 64, B bn x 64} bf16 tiles across tile boundaries
//   warp 1   MMA issuer (one elected lane): tcgen05.mma into one of two TMEM accumulators (256 columns each)
//   warps 2-5 epilogue: tcgen05.ld of the finished accumulator, conversion, global stores (or fp32 accumulation)
//
// bn (the UMMA N) is chosen per problem as a multiple of 16 up to 256 that tiles N with little waste (576 -> 192,
// 2240 -> 224, 10112 -> 256).  Operands may be K-major or MN-major exactly as in gemm.cu; all waits are bounded.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <cstdio>
#include <cstdlib>

#include "ptx.cuh"
#include "host.h"

namespace q38 {

constexpr int P_BM = 128, P_BK = 64, P_STAGES = 4, P_THREADS = 192, P_ACC_COLS = 256;

struct PGemmArgs {
  int M, N, K, batch, bn;
  int tiles_m, tiles_n, splits, kb_per_split, total_kb, work_items;
  void* C;
  long long ldc, c_batch_stride;
  float alpha;
  int* err;
  // optional addend (bf16 outputs): C = alpha * A.B^T + beta * Cin, Cin bf16 with the shape of C and its own strides
  const __nv_bfloat16* Cin;
  long long ldcin, cin_batch_stride;
  float beta;
};

// TMA_OUT: every epilogue warp stages 32 rows x 32 columns in shared memory (64-byte swizzle for bf16, 128-byte for fp32, both
// conflict free) and hands the box to the TMA unit, which writes full lines and clips rows >= M and columns >= N; with ACCUM the
// box is added to global memory by the TMA unit (one reduction per element, so split-K partial sums need no atomics loop).
// Two staging buffers per warp.
// TF32: fp32 operands (K-major only) read by TMA and multiplied as tf32; a stage then holds 32 elements of K per row.
template <bool A_MN, bool B_MN, typename OutT, bool ACCUM, bool TMA_OUT, bool TF32 = false>
__global__ void __launch_bounds__(P_THREADS) gemm_persistent_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                                                                    const __grid_constant__ CUtensorMap tmC, PGemmArgs p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  const int A_BYTES = P_BM * 128, B_BYTES = p.bn * 128, STAGE_BYTES = A_BYTES + B_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + P_STAGES * STAGE_BYTES);
  uint64_t* empty = full + P_STAGES;
  uint64_t* acc_full = empty + P_STAGES;        // [2]
  uint64_t* acc_empty = acc_full + 2;           // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  uint8_t* stage_out = smem + P_STAGES * STAGE_BYTES + 1024;     // [4 warps][2 buffers][32 rows x 128 bytes], 1024-byte aligned
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&tmA);
    ptx::prefetch_tensormap(&tmB);
    if (TMA_OUT) ptx::prefetch_tensormap(&tmC);
    for (int s = 0; s < P_STAGES; ++s) { ptx::mbar_init(&full[s], 1); ptx::mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { ptx::mbar_init(&acc_full[a], 1); ptx::mbar_init(&acc_empty[a], 4); }   // four epilogue warps release an accumulator
    ptx::fence_barrier_init();
  }
  if (warp == 1) { ptx::tmem_alloc(tmem_slot, 512); ptx::tmem_relinquish(); }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // work item -> (batch, m tile, n tile, split); n fastest so consecutive items reuse the A tile from L2
  auto decode = [&](int w, int& bz, int& m0, int& n0, int& kb_begin, int& num_kb) {
    const int split = w % p.splits; w /= p.splits;
    const int tn = w % p.tiles_n; w /= p.tiles_n;
    const int tm = w % p.tiles_m; bz = w / p.tiles_m;
    m0 = tm * P_BM; n0 = tn * p.bn;
    kb_begin = split * p.kb_per_split;
    num_kb = min(p.kb_per_split, p.total_kb - kb_begin);
  };

  if (warp == 0) {
    if (ptx::elect_one()) {
      uint32_t it = 0;                                       // global K-block counter: stage = it % STAGES, round = it / STAGES
      bool ok = true;
      for (int w = blockIdx.x; w < p.work_items && ok; w += gridDim.x) {
        int bz, m0, n0, kb_begin, num_kb;
        decode(w, bz, m0, n0, kb_begin, num_kb);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % P_STAGES;
          if (!ptx::mbar_wait(&empty[s], ((it / P_STAGES) & 1) ^ 1, 1u << 20)) { report_error(p.err, ERR_MMA_WAIT); ok = false; break; }
          uint8_t* a_dst = smem + s * STAGE_BYTES;
          uint8_t* b_dst = a_dst + A_BYTES;
          ptx::mbar_expect_tx(&full[s], STAGE_BYTES);
          const int k0 = (kb_begin + kb) * (TF32 ? P_BK / 2 : P_BK);
          if (A_MN) {
#pragma unroll
            for (int i = 0; i < P_BM / 64; ++i) ptx::tma_load_3d(a_dst + i * 8192, &tmA, &full[s], m0 + 64 * i, k0, bz);
          } else {
            ptx::tma_load_3d(a_dst, &tmA, &full[s], k0, m0, bz);
          }
          if (B_MN) {
            for (int i = 0; i < p.bn / 64; ++i) ptx::tma_load_3d(b_dst + i * 8192, &tmB, &full[s], n0 + 64 * i, k0, bz);
          } else {
            ptx::tma_load_3d(b_dst, &tmB, &full[s], k0, n0, bz);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (ptx::elect_one()) {
      const uint32_t idesc = TF32 ? ptx::umma_idesc_tf32(P_BM, p.bn, false, false) : ptx::umma_idesc_bf16(P_BM, p.bn, A_MN, B_MN);
      uint32_t it = 0, tile = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < p.work_items && ok; w += gridDim.x, ++tile) {
        int bz, m0, n0, kb_begin, num_kb;
        decode(w, bz, m0, n0, kb_begin, num_kb);
        const int acc = tile & 1;
        // the epilogue must have drained this accumulator (two tiles ago)
        if (!ptx::mbar_wait(&acc_empty[acc], ((tile >> 1) & 1) ^ 1, 1u << 22)) { report_error(p.err, ERR_EPILOGUE_WAIT); ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * P_ACC_COLS;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % P_STAGES;
          if (!ptx::mbar_wait(&full[s], (it / P_STAGES) & 1, 1u << 20)) { report_error(p.err, ERR_TMA_WAIT); ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t a_base = ptx::smem_u32(smem + s * STAGE_BYTES), b_base = a_base + A_BYTES;
#pragma unroll
          for (int j = 0; j < P_BK / 16; ++j) {
            const uint64_t a_desc = A_MN ? ptx::umma_smem_desc_sw128(a_base + j * 2048, 8192, 1024) : ptx::umma_smem_desc_sw128(a_base + j * 32, 0, 1024);
            const uint64_t b_desc = B_MN ? ptx::umma_smem_desc_sw128(b_base + j * 2048, 8192, 1024) : ptx::umma_smem_desc_sw128(b_base + j * 32, 0, 1024);
            if (TF32) ptx::umma_tf32(d_tmem, a_desc, b_desc, idesc, (kb | j) != 0);
            else ptx::umma_f16(d_tmem, a_desc, b_desc, idesc, (kb | j) != 0);
          }
          ptx::umma_commit(&empty[s]);
        }
        if (ok) ptx::umma_commit(&acc_full[acc]);
      }
    }
  } else {
    const int quarter = warp & 3;
    uint32_t tile = 0, chunk = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < p.work_items && ok; w += gridDim.x, ++tile) {
      int bz, m0, n0, kb_begin, num_kb;
      decode(w, bz, m0, n0, kb_begin, num_kb);
      const int acc = tile & 1;
      if (!ptx::mbar_wait(&acc_full[acc], (tile >> 1) & 1, 1u << 22)) { report_error(p.err, ERR_EPILOGUE_WAIT); ok = false; break; }
      ptx::tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      OutT* c_row = reinterpret_cast<OutT*>(p.C) + bz * p.c_batch_stride + (long long)row * p.ldc;
      const bool vec_ok = (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) && (p.c_batch_stride % 8 == 0);
      const uint32_t t_addr = tmem_base + acc * P_ACC_COLS + (uint32_t(quarter * 32) << 16);
      for (int c0 = 0; c0 < p.bn; c0 += 32) {
        uint32_t r[32];
        ptx::tmem_ld_32x32b_x32(t_addr + c0, r);
        ptx::tmem_ld_wait();
        float alpha = p.alpha;
        if constexpr (sizeof(OutT) == 2) {
          if (p.Cin != nullptr) {                              // fold alpha * acc + beta * Cin into the registers
            if (row < p.M) {
              const __nv_bfloat16* cin_row = p.Cin + bz * p.cin_batch_stride + (long long)row * p.ldcin;
              const bool cin_vec = (p.ldcin % 8 == 0) && (p.cin_batch_stride % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.Cin) & 15) == 0);
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                const int col = n0 + c0 + v * 8;
                if (cin_vec && col + 8 <= p.N) {
                  const uint4 q = *reinterpret_cast<const uint4*>(cin_row + col);
                  const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qw[e]));
                    r[v * 8 + 2 * e] = __float_as_uint(__uint_as_float(r[v * 8 + 2 * e]) * alpha + p.beta * f.x);
                    r[v * 8 + 2 * e + 1] = __float_as_uint(__uint_as_float(r[v * 8 + 2 * e + 1]) * alpha + p.beta * f.y);
                  }
                } else {
#pragma unroll
                  for (int e = 0; e < 8; ++e) {
                    const float c = (col + e < p.N) ? __bfloat162float(cin_row[col + e]) : 0.f;
                    r[v * 8 + e] = __float_as_uint(__uint_as_float(r[v * 8 + e]) * alpha + p.beta * c);
                  }
                }
              }
            }
            alpha = 1.f;
          }
        }
        if constexpr (TMA_OUT) {
          uint8_t* buf = stage_out + (quarter * 2 + (chunk & 1)) * 4096;
          if (lane == 0) ptx::bulk_wait_read<1>();               // the store issued two chunks ago has read this buffer
          __syncwarp();
          if constexpr (sizeof(OutT) == 2) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint32_t wd[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * e]) * alpha, __uint_as_float(r[v * 8 + 2 * e + 1]) * alpha);
                wd[e] = *reinterpret_cast<uint32_t*>(&h2);
              }
              *reinterpret_cast<uint4*>(buf + lane * 64 + ((v ^ ((lane >> 1) & 3)) << 4)) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
            }
          } else {
#pragma unroll
            for (int v = 0; v < 8; ++v)
              *reinterpret_cast<float4*>(buf + lane * 128 + ((v ^ (lane & 7)) << 4)) =
                  make_float4(__uint_as_float(r[v * 4]) * alpha, __uint_as_float(r[v * 4 + 1]) * alpha, __uint_as_float(r[v * 4 + 2]) * alpha,
                              __uint_as_float(r[v * 4 + 3]) * alpha);
          }
          ptx::fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            if (n0 + c0 < p.N && m0 + quarter * 32 < p.M) {
              if constexpr (ACCUM) ptx::tma_reduce_add_3d(&tmC, buf, n0 + c0, m0 + quarter * 32, bz);
              else ptx::tma_store_3d(&tmC, buf, n0 + c0, m0 + quarter * 32, bz);
            }
            ptx::bulk_commit();                                  // possibly empty: keeps the buffer accounting uniform
          }
          ++chunk;
          continue;
        }
        if (row < p.M) {
          const int col0 = n0 + c0;
          if (vec_ok && col0 + 32 <= p.N && c0 + 32 <= p.bn) {
            if constexpr (sizeof(OutT) == 2) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint32_t wd[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * e]) * alpha, __uint_as_float(r[v * 8 + 2 * e + 1]) * alpha);
                  wd[e] = *reinterpret_cast<uint32_t*>(&h2);
                }
                *reinterpret_cast<uint4*>(c_row + col0 + v * 8) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
              }
            } else {
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                float4* dst = reinterpret_cast<float4*>(c_row + col0 + v * 4);
                float4 o = make_float4(__uint_as_float(r[v * 4]) * alpha, __uint_as_float(r[v * 4 + 1]) * alpha,
                                       __uint_as_float(r[v * 4 + 2]) * alpha, __uint_as_float(r[v * 4 + 3]) * alpha);
                if (ACCUM && p.splits > 1) {
                  float* d = reinterpret_cast<float*>(dst);
                  atomicAdd(d, o.x); atomicAdd(d + 1, o.y); atomicAdd(d + 2, o.z); atomicAdd(d + 3, o.w);
                } else {
                  if (ACCUM) { float4 c = *dst; o.x += c.x; o.y += c.y; o.z += c.z; o.w += c.w; }
                  *dst = o;
                }
              }
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              if (col0 + e < p.N && c0 + e < p.bn) {
                float v = __uint_as_float(r[e]) * alpha;
                if constexpr (ACCUM && sizeof(OutT) == 4) {
                  if (p.splits > 1) { atomicAdd(reinterpret_cast<float*>(c_row) + col0 + e, v); continue; }
                }
                if (ACCUM) v += to_float<OutT>(c_row[col0 + e]);
                c_row[col0 + e] = from_float<OutT>(v);
              }
            }
          }
        }
      }
      // this warp is done reading the accumulator
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&acc_empty[acc]);
    }
    if (TMA_OUT && lane == 0) ptx::bulk_wait<0>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) ptx::tmem_dealloc(tmem_base, 512);
}

static bool trace_on() { static const bool on = std::getenv("Q38_GEMM_TRACE") != nullptr; return on; }   // host-side launch log on stderr
#define Q38_TRACE(...) do { if (trace_on()) { std::fprintf(stderr, __VA_ARGS__); std::fflush(stderr); } } while (0)

// Width of the N tile: most useful columns per unit of tile time, where a tile costs its width plus a fixed part
// (pipeline fill, accumulator hand-over) worth about 32 columns.
static int pick_bn(int N, int step) {
  if (N <= 256) return (N + step - 1) / step * step;
  int best = 256;
  double best_eff = 0.0;
  for (int bn = 256; bn >= 128; bn -= step) {
    const int tiles = (N + bn - 1) / bn;
    const double eff = double(N) / double(tiles * (bn + 32));
    if (eff > best_eff + 1e-9) { best = bn; best_eff = eff; }
  }
  return best;
}

// Number of K slices for an accumulating product: minimise rounds(items / SMs) x (K blocks per slice + fixed cost of an item).
static int pick_splits(int tiles, int total_kb) {
  int best = 1;
  double best_cost = 1e30;
  for (int s = 1; s <= 32 && total_kb / s >= 4; ++s) {
    const int kbps = (total_kb + s - 1) / s, real = (total_kb + kbps - 1) / kbps;
    const int rounds = (tiles * real + kNumSMs - 1) / kNumSMs;
    const double cost = rounds * (kbps + 4.0);
    if (cost < best_cost - 1e-9) { best = real; best_cost = cost; }
  }
  return best;
}

template <bool A_MN, bool B_MN, bool TF32 = false>
static void launch_p(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, bool tma_out, const PGemmArgs& p, bool out_fp32, bool accum,
                     cudaStream_t stream) {
  const int smem = P_STAGES * (P_BM * 128 + p.bn * 128) + 1024 /* alignment */ + 1024 /* barriers */ + 4 * 2 * 4096 /* output staging */;
  const int grid = std::min(p.work_items, kNumSMs);
  Q38_TRACE("[gemm_p] launch grid=%d smem=%d bn=%d items=%d splits=%d kb=%d tma_out=%d fp32=%d acc=%d amn=%d bmn=%d\n", grid, smem, p.bn, p.work_items, p.splits,
            p.total_kb, (int)tma_out, (int)out_fp32, (int)accum, (int)A_MN, (int)B_MN);
#define Q38_LAUNCH(OutT, ACC, TMAO) { auto k = gemm_persistent_kernel<A_MN, B_MN, OutT, ACC, TMAO, TF32>; static bool cfg = false; \
    if (!cfg) { C10_CUDA_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024)); cfg = true; } \
    k<<<grid, P_THREADS, smem, stream>>>(ta, tb, tc, p); }
  if constexpr (TF32) {
    if (!out_fp32) { if (tma_out) Q38_LAUNCH(__nv_bfloat16, false, true) else Q38_LAUNCH(__nv_bfloat16, false, false) }
    else if (tma_out) { if (accum) Q38_LAUNCH(float, true, true) else Q38_LAUNCH(float, false, true) }
    else { if (accum) Q38_LAUNCH(float, true, false) else Q38_LAUNCH(float, false, false) }
  } else if (tma_out) {
    if (!out_fp32) { if (accum) Q38_LAUNCH(__nv_bfloat16, true, true) else Q38_LAUNCH(__nv_bfloat16, false, true) }
    else if (accum) Q38_LAUNCH(float, true, true)
    else Q38_LAUNCH(float, false, true)
  } else {
    if (!out_fp32) Q38_LAUNCH(__nv_bfloat16, false, false)
    else if (accum) Q38_LAUNCH(float, true, false)
    else Q38_LAUNCH(float, false, false)
  }
#undef Q38_LAUNCH
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  if (trace_on()) {
    cudaError_t e = cudaStreamSynchronize(stream);
    Q38_TRACE("[gemm_p] done: %s\n", cudaGetErrorString(e));
  }
}

bool gemm_pair_enabled();                                                                                                         // gemm_pair.cu
bool gemm_bf16_pair(const at::Tensor& a, const at::Tensor& b, at::Tensor& c, double alpha, bool accumulate, at::Tensor& err);   // gemm_pair.cu

// Same contract as gemm_bf16 (bf16 operands only).
void gemm_bf16_persistent(const at::Tensor& a, const at::Tensor& b, at::Tensor& c, bool a_mn_major, bool b_mn_major, double alpha,
                          bool accumulate, at::Tensor& err, int64_t splits, const c10::optional<at::Tensor>& addend, double beta) {
  const bool tf32 = a.scalar_type() == at::kFloat;
  TORCH_CHECK(a.is_cuda() && (tf32 || a.scalar_type() == at::kBFloat16) && b.scalar_type() == a.scalar_type() && a.dim() == 3 && b.dim() == 3 && c.dim() == 3,
              "gemm_bf16_persistent: bf16 (or fp32 for tf32 math) [batch, rows, cols] operands required");
  TORCH_CHECK(!tf32 || (!a_mn_major && !b_mn_major), "gemm_bf16_persistent: the tf32 path takes K-major operands only");
  const int eb = tf32 ? 4 : 2, bk = 128 / eb;
  TORCH_CHECK(a.stride(2) == 1 && b.stride(2) == 1 && c.stride(2) == 1, "gemm_bf16_persistent: innermost dimension must be contiguous");
  const c10::cuda::CUDAGuard guard(a.device());
  const int batch = a.size(0);
  const int M = a_mn_major ? a.size(2) : a.size(1), K = a_mn_major ? a.size(1) : a.size(2);
  const int N = b_mn_major ? b.size(2) : b.size(1), Kb = b_mn_major ? b.size(1) : b.size(2);
  TORCH_CHECK(K == Kb && b.size(0) == batch && c.size(0) == batch && c.size(1) == M && c.size(2) == N, "gemm_bf16_persistent: shape mismatch");
  const bool out_fp32 = c.scalar_type() == at::kFloat;
  TORCH_CHECK(out_fp32 || c.scalar_type() == at::kBFloat16, "gemm_bf16_persistent: output must be bf16 or fp32");
  const int c_eb = out_fp32 ? 4 : 2, c_vec = 16 / c_eb;
  const bool tma_out = c.stride(1) % c_vec == 0 && (reinterpret_cast<uintptr_t>(c.data_ptr()) & 15) == 0 && (batch == 1 || c.stride(0) % c_vec == 0);
  // bf16 outputs accumulate through the TMA unit only (cp.reduce.async.bulk.tensor adds in the tensor's element type)
  TORCH_CHECK(!accumulate || out_fp32 || (tma_out && !tf32 && !addend.has_value()), "accumulating into a bf16 output requires a TMA-storable output and no addend");
  // K-major x K-major products with a TMA-storable output may run on SM pairs (cta_group::2, gemm_pair.cu) when switched on
  if (gemm_pair_enabled() && !tf32 && !a_mn_major && !b_mn_major && tma_out && !addend.has_value() && (!accumulate || !out_fp32) &&
      gemm_bf16_pair(a, b, c, alpha, accumulate, err))
    return;
  int bn = pick_bn(N, tma_out ? 32 : 16);
  if (b_mn_major) bn = (bn + 63) / 64 * 64;                    // MN-major B is loaded in 64-wide boxes
  bn = std::min(bn, 256);
  Q38_TRACE("[gemm_p] M=%d N=%d K=%d batch=%d a=%p b=%p c=%p strides a(%lld,%lld) b(%lld,%lld) c(%lld,%lld)\n", M, N, K, batch, a.data_ptr(), b.data_ptr(), c.data_ptr(),
            (long long)a.stride(0), (long long)a.stride(1), (long long)b.stride(0), (long long)b.stride(1), (long long)c.stride(0), (long long)c.stride(1));
  PGemmArgs p{};
  p.M = M; p.N = N; p.K = K; p.batch = batch; p.bn = bn;
  p.tiles_m = (M + P_BM - 1) / P_BM; p.tiles_n = (N + bn - 1) / bn;
  p.total_kb = (K + bk - 1) / bk;
  int nsplit = 1;
  if (accumulate && out_fp32) {
    if (splits > 0) nsplit = (int)splits;
    else if (splits == 0) {
      const int tiles = p.tiles_m * p.tiles_n * batch;
      nsplit = pick_splits(tiles, p.total_kb);
    }
  }
  p.kb_per_split = (p.total_kb + nsplit - 1) / nsplit;
  p.splits = (p.total_kb + p.kb_per_split - 1) / p.kb_per_split;
  p.work_items = p.tiles_m * p.tiles_n * batch * p.splits;
  p.C = c.data_ptr(); p.ldc = c.stride(1); p.c_batch_stride = c.stride(0); p.alpha = (float)alpha; p.err = err.data_ptr<int>();
  p.Cin = nullptr; p.ldcin = 0; p.cin_batch_stride = 0; p.beta = 0.f;
  if (addend.has_value()) {
    TORCH_CHECK(!out_fp32 && addend->scalar_type() == at::kBFloat16 && addend->dim() == 3 && addend->size(0) == batch && addend->size(1) == M &&
                addend->size(2) == N && addend->stride(2) == 1, "gemm_bf16_persistent: the addend must be a bf16 tensor of the output's shape (bf16 output only)");
    p.Cin = (const __nv_bfloat16*)addend->data_ptr(); p.ldcin = addend->stride(1); p.cin_batch_stride = addend->stride(0); p.beta = (float)beta;
  }
  CUtensorMap ta, tb;
  Q38_TRACE("[gemm_p] args bn=%d tiles=%dx%d splits=%d items=%d\n", bn, p.tiles_m, p.tiles_n, p.splits, p.work_items);
  ta = make_tmap_box(a.data_ptr(), eb, a.size(2), a.size(1), batch, a.stride(1), a.stride(0), a_mn_major ? 64 : P_BM, 128);
  Q38_TRACE("[gemm_p] map A encoded\n");
  tb = make_tmap_box(b.data_ptr(), eb, b.size(2), b.size(1), batch, b.stride(1), b.stride(0), b_mn_major ? 64 : bn, 128);
  Q38_TRACE("[gemm_p] operand maps encoded\n");
  CUtensorMap tc = tma_out ? make_tmap_box(c.data_ptr(), c_eb, N, M, batch, c.stride(1), c.stride(0), 32, 32 * c_eb) : ta;
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  if (tf32) {
    launch_p<false, false, true>(ta, tb, tc, tma_out, p, out_fp32, accumulate, stream);
  } else if (a_mn_major) {
    if (b_mn_major) launch_p<true, true>(ta, tb, tc, tma_out, p, out_fp32, accumulate, stream);
    else launch_p<true, false>(ta, tb, tc, tma_out, p, out_fp32, accumulate, stream);
  } else {
    if (b_mn_major) launch_p<false, true>(ta, tb, tc, tma_out, p, out_fp32, accumulate, stream);
    else launch_p<false, false>(ta, tb, tc, tma_out, p, out_fp32, accumulate, stream);
  }
}

}  // namespace q38
