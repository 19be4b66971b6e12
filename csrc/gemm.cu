// bf16 GEMM on the 5th-generation tensor cores: TMA -> 128B-swizzled shared memory -> tcgen05.mma -> TMEM -> epilogue.
//
//   C[b][M,N] (=|+=) alpha * A[b] . B[b]^T      fp32 accumulation in TMEM, C stored as bf16 or fp32
//
// Operand layouts (per batch entry), chosen independently for A and B:
//   K-major  : the operand is stored [rows, K] with K contiguous        (forward x.W^T, dgrad with a transposed shadow)
//   MN-major : the operand is stored [K, rows] with rows contiguous     (wgrad dW = dY^T.X reduces over tokens)
// Both are fed by non-multicast TMA tile loads; the MN-major case uses 64x64 boxes, the K-major case 64 x rows boxes.
//
// CTA = 192 threads: warp 0 issues TMA, warp 1 owns TMEM and issues the MMAs (one elected lane), warps 2..5 read
// the 128 x BN accumulator out of TMEM (warp w owns lanes 32*(w%4)..+31) and write C.  Three pipeline stages let two
// CTAs share an SM, so one CTA's epilogue overlaps the other's main loop.  Every wait is bounded; on a timeout the
// role records an error code, falls through to the common exit and TMEM is released.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <mutex>

#include <cstdio>
#include <cstdlib>

#include "ptx.cuh"
#include "host.h"

namespace q38 {

constexpr int BM = 128, STAGES = 3, GEMM_THREADS = 192;
// One pipeline stage holds 128 bytes of K per row: 64 bf16 or 32 fp32 (tf32) elements; one UMMA consumes 32 bytes of K.
template <int EB> struct Elem { static constexpr int BK = 128 / EB, UMMA_K = 32 / EB, MN_BOX = 128 / EB; };

struct GemmArgs {
  int M, N, K, batch;
  int splits, kb_per_split;     // split-K: blockIdx.z = batch * splits + split; partial sums are added atomically
  void* C;
  long long ldc, c_batch_stride;
  float alpha;
  int* err;
};

template <int BN>
constexpr int gemm_smem_bytes() { return STAGES * (BM * 128 + BN * 128) + 1024 /*alignment slack*/ + 256 /*barriers*/; }

template <int EB, int BN, bool A_MN, bool B_MN, typename OutT, bool ACCUM>
__global__ void __launch_bounds__(GEMM_THREADS) gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA,
                                                                  const __grid_constant__ CUtensorMap tmB, GemmArgs p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  constexpr int BK = Elem<EB>::BK, UMMA_K = Elem<EB>::UMMA_K, MN_BOX = Elem<EB>::MN_BOX;
  constexpr int MN_BOX_BYTES = BK * 128;                      // one MN-major TMA box: BK rows of 128 bytes
  constexpr int A_BYTES = BM * 128, B_BYTES = BN * 128, STAGE_BYTES = A_BYTES + B_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_ready = empty + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);
  constexpr uint32_t TMEM_COLS = BN <= 32 ? 32 : BN <= 64 ? 64 : BN <= 128 ? 128 : 256;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM, bz = blockIdx.z / p.splits, split = blockIdx.z % p.splits;
  const int total_kb = (p.K + Elem<EB>::BK - 1) / Elem<EB>::BK;
  const int kb_begin = split * p.kb_per_split;
  const int num_kb = min(p.kb_per_split, total_kb - kb_begin);

  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&tmA);
    ptx::prefetch_tensormap(&tmB);
    for (int s = 0; s < STAGES; ++s) { ptx::mbar_init(&full[s], 1); ptx::mbar_init(&empty[s], 1); }
    ptx::mbar_init(acc_ready, 1);
    ptx::fence_barrier_init();
  }
  if (warp == 1) { ptx::tmem_alloc(tmem_slot, TMEM_COLS); ptx::tmem_relinquish(); }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (ptx::elect_one()) {
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % STAGES, round = kb / STAGES;
        if (!ptx::mbar_wait(&empty[s], (round & 1) ^ 1, 1u << 20)) { report_error(p.err, ERR_MMA_WAIT); break; }
        uint8_t* a_dst = smem + s * STAGE_BYTES;
        uint8_t* b_dst = a_dst + A_BYTES;
        ptx::mbar_expect_tx(&full[s], STAGE_BYTES);
        const int k0 = (kb_begin + kb) * BK;
        if (A_MN) {
#pragma unroll
          for (int i = 0; i < BM / MN_BOX; ++i) ptx::tma_load_3d(a_dst + i * MN_BOX_BYTES, &tmA, &full[s], m0 + MN_BOX * i, k0, bz);
        } else {
          ptx::tma_load_3d(a_dst, &tmA, &full[s], k0, m0, bz);
        }
        if (B_MN) {
#pragma unroll
          for (int i = 0; i < BN / MN_BOX; ++i) ptx::tma_load_3d(b_dst + i * MN_BOX_BYTES, &tmB, &full[s], n0 + MN_BOX * i, k0, bz);
        } else {
          ptx::tma_load_3d(b_dst, &tmB, &full[s], k0, n0, bz);
        }
      }
    }
  } else if (warp == 1) {
    if (ptx::elect_one()) {
      constexpr uint32_t idesc = EB == 2 ? ptx::umma_idesc_bf16(BM, BN, A_MN, B_MN) : ptx::umma_idesc_tf32(BM, BN, A_MN, B_MN);
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % STAGES, round = kb / STAGES;
        if (!ptx::mbar_wait(&full[s], round & 1, 1u << 20)) { report_error(p.err, ERR_TMA_WAIT); ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t a_base = ptx::smem_u32(smem + s * STAGE_BYTES), b_base = a_base + A_BYTES;
#pragma unroll
        for (int j = 0; j < BK / UMMA_K; ++j) {
          // K-major: one UMMA reads 32 bytes of K inside the 128-byte swizzle row; 8-row groups are 1024 bytes apart.
          // MN-major: one UMMA reads UMMA_K rows of 128 bytes; 128-byte MN chunks (one TMA box each) are MN_BOX_BYTES apart.
          const uint64_t a_desc = A_MN ? ptx::umma_smem_desc_sw128(a_base + j * UMMA_K * 128, MN_BOX_BYTES, 1024)
                                       : ptx::umma_smem_desc_sw128(a_base + j * 32, 0, 1024);
          const uint64_t b_desc = B_MN ? ptx::umma_smem_desc_sw128(b_base + j * UMMA_K * 128, MN_BOX_BYTES, 1024)
                                       : ptx::umma_smem_desc_sw128(b_base + j * 32, 0, 1024);
          if (EB == 2) ptx::umma_f16(tmem_base, a_desc, b_desc, idesc, (kb | j) != 0);
          else ptx::umma_tf32(tmem_base, a_desc, b_desc, idesc, (kb | j) != 0);
        }
        ptx::umma_commit(&empty[s]);          // the stage may be refilled once these MMAs have read it
      }
      ptx::umma_commit(acc_ready);            // arrives when every MMA issued above has completed
    }
  } else {
    const int quarter = warp & 3;             // TMEM lanes this warp may read
    const int row = m0 + quarter * 32 + lane;
    bool ok = ptx::mbar_wait(acc_ready, 0, 1u << 22);
    if (!ok) report_error(p.err, ERR_EPILOGUE_WAIT);
    ptx::tc_fence_after();
    if (ok) {
      OutT* c_row = reinterpret_cast<OutT*>(p.C) + bz * p.c_batch_stride + (long long)row * p.ldc;
      const bool vec_ok = (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) && (p.c_batch_stride % 8 == 0);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        ptx::tmem_ld_32x32b_x32(tmem_base + (uint32_t(quarter * 32) << 16) + c0, r);
        ptx::tmem_ld_wait();
        if (row < p.M) {
          const int col0 = n0 + c0;
          if (vec_ok && col0 + 32 <= p.N) {
            if constexpr (sizeof(OutT) == 2) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * e]) * p.alpha,
                                                          __uint_as_float(r[v * 8 + 2 * e + 1]) * p.alpha);
                  w[e] = *reinterpret_cast<uint32_t*>(&h);
                }
                *reinterpret_cast<uint4*>(c_row + col0 + v * 8) = make_uint4(w[0], w[1], w[2], w[3]);
              }
            } else {
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                float4* dst = reinterpret_cast<float4*>(c_row + col0 + v * 4);
                float4 o = make_float4(__uint_as_float(r[v * 4]) * p.alpha, __uint_as_float(r[v * 4 + 1]) * p.alpha,
                                       __uint_as_float(r[v * 4 + 2]) * p.alpha, __uint_as_float(r[v * 4 + 3]) * p.alpha);
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
              if (col0 + e < p.N) {
                float v = __uint_as_float(r[e]) * p.alpha;
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
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) ptx::tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---- host side ---------------------------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q);
    TORCH_CHECK(e == cudaSuccess && q == cudaDriverEntryPointSuccess && ptr, "cuTensorMapEncodeTiled is unavailable");
    fn = reinterpret_cast<EncodeFn>(ptr);
  });
  return fn;
}

// 3-D tensor map {inner, rows, batch} with a 128-byte-swizzled {128 bytes, box_rows, 1} box; out-of-range elements read 0.
static CUtensorMap make_tmap(const void* base, int elem_bytes, int64_t inner, int64_t rows, int64_t batch, int64_t row_stride_elems,
                             int64_t batch_stride_elems, int box_rows, int box_inner_bytes = 128);

CUtensorMap make_tmap_bf16(const void* base, int64_t inner, int64_t rows, int64_t batch, int64_t row_stride_elems,
                           int64_t batch_stride_elems, int box_rows) {
  return make_tmap(base, 2, inner, rows, batch, row_stride_elems, batch_stride_elems, box_rows);
}

// Box of `box_rows` rows x `box_inner_bytes` (128 with the 128-byte swizzle, 64 with the 64-byte swizzle).
CUtensorMap make_tmap_box(const void* base, int elem_bytes, int64_t inner, int64_t rows, int64_t batch, int64_t row_stride_elems,
                          int64_t batch_stride_elems, int box_rows, int box_inner_bytes) {
  return make_tmap(base, elem_bytes, inner, rows, batch, row_stride_elems, batch_stride_elems, box_rows, box_inner_bytes);
}

static CUtensorMap make_tmap(const void* base, int elem_bytes, int64_t inner, int64_t rows, int64_t batch, int64_t row_stride_elems,
                             int64_t batch_stride_elems, int box_rows, int box_inner_bytes) {
  TORCH_CHECK(box_inner_bytes == 128 || box_inner_bytes == 64, "TMA box must be 64 or 128 bytes wide");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(base) & 15) == 0, "TMA base must be 16-byte aligned");
  TORCH_CHECK((row_stride_elems * elem_bytes) % 16 == 0 && (batch <= 1 || (batch_stride_elems * elem_bytes) % 16 == 0), "TMA strides must be multiples of 16 bytes");
  TORCH_CHECK(box_rows >= 1 && box_rows <= 256, "TMA box rows out of range");
  CUtensorMap m;
  cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)(batch < 1 ? 1 : batch)};
  cuuint64_t strides[2] = {(cuuint64_t)row_stride_elems * elem_bytes, (cuuint64_t)(batch <= 1 ? row_stride_elems * rows : batch_stride_elems) * elem_bytes};
  cuuint32_t box[3] = {(cuuint32_t)(box_inner_bytes / elem_bytes), (cuuint32_t)box_rows, 1};
  cuuint32_t elem[3] = {1, 1, 1};
  auto encode = [&] {
    return encode_fn()(&m, elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, elem,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, box_inner_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  CUresult r = encode();
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // A thread that has issued no runtime call yet (an autograd worker whose first op is this one) has no current context:
    // bind the device's primary context and encode again.
    int dev = 0;
    C10_CUDA_CHECK(cudaGetDevice(&dev));
    C10_CUDA_CHECK(cudaSetDevice(dev));
    C10_CUDA_CHECK(cudaFree(nullptr));
    r = encode();
  }
  if (r != CUDA_SUCCESS) {
    char msg[384];
    std::snprintf(msg, sizeof msg, "cuTensorMapEncodeTiled failed with code %d (base %p, dims %llu x %llu x %llu, strides %llu / %llu bytes, box %u x %u, map at %p)", (int)r, base,
                  (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)dims[2], (unsigned long long)strides[0], (unsigned long long)strides[1], box[0], box[1], (void*)&m);
    if (std::getenv("Q38_GEMM_TRACE")) { std::fprintf(stderr, "%s\n", msg); std::fflush(stderr); }
    TORCH_CHECK(false, msg);
  }
  return m;
}

template <int EB, int BN, bool A_MN, bool B_MN, typename OutT, bool ACCUM>
static void launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& p, cudaStream_t stream) {
  auto kernel = gemm_bf16_kernel<EB, BN, A_MN, B_MN, OutT, ACCUM>;
  constexpr int smem = gemm_smem_bytes<BN>();
  static bool configured = false;
  if (!configured) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  dim3 grid((p.N + BN - 1) / BN, (p.M + BM - 1) / BM, p.batch * p.splits);
  kernel<<<grid, GEMM_THREADS, smem, stream>>>(ta, tb, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

template <int EB, bool A_MN, bool B_MN>
static void dispatch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& p, bool out_fp32, bool accum, int bn,
                     cudaStream_t stream) {
  TORCH_CHECK(!accum || out_fp32, "accumulating epilogue requires an fp32 output");
  if constexpr (EB == 4) {
    TORCH_CHECK(out_fp32, "tf32 products write fp32");
    if (bn == 64) { if (accum) launch<EB, 64, A_MN, B_MN, float, true>(ta, tb, p, stream); else launch<EB, 64, A_MN, B_MN, float, false>(ta, tb, p, stream); }
    else { if (accum) launch<EB, 128, A_MN, B_MN, float, true>(ta, tb, p, stream); else launch<EB, 128, A_MN, B_MN, float, false>(ta, tb, p, stream); }
    return;
  }
  if (bn == 64) {
    if (!out_fp32) launch<EB, 64, A_MN, B_MN, __nv_bfloat16, false>(ta, tb, p, stream);
    else if (accum) launch<EB, 64, A_MN, B_MN, float, true>(ta, tb, p, stream);
    else launch<EB, 64, A_MN, B_MN, float, false>(ta, tb, p, stream);
  } else {
    if (!out_fp32) launch<EB, 128, A_MN, B_MN, __nv_bfloat16, false>(ta, tb, p, stream);
    else if (accum) launch<EB, 128, A_MN, B_MN, float, true>(ta, tb, p, stream);
    else launch<EB, 128, A_MN, B_MN, float, false>(ta, tb, p, stream);
  }
}

// a: K-major [batch, M, K] or MN-major [batch, K, M]; b likewise with N; c: [batch, M, N] bf16 or fp32 (last dim contiguous).
void gemm_bf16(const at::Tensor& a, const at::Tensor& b, at::Tensor& c, bool a_mn_major, bool b_mn_major, double alpha,
               bool accumulate, at::Tensor& err, int64_t splits) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && c.is_cuda(), "gemm_bf16: CUDA tensors required");
  const bool tf32 = a.scalar_type() == at::kFloat;
  TORCH_CHECK((a.scalar_type() == at::kBFloat16 || tf32) && b.scalar_type() == a.scalar_type(), "gemm_bf16: operands must both be bf16 or both fp32 (tf32 math)");
  TORCH_CHECK(a.dim() == 3 && b.dim() == 3 && c.dim() == 3, "gemm_bf16: [batch, rows, cols] tensors required");
  TORCH_CHECK(a.stride(2) == 1 && b.stride(2) == 1 && c.stride(2) == 1, "gemm_bf16: innermost dimension must be contiguous");
  const c10::cuda::CUDAGuard guard(a.device());
  const int batch = a.size(0);
  const int M = a_mn_major ? a.size(2) : a.size(1), K = a_mn_major ? a.size(1) : a.size(2);
  const int N = b_mn_major ? b.size(2) : b.size(1), Kb = b_mn_major ? b.size(1) : b.size(2);
  TORCH_CHECK(K == Kb && b.size(0) == batch && c.size(0) == batch && c.size(1) == M && c.size(2) == N, "gemm_bf16: shape mismatch");
  const bool out_fp32 = c.scalar_type() == at::kFloat;
  TORCH_CHECK(out_fp32 || c.scalar_type() == at::kBFloat16, "gemm_bf16: output must be bf16 or fp32");
  const int bn = (N <= 64) ? 64 : 128;
  const int eb = tf32 ? 4 : 2, bk = 128 / eb;
  TORCH_CHECK(!tf32 || out_fp32, "gemm_bf16: tf32 products write fp32");
  CUtensorMap ta = make_tmap(a.data_ptr(), eb, a.size(2), a.size(1), batch, a.stride(1), a.stride(0), a_mn_major ? bk : BM);
  CUtensorMap tb = make_tmap(b.data_ptr(), eb, b.size(2), b.size(1), batch, b.stride(1), b.stride(0), b_mn_major ? bk : bn);
  const int total_kb = (K + bk - 1) / bk;
  int nsplit = 1;
  if (accumulate && out_fp32) {
    if (splits > 0) nsplit = (int)splits;
    else if (splits == 0) {
      // automatic: enough CTAs for two per SM, at least eight K blocks per split
      const int tiles = ((N + bn - 1) / bn) * ((M + BM - 1) / BM) * batch;
      nsplit = std::max(1, std::min({(2 * kNumSMs + tiles - 1) / tiles, total_kb / 8, 32}));
    }
  }
  const int kb_per_split = (total_kb + nsplit - 1) / nsplit;
  nsplit = (total_kb + kb_per_split - 1) / kb_per_split;
  GemmArgs p{M, N, K, batch, nsplit, kb_per_split, c.data_ptr(), c.stride(1), c.stride(0), (float)alpha, err.data_ptr<int>()};
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  if (tf32) {
    TORCH_CHECK(!a_mn_major && !b_mn_major, "gemm_bf16: the tf32 path takes K-major operands only");
    dispatch<4, false, false>(ta, tb, p, true, accumulate, bn, stream);
  } else if (a_mn_major) {
    if (b_mn_major) dispatch<2, true, true>(ta, tb, p, out_fp32, accumulate, bn, stream);
    else dispatch<2, true, false>(ta, tb, p, out_fp32, accumulate, bn, stream);
  } else {
    if (b_mn_major) dispatch<2, false, true>(ta, tb, p, out_fp32, accumulate, bn, stream);
    else dispatch<2, false, false>(ta, tb, p, out_fp32, accumulate, bn, stream);
  }
}

}  // namespace q38
