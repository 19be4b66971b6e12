// Elementwise halves of the Muon step on flat arenas (the Newton-Schulz products in between run on the tensor-core GEMM).
//
// The matrices a rank owns are described once by two small device tables:
//   mats   [n_mat, 4] int64: {arena offset, offset in the bf16 work buffer, numel, 0}
//   tiles  [n_tile, 2] int32: {matrix index, first element of the tile inside the matrix}; a tile is MUON_TILE elements
//   scales [n_mat] fp32: 0.2 * sqrt(max(rows, cols)), the update-RMS alignment of each matrix
//
//   muon_prepass    buf <- momentum * buf + g * clip;  u <- g * clip + momentum * buf;  work <- bf16(u);
//                   sumsq[matrix] += bf16(u)^2           (one pass over gradient and momentum buffer)
//   muon_normalize  work <- bf16(work / max(bf16(sqrt(sumsq[matrix])), eps))   and clears sumsq for the next step
//   muon_apply      W <- W * (1 - lr * wd) - lr * scale[matrix] * work;  shadow <- bf16(W)
//
// The work buffer keeps every matrix in the layout of its parameter (no transposes: for tall matrices the Newton-Schulz
// chain runs on the transposed problem through the GEMM's MN-major operand modes), and groups matrices of one shape
// contiguously so that one batched GEMM call covers all of them.  Arithmetic follows the reference's Muon
// (q38/muon.py:12-25, 93-104): the update is cast to bf16 before its Frobenius norm is taken, the norm is rounded to bf16
// and the division result is rounded to bf16 again.
// lr comes from device memory (hyper[0]) so a captured launch can be replayed with a new value.  All three kernels return
// without writing when the error word is set (a peer missed a barrier): parameters and optimizer state stay untouched.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"
#include "host.h"

namespace q38 {

constexpr int MUON_TILE = 4096, MUON_THREADS = 256;

__device__ __forceinline__ bool muon_aborted(const int* err) {
  if (err == nullptr) return false;
  int v;
  asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(err) : "memory");
  return v != 0;
}

__global__ void __launch_bounds__(MUON_THREADS) muon_prepass_kernel(const float* __restrict__ grads, float* __restrict__ buf, __nv_bfloat16* __restrict__ work,
                                                                    float* __restrict__ sumsq, const long long* __restrict__ mats, const int* __restrict__ tiles,
                                                                    const float* __restrict__ grad_scale, float momentum, const int* __restrict__ err) {
  if (muon_aborted(err)) return;
  __shared__ float scratch[32];
  const int m = tiles[2 * blockIdx.x], first = tiles[2 * blockIdx.x + 1];
  const long long off = mats[4 * m], woff = mats[4 * m + 1], numel = mats[4 * m + 2];
  const float gs = grad_scale ? *grad_scale : 1.f;
  const int count = (int)min((long long)MUON_TILE, numel - first);
  const float* g = grads + off + first;
  float* b = buf + off + first;
  __nv_bfloat16* w = work + woff + first;
  float acc = 0.f;
  // 16-byte accesses when this tile starts on a 4-element boundary in both buffers (arena units are 64-element aligned and tiles
  // are 4096 long, so only stacks of matrices whose size is not a multiple of 4 take the scalar path)
  const bool vec = (((off + first) | (woff + first)) & 3) == 0;
  const int n4 = vec ? (count >> 2) : 0;
  for (int i = threadIdx.x; i < n4; i += MUON_THREADS) {
    float4 gv = reinterpret_cast<const float4*>(g)[i];
    float4 bv = reinterpret_cast<float4*>(b)[i];
    gv.x *= gs; gv.y *= gs; gv.z *= gs; gv.w *= gs;
    bv.x = momentum * bv.x + gv.x; bv.y = momentum * bv.y + gv.y; bv.z = momentum * bv.z + gv.z; bv.w = momentum * bv.w + gv.w;
    reinterpret_cast<float4*>(b)[i] = bv;
    const __nv_bfloat162 lo = __floats2bfloat162_rn(gv.x + momentum * bv.x, gv.y + momentum * bv.y);
    const __nv_bfloat162 hi = __floats2bfloat162_rn(gv.z + momentum * bv.z, gv.w + momentum * bv.w);
    uint2 packed;
    packed.x = *reinterpret_cast<const uint32_t*>(&lo); packed.y = *reinterpret_cast<const uint32_t*>(&hi);
    reinterpret_cast<uint2*>(w)[i] = packed;
    const float2 l = __bfloat1622float2(lo), h = __bfloat1622float2(hi);
    acc += l.x * l.x + l.y * l.y + h.x * h.x + h.y * h.y;
  }
  for (int i = (n4 << 2) + threadIdx.x; i < count; i += MUON_THREADS) {
    const float gi = g[i] * gs;
    const float bi = momentum * b[i] + gi;
    b[i] = bi;
    const __nv_bfloat16 u = __float2bfloat16_rn(gi + momentum * bi);
    w[i] = u;
    const float uf = __bfloat162float(u);
    acc += uf * uf;
  }
  acc = block_sum(acc, scratch);
  if (threadIdx.x == 0) atomicAdd(sumsq + m, acc);
}

__global__ void __launch_bounds__(MUON_THREADS) muon_normalize_kernel(__nv_bfloat16* __restrict__ work, const float* __restrict__ sumsq,
                                                                      const long long* __restrict__ mats, const int* __restrict__ tiles, float eps,
                                                                      const int* __restrict__ err) {
  if (muon_aborted(err)) return;
  const int m = tiles[2 * blockIdx.x], first = tiles[2 * blockIdx.x + 1];
  const long long woff = mats[4 * m + 1], numel = mats[4 * m + 2];
  const int count = (int)min((long long)MUON_TILE, numel - first);
  const float norm = fmaxf(bf16_round(sqrtf(sumsq[m])), eps);
  __nv_bfloat16* w = work + woff + first;
  for (int i = threadIdx.x; i < count; i += MUON_THREADS) w[i] = __float2bfloat16_rn(__bfloat162float(w[i]) / norm);
}

__global__ void muon_clear_kernel(float* __restrict__ sumsq, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) sumsq[i] = 0.f;
}

__global__ void __launch_bounds__(MUON_THREADS) muon_apply_kernel(float* __restrict__ params, __nv_bfloat16* __restrict__ shadow, const __nv_bfloat16* __restrict__ work,
                                                                  const long long* __restrict__ mats, const int* __restrict__ tiles, const float* __restrict__ scales,
                                                                  const float* __restrict__ hyper, float lr, float wd, const int* __restrict__ err) {
  if (muon_aborted(err)) return;
  const int m = tiles[2 * blockIdx.x], first = tiles[2 * blockIdx.x + 1];
  const long long off = mats[4 * m], woff = mats[4 * m + 1], numel = mats[4 * m + 2];
  const int count = (int)min((long long)MUON_TILE, numel - first);
  if (hyper) lr = hyper[0];
  const float decay = 1.f - lr * wd, step = lr * scales[m];
  float* p = params + off + first;
  const __nv_bfloat16* x = work + woff + first;
  __nv_bfloat16* s = shadow ? shadow + off + first : nullptr;
  const bool vec = (((off + first) | (woff + first)) & 3) == 0;
  const int n4 = vec ? (count >> 2) : 0;
  for (int i = threadIdx.x; i < n4; i += MUON_THREADS) {
    float4 v = reinterpret_cast<float4*>(p)[i];
    const uint2 raw = reinterpret_cast<const uint2*>(x)[i];
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x)), hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    v.x = v.x * decay - step * lo.x; v.y = v.y * decay - step * lo.y; v.z = v.z * decay - step * hi.x; v.w = v.w * decay - step * hi.y;
    reinterpret_cast<float4*>(p)[i] = v;
    if (s) {
      const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
      uint2 packed;
      packed.x = *reinterpret_cast<const uint32_t*>(&a); packed.y = *reinterpret_cast<const uint32_t*>(&b);
      reinterpret_cast<uint2*>(s)[i] = packed;
    }
  }
  for (int i = (n4 << 2) + threadIdx.x; i < count; i += MUON_THREADS) {
    const float v = p[i] * decay - step * __bfloat162float(x[i]);
    p[i] = v;
    if (s) s[i] = __float2bfloat16_rn(v);
  }
}

// Newton-Schulz for stacks of tiny matrices (min(rows, cols) <= 8, e.g. the depthwise conv taps 1 x 4 and 4-row projections),
// one CTA per matrix, everything in shared memory.  Same rounding points as the tensor-core chain: G, b G + c G G and
// a X + P X are each rounded to bf16 once.  `src`/`dst`: [n, rows, cols] bf16, already normalised.
constexpr int SMALL_M = 8, SMALL_K = 2048;
__global__ void __launch_bounds__(128) muon_small_ns_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst, int rows, int cols, int steps,
                                                            float a, float b, float c, const int* __restrict__ err) {
  if (muon_aborted(err)) return;
  extern __shared__ float sm[];
  const bool tall = rows > cols;
  const int m = tall ? cols : rows, k = tall ? rows : cols;
  float* X = sm;                         // [m][k]
  float* G = X + m * k;                  // [m][m]
  float* P = G + m * m;                  // [m][m]
  const long long base = (long long)blockIdx.x * rows * cols;
  for (int i = threadIdx.x; i < m * k; i += blockDim.x) {
    const int r = i / k, l = i % k;
    X[i] = __bfloat162float(src[base + (tall ? (long long)l * cols + r : (long long)r * cols + l)]);
  }
  __syncthreads();
  for (int it = 0; it < steps; ++it) {
    for (int e = threadIdx.x; e < m * m; e += blockDim.x) {
      const int i = e / m, j = e % m;
      float acc = 0.f;
      for (int l = 0; l < k; ++l) acc += X[i * k + l] * X[j * k + l];
      G[e] = bf16_round(acc);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < m * m; e += blockDim.x) {
      const int i = e / m, j = e % m;
      float acc = 0.f;
      for (int l = 0; l < m; ++l) acc += G[i * m + l] * G[l * m + j];
      P[e] = bf16_round(c * acc + b * G[e]);
    }
    __syncthreads();
    // X <- a X + P X; every thread owns whole columns, so the update of a column only reads that column
    for (int l = threadIdx.x; l < k; l += blockDim.x) {
      float col[SMALL_M];
      for (int i = 0; i < m; ++i) col[i] = X[i * k + l];
      for (int i = 0; i < m; ++i) {
        float acc = 0.f;
        for (int j = 0; j < m; ++j) acc += P[i * m + j] * col[j];
        X[i * k + l] = bf16_round(acc + a * col[i]);
      }
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < m * k; i += blockDim.x) {
    const int r = i / k, l = i % k;
    dst[base + (tall ? (long long)l * cols + r : (long long)r * cols + l)] = __float2bfloat16_rn(X[i]);
  }
}

static const int* err_ptr(const c10::optional<at::Tensor>& err) { return err.has_value() ? err->data_ptr<int>() : nullptr; }

void muon_prepass(const at::Tensor& grads, at::Tensor& buf, at::Tensor& work, at::Tensor& sumsq, const at::Tensor& mats, const at::Tensor& tiles,
                  const c10::optional<at::Tensor>& grad_scale, double momentum, const c10::optional<at::Tensor>& err) {
  TORCH_CHECK(grads.is_cuda() && grads.scalar_type() == at::kFloat && buf.scalar_type() == at::kFloat && work.scalar_type() == at::kBFloat16 &&
              sumsq.scalar_type() == at::kFloat && mats.scalar_type() == at::kLong && tiles.scalar_type() == at::kInt, "muon_prepass: dtype mismatch");
  const c10::cuda::CUDAGuard guard(grads.device());
  const int n_tiles = (int)tiles.size(0);
  if (!n_tiles) return;
  muon_prepass_kernel<<<n_tiles, MUON_THREADS, 0, at::cuda::getCurrentCUDAStream()>>>(
      grads.data_ptr<float>(), buf.data_ptr<float>(), (__nv_bfloat16*)work.data_ptr(), sumsq.data_ptr<float>(), (const long long*)mats.data_ptr<int64_t>(),
      tiles.data_ptr<int>(), grad_scale.has_value() ? grad_scale->data_ptr<float>() : nullptr, (float)momentum, err_ptr(err));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

void muon_normalize(at::Tensor& work, at::Tensor& sumsq, const at::Tensor& mats, const at::Tensor& tiles, double eps, const c10::optional<at::Tensor>& err) {
  const c10::cuda::CUDAGuard guard(work.device());
  const int n_tiles = (int)tiles.size(0);
  if (!n_tiles) return;
  auto stream = at::cuda::getCurrentCUDAStream();
  muon_normalize_kernel<<<n_tiles, MUON_THREADS, 0, stream>>>((__nv_bfloat16*)work.data_ptr(), sumsq.data_ptr<float>(), (const long long*)mats.data_ptr<int64_t>(),
                                                             tiles.data_ptr<int>(), (float)eps, err_ptr(err));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  const int n = (int)sumsq.numel();
  muon_clear_kernel<<<(n + 255) / 256, 256, 0, stream>>>(sumsq.data_ptr<float>(), n);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch(2);
}

void muon_apply(at::Tensor& params, const c10::optional<at::Tensor>& shadow, const at::Tensor& work, const at::Tensor& mats, const at::Tensor& tiles,
                const at::Tensor& scales, const c10::optional<at::Tensor>& hyper, double lr, double wd, const c10::optional<at::Tensor>& err) {
  TORCH_CHECK(params.is_cuda() && params.scalar_type() == at::kFloat && work.scalar_type() == at::kBFloat16 && scales.scalar_type() == at::kFloat,
              "muon_apply: dtype mismatch");
  const c10::cuda::CUDAGuard guard(params.device());
  const int n_tiles = (int)tiles.size(0);
  if (!n_tiles) return;
  muon_apply_kernel<<<n_tiles, MUON_THREADS, 0, at::cuda::getCurrentCUDAStream()>>>(
      params.data_ptr<float>(), shadow.has_value() ? (__nv_bfloat16*)shadow->data_ptr() : nullptr, (const __nv_bfloat16*)work.data_ptr(),
      (const long long*)mats.data_ptr<int64_t>(), tiles.data_ptr<int>(), scales.data_ptr<float>(), hyper.has_value() ? hyper->data_ptr<float>() : nullptr, (float)lr,
      (float)wd, err_ptr(err));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

void muon_small_ns(const at::Tensor& src, at::Tensor& dst, int64_t rows, int64_t cols, int64_t steps, const c10::optional<at::Tensor>& err) {
  TORCH_CHECK(src.is_cuda() && src.scalar_type() == at::kBFloat16 && dst.scalar_type() == at::kBFloat16 && src.is_contiguous() && dst.is_contiguous() &&
              src.numel() == dst.numel() && src.numel() % (rows * cols) == 0, "muon_small_ns: contiguous bf16 [n, rows, cols] stacks required");
  const int m = (int)std::min(rows, cols), k = (int)std::max(rows, cols);
  TORCH_CHECK(m <= SMALL_M && k <= SMALL_K, "muon_small_ns: min(rows, cols) <= 8 and max(rows, cols) <= 2048 required");
  const c10::cuda::CUDAGuard guard(src.device());
  const int n = (int)(src.numel() / (rows * cols));
  if (!n) return;
  const int smem = (m * k + 2 * m * m) * (int)sizeof(float);
  static bool configured = false;
  if (!configured) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(muon_small_ns_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (SMALL_M * SMALL_K + 2 * SMALL_M * SMALL_M) * 4));
    configured = true;
  }
  muon_small_ns_kernel<<<n, 128, smem, at::cuda::getCurrentCUDAStream()>>>((const __nv_bfloat16*)src.data_ptr(), (__nv_bfloat16*)dst.data_ptr(), (int)rows, (int)cols,
                                                                          (int)steps, 3.4445f, -4.7750f, 2.0315f, err_ptr(err));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

}  // namespace q38
