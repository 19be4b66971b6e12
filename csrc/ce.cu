// Cross-entropy over bf16 logits, one CTA per row, in place: the row is read once into registers, the loss
// (log-sum-exp minus the target logit) is written to `loss[row]`, and the row is overwritten with its own gradient
// softmax(logits) - onehot(target) (zeros for ignored rows, target == -100).  The vocabulary projection before it and
// the two gradient GEMMs after it run on the tcgen05 GEMM; fp32 logits are never materialised.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"
#include "host.h"

namespace q38 {

constexpr int CE_THREADS = 256, CE_MAX_PER_THREAD = 64;          // rows up to 16384 * 2 elements... see host check

__global__ void __launch_bounds__(CE_THREADS) ce_inplace_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ target,
                                                                float* __restrict__ loss, int V, long long ld) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(logits + row * ld);
  const long long tgt = target[row];
  const int pairs = V / 2;
  float2 vals[CE_MAX_PER_THREAD / 2];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < CE_MAX_PER_THREAD / 2; ++i) {
    const int idx = threadIdx.x + i * CE_THREADS;
    if (idx < pairs) {
      const __nv_bfloat162 v = p[idx];
      vals[i] = make_float2(__low2float(v), __high2float(v));
      m = fmaxf(m, fmaxf(vals[i].x, vals[i].y));
    }
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = m;
  __syncthreads();
  m = scratch[0];
#pragma unroll
  for (int w = 1; w < CE_THREADS / 32; ++w) m = fmaxf(m, scratch[w]);
  float s = 0.f, tl = 0.f;
#pragma unroll
  for (int i = 0; i < CE_MAX_PER_THREAD / 2; ++i) {
    const int idx = threadIdx.x + i * CE_THREADS;
    if (idx < pairs) {
      if (2 * idx == tgt) tl = vals[i].x;
      if (2 * idx + 1 == tgt) tl = vals[i].y;
      vals[i].x = __expf(vals[i].x - m); vals[i].y = __expf(vals[i].y - m);
      s += vals[i].x + vals[i].y;
    }
  }
  s = block_sum(s, scratch);
  tl = block_sum(tl, scratch);
  const bool ignored = tgt < 0;
  if (threadIdx.x == 0) loss[row] = ignored ? 0.f : (m + __logf(s) - tl);
  const float inv = ignored ? 0.f : 1.f / s;
#pragma unroll
  for (int i = 0; i < CE_MAX_PER_THREAD / 2; ++i) {
    const int idx = threadIdx.x + i * CE_THREADS;
    if (idx < pairs) {
      float a = vals[i].x * inv, b = vals[i].y * inv;
      if (2 * idx == tgt) a -= 1.f;
      if (2 * idx + 1 == tgt) b -= 1.f;
      p[idx] = __floats2bfloat162_rn(a, b);
    }
  }
}

// The same row-in-registers scheme with 16-byte accesses: thread t holds the 8-element groups t, t + 256, ... (NV of them).  Fewer
// and wider memory instructions and fewer registers than the 4-byte version, so more rows are resident per SM while one row is
// between its load and its store phase.  Needs V % 8 == 0 and a 16-byte aligned buffer.
template <int NV>
__global__ void __launch_bounds__(CE_THREADS) ce_inplace_vec_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ target,
                                                                    float* __restrict__ loss, int V, long long ld) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  uint4* p = reinterpret_cast<uint4*>(logits + row * ld);
  const int tgt = (int)target[row];
  const int groups = V / 8;
  float vals[NV][8];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int idx = threadIdx.x + i * CE_THREADS;
    if (idx < groups) {
      const uint4 raw = p[idx];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        vals[i][2 * e] = __low2float(h[e]); vals[i][2 * e + 1] = __high2float(h[e]);
        m = fmaxf(m, fmaxf(vals[i][2 * e], vals[i][2 * e + 1]));
      }
    }
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = m;
  __syncthreads();
  m = scratch[0];
#pragma unroll
  for (int w = 1; w < CE_THREADS / 32; ++w) m = fmaxf(m, scratch[w]);
  float s = 0.f, tl = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int idx = threadIdx.x + i * CE_THREADS;
    if (idx < groups) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (8 * idx + e == tgt) tl = vals[i][e];
        vals[i][e] = __expf(vals[i][e] - m);
        s += vals[i][e];
      }
    }
  }
  __syncthreads();                                   // every thread has read the maxima before the sums reuse the scratch
  s = block_sum(s, scratch);
  tl = block_sum(tl, scratch);
  const bool ignored = tgt < 0;
  if (threadIdx.x == 0) loss[row] = ignored ? 0.f : (m + __logf(s) - tl);
  const float inv = ignored ? 0.f : 1.f / s;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int idx = threadIdx.x + i * CE_THREADS;
    if (idx < groups) {
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float a = vals[i][2 * e] * inv, b = vals[i][2 * e + 1] * inv;
        if (8 * idx + 2 * e == tgt) a -= 1.f;
        if (8 * idx + 2 * e + 1 == tgt) b -= 1.f;
        const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        w[e] = *reinterpret_cast<const uint32_t*>(&h);
      }
      p[idx] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

template <int NV>
static void launch_ce_vec(at::Tensor& logits, const at::Tensor& target, at::Tensor& loss, int V) {
  ce_inplace_vec_kernel<NV><<<(unsigned)logits.size(0), CE_THREADS, 0, at::cuda::getCurrentCUDAStream()>>>(
      (__nv_bfloat16*)logits.data_ptr(), reinterpret_cast<const long long*>(target.data_ptr<int64_t>()), loss.data_ptr<float>(), V, V);
}

// logits [R, V] bf16 (row stride = V), target [R] int64 -> loss [R] fp32; logits become d(loss_row)/d(logits).
at::Tensor ce_inplace(at::Tensor& logits, const at::Tensor& target) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kBFloat16 && logits.dim() == 2 && logits.is_contiguous(), "ce_inplace: contiguous bf16 [R,V] logits required");
  TORCH_CHECK(target.scalar_type() == at::kLong && target.is_contiguous() && target.numel() == logits.size(0), "ce_inplace: int64 targets required");
  const int V = logits.size(1);
  TORCH_CHECK(V % 2 == 0 && V <= CE_THREADS * CE_MAX_PER_THREAD, "ce_inplace: vocabulary must be even and at most 16384");
  const c10::cuda::CUDAGuard guard(logits.device());
  auto loss = at::empty({logits.size(0)}, logits.options().dtype(at::kFloat));
  const int nv = (V / 8 + CE_THREADS - 1) / CE_THREADS;
  if (logits.size(0) && V % 8 == 0 && (reinterpret_cast<uintptr_t>(logits.data_ptr()) & 15) == 0) {
    switch (nv) {
      case 1: launch_ce_vec<1>(logits, target, loss, V); break;
      case 2: launch_ce_vec<2>(logits, target, loss, V); break;
      case 3: launch_ce_vec<3>(logits, target, loss, V); break;
      case 4: launch_ce_vec<4>(logits, target, loss, V); break;
      case 5: launch_ce_vec<5>(logits, target, loss, V); break;
      case 6: launch_ce_vec<6>(logits, target, loss, V); break;
      case 7: launch_ce_vec<7>(logits, target, loss, V); break;
      default: launch_ce_vec<8>(logits, target, loss, V); break;
    }
  } else if (logits.size(0))
    ce_inplace_kernel<<<(unsigned)logits.size(0), CE_THREADS, 0, at::cuda::getCurrentCUDAStream()>>>((__nv_bfloat16*)logits.data_ptr(), reinterpret_cast<const long long*>(target.data_ptr<int64_t>()),
                                                                                                    loss.data_ptr<float>(), V, V);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return loss;
}

}  // namespace q38
