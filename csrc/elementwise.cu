// Memory-bound kernels: RMSNorm variants (forward/backward), flat AdamW, sum of squares.
// One warp handles one row where rows are short (<= 1024 elements per lane-strided pass); all math in fp32.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"
#include "host.h"

namespace q38 {

constexpr int ROWS_PER_CTA = 8;   // 8 warps, one row each

// ---- zero-centred RMSNorm: y = x * rsqrt(mean(x^2) + eps) * (1 + w) ----------------------------------------------
template <typename InT, typename OutT>
__global__ void __launch_bounds__(32 * ROWS_PER_CTA) rmsnorm_fwd_kernel(const InT* __restrict__ x, const float* __restrict__ w,
                                                                        OutT* __restrict__ y, float* __restrict__ rstd,
                                                                        int rows, int dim, float eps) {
  const int row = blockIdx.x * ROWS_PER_CTA + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const InT* xr = x + (size_t)row * dim;
  float ss = 0.f;
  for (int i = lane; i < dim; i += 32) { float v = to_float(xr[i]); ss += v * v; }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / dim + eps);
  if (lane == 0) rstd[row] = r;
  OutT* yr = y + (size_t)row * dim;
  for (int i = lane; i < dim; i += 32) yr[i] = from_float<OutT>(to_float(xr[i]) * r * (1.f + w[i]));
}

// dx = r * (g - xhat * mean(g * xhat)),  g = dy * (1 + w);  dw += dy * xhat (summed over rows)
template <typename InT, typename GradT>
__global__ void __launch_bounds__(32 * ROWS_PER_CTA) rmsnorm_bwd_kernel(const GradT* __restrict__ dy, const InT* __restrict__ x,
                                                                        const float* __restrict__ w, const float* __restrict__ rstd,
                                                                        InT* __restrict__ dx, float* __restrict__ dw_partial,
                                                                        int rows, int dim) {
  extern __shared__ float dw_acc[];            // [dim], accumulated over this CTA's rows
  for (int i = threadIdx.x; i < dim; i += blockDim.x) dw_acc[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int row = blockIdx.x * ROWS_PER_CTA + warp; row < rows; row += gridDim.x * ROWS_PER_CTA) {
    const InT* xr = x + (size_t)row * dim;
    const GradT* gr = dy + (size_t)row * dim;
    const float r = rstd[row];
    float dot = 0.f;
    for (int i = lane; i < dim; i += 32) dot += to_float(gr[i]) * (1.f + w[i]) * to_float(xr[i]) * r;
    dot = warp_sum(dot) / dim;
    InT* dxr = dx + (size_t)row * dim;
    for (int i = lane; i < dim; i += 32) {
      const float xhat = to_float(xr[i]) * r, g = to_float(gr[i]);
      dxr[i] = from_float<InT>(r * (g * (1.f + w[i]) - xhat * dot));
      atomicAdd(&dw_acc[i], g * xhat);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < dim; i += blockDim.x) atomicAdd(&dw_partial[i], dw_acc[i]);
}

std::vector<at::Tensor> rmsnorm_fwd(const at::Tensor& x, const at::Tensor& w, double eps, bool out_bf16) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && w.scalar_type() == at::kFloat && w.is_contiguous(), "rmsnorm_fwd: bad inputs");
  const c10::cuda::CUDAGuard guard(x.device());
  const int dim = x.size(-1);
  const int rows = x.numel() / dim;
  auto y = at::empty(x.sizes(), x.options().dtype(out_bf16 ? at::kBFloat16 : at::kFloat));
  auto rstd = at::empty({rows}, x.options().dtype(at::kFloat));
  if (rows == 0) return {y, rstd};
  const int grid = (rows + ROWS_PER_CTA - 1) / ROWS_PER_CTA;
  auto stream = at::cuda::getCurrentCUDAStream();
#define LAUNCH(InT, OutT) rmsnorm_fwd_kernel<InT, OutT><<<grid, 32 * ROWS_PER_CTA, 0, stream>>>( \
      (const InT*)x.data_ptr(), w.data_ptr<float>(), (OutT*)y.data_ptr(), rstd.data_ptr<float>(), rows, dim, (float)eps)
  if (x.scalar_type() == at::kFloat) { if (out_bf16) LAUNCH(float, __nv_bfloat16); else LAUNCH(float, float); }
  else if (x.scalar_type() == at::kBFloat16) { if (out_bf16) LAUNCH(__nv_bfloat16, __nv_bfloat16); else LAUNCH(__nv_bfloat16, float); }
  else TORCH_CHECK(false, "rmsnorm_fwd: fp32 or bf16 input required");
#undef LAUNCH
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {y, rstd};
}

std::vector<at::Tensor> rmsnorm_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& w, const at::Tensor& rstd) {
  TORCH_CHECK(dy.is_cuda() && dy.is_contiguous() && x.is_contiguous(), "rmsnorm_bwd: bad inputs");
  const c10::cuda::CUDAGuard guard(x.device());
  const int dim = x.size(-1);
  const int rows = x.numel() / dim;
  auto dx = at::empty_like(x);
  auto dw = at::zeros({dim}, x.options().dtype(at::kFloat));
  if (rows == 0) return {dx, dw};
  const int grid = std::min((rows + ROWS_PER_CTA - 1) / ROWS_PER_CTA, kNumSMs * 4);
  auto stream = at::cuda::getCurrentCUDAStream();
  const size_t smem = dim * sizeof(float);
#define LAUNCH(InT, GradT) rmsnorm_bwd_kernel<InT, GradT><<<grid, 32 * ROWS_PER_CTA, smem, stream>>>( \
      (const GradT*)dy.data_ptr(), (const InT*)x.data_ptr(), w.data_ptr<float>(), rstd.data_ptr<float>(), (InT*)dx.data_ptr(), \
      dw.data_ptr<float>(), rows, dim)
  const bool xf = x.scalar_type() == at::kFloat, gf = dy.scalar_type() == at::kFloat;
  if (xf && gf) LAUNCH(float, float); else if (xf) LAUNCH(float, __nv_bfloat16);
  else if (gf) LAUNCH(__nv_bfloat16, float); else LAUNCH(__nv_bfloat16, __nv_bfloat16);
#undef LAUNCH
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {dx, dw};
}

// ---- gated RMSNorm over one 64-wide head: y = bf16( w * bf16(xhat) * silu(gate) ) ------------------------------------
// Eight lanes per row, eight elements (16 bytes) per lane, so a warp moves four rows per access (dim is fixed at 64 by the
// model's linear_value_head_dim).  Row reductions are three xor-shuffles inside the 8-lane group.
__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) { v[2 * i] = __low2float(h[i]); v[2 * i + 1] = __high2float(h[i]); }
}
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  uint4 out;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  return out;
}
__device__ __forceinline__ float group8_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  return v;
}

__global__ void __launch_bounds__(256) gated_rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gate,
                                                                 const float* __restrict__ w, __nv_bfloat16* __restrict__ y, int rows, float eps) {
  const int sub = threadIdx.x & 7;
  const long long row = ((long long)blockIdx.x * 256 + threadIdx.x) >> 3;
  const bool live = row < rows;
  float xv[8], gv[8], wv[8];
  if (live) {
    unpack8(reinterpret_cast<const uint4*>(x + row * 64)[sub], xv);
    unpack8(reinterpret_cast<const uint4*>(gate + row * 64)[sub], gv);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) xv[i] = gv[i] = 0.f;
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) wv[i] = w[8 * sub + i];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) ss += xv[i] * xv[i];
  const float r = rsqrtf(group8_sum(ss) / 64.f + eps);
  float out[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) out[i] = wv[i] * bf16_round(xv[i] * r) * siluf_(gv[i]);
  if (live) reinterpret_cast<uint4*>(y + row * 64)[sub] = pack8(out);
}

__global__ void __launch_bounds__(256) gated_rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                                 const __nv_bfloat16* __restrict__ gate, const float* __restrict__ w,
                                                                 __nv_bfloat16* __restrict__ dx, __nv_bfloat16* __restrict__ dgate,
                                                                 float* __restrict__ dw, int rows, float eps) {
  __shared__ float dw_acc[64];
  if (threadIdx.x < 64) dw_acc[threadIdx.x] = 0.f;
  __syncthreads();
  const int sub = threadIdx.x & 7;
  float wv[8], dwv[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { wv[i] = w[8 * sub + i]; dwv[i] = 0.f; }
  const long long stride = ((long long)gridDim.x * 256) >> 3;
  const long long first = ((long long)blockIdx.x * 256 + threadIdx.x) >> 3;
  // every 8-lane group walks rows first, first + stride, ...; the loop bound is uniform per warp up to the last iteration,
  // where finished groups keep shuffling on zeros
  for (long long base = first - (threadIdx.x >> 3 & 3); base < rows; base += stride) {
    const long long row = base + (threadIdx.x >> 3 & 3);
    const bool live = row < rows;
    float xv[8], gv[8], dv[8];
    if (live) {
      unpack8(reinterpret_cast<const uint4*>(x + row * 64)[sub], xv);
      unpack8(reinterpret_cast<const uint4*>(gate + row * 64)[sub], gv);
      unpack8(reinterpret_cast<const uint4*>(dy + row * 64)[sub], dv);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) xv[i] = gv[i] = dv[i] = 0.f;
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += xv[i] * xv[i];
    const float r = rsqrtf(group8_sum(ss) / 64.f + eps);
    float hv[8], sv[8], dh[8], dot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      hv[i] = xv[i] * r;
      sv[i] = sigmoidf_(gv[i]);
      dwv[i] += dv[i] * hv[i] * gv[i] * sv[i];                 // y = w * xhat * g * s
      dh[i] = dv[i] * wv[i] * gv[i] * sv[i];
      dot += dh[i] * hv[i];
    }
    dot = group8_sum(dot) / 64.f;
    float ox[8], og[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      ox[i] = r * (dh[i] - hv[i] * dot);
      og[i] = dv[i] * wv[i] * hv[i] * sv[i] * (1.f + gv[i] * (1.f - sv[i]));   // d silu(g) = s (1 + g (1 - s))
    }
    if (live) {
      reinterpret_cast<uint4*>(dx + row * 64)[sub] = pack8(ox);
      reinterpret_cast<uint4*>(dgate + row * 64)[sub] = pack8(og);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) atomicAdd(&dw_acc[8 * sub + i], dwv[i]);
  __syncthreads();
  if (threadIdx.x < 64) atomicAdd(&dw[threadIdx.x], dw_acc[threadIdx.x]);
}

// ---- SwiGLU: y = bf16(silu(g)) * u, elementwise on bf16 (eight elements per thread) --------------------------------------
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u,
                                                          __nv_bfloat16* __restrict__ y, long long n8) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= n8) return;
  float gv[8], uv[8], o[8];
  unpack8(reinterpret_cast<const uint4*>(g)[i], gv);
  unpack8(reinterpret_cast<const uint4*>(u)[i], uv);
#pragma unroll
  for (int k = 0; k < 8; ++k) o[k] = bf16_round(siluf_(gv[k])) * uv[k];
  reinterpret_cast<uint4*>(y)[i] = pack8(o);
}

__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ g,
                                                          const __nv_bfloat16* __restrict__ u, __nv_bfloat16* __restrict__ dg,
                                                          __nv_bfloat16* __restrict__ du, long long n8) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= n8) return;
  float dv[8], gv[8], uv[8], og[8], ou[8];
  unpack8(reinterpret_cast<const uint4*>(dy)[i], dv);
  unpack8(reinterpret_cast<const uint4*>(g)[i], gv);
  unpack8(reinterpret_cast<const uint4*>(u)[i], uv);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float s = sigmoidf_(gv[k]);
    ou[k] = dv[k] * gv[k] * s;
    og[k] = dv[k] * uv[k] * s * (1.f + gv[k] * (1.f - s));
  }
  reinterpret_cast<uint4*>(dg)[i] = pack8(og);
  reinterpret_cast<uint4*>(du)[i] = pack8(ou);
}

at::Tensor swiglu_fwd(const at::Tensor& g, const at::Tensor& u) {
  TORCH_CHECK(g.is_cuda() && g.scalar_type() == at::kBFloat16 && u.scalar_type() == at::kBFloat16 && g.is_contiguous() && u.is_contiguous() &&
                  g.sizes() == u.sizes() && g.numel() % 8 == 0, "swiglu_fwd: contiguous bf16 tensors of equal shape (a multiple of 8 elements) required");
  const c10::cuda::CUDAGuard guard(g.device());
  auto y = at::empty_like(g);
  const long long n8 = g.numel() / 8;
  if (n8) swiglu_fwd_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      (const __nv_bfloat16*)g.data_ptr(), (const __nv_bfloat16*)u.data_ptr(), (__nv_bfloat16*)y.data_ptr(), n8);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return y;
}

std::vector<at::Tensor> swiglu_bwd(const at::Tensor& dy, const at::Tensor& g, const at::Tensor& u) {
  TORCH_CHECK(dy.is_cuda() && dy.scalar_type() == at::kBFloat16 && dy.is_contiguous() && dy.sizes() == g.sizes(), "swiglu_bwd: bad gradient");
  const c10::cuda::CUDAGuard guard(g.device());
  auto dg = at::empty_like(g), du = at::empty_like(u);
  const long long n8 = g.numel() / 8;
  if (n8) swiglu_bwd_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      (const __nv_bfloat16*)dy.data_ptr(), (const __nv_bfloat16*)g.data_ptr(), (const __nv_bfloat16*)u.data_ptr(), (__nv_bfloat16*)dg.data_ptr(),
      (__nv_bfloat16*)du.data_ptr(), n8);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {dg, du};
}

// ---- output gate of the attention layer: y = x * bf16(sigmoid(g)), elementwise on bf16 (eight elements per thread) -------
__global__ void __launch_bounds__(256) sigmoid_mul_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ g,
                                                               __nv_bfloat16* __restrict__ y, long long n8) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= n8) return;
  float xv[8], gv[8], o[8];
  unpack8(reinterpret_cast<const uint4*>(x)[i], xv);
  unpack8(reinterpret_cast<const uint4*>(g)[i], gv);
#pragma unroll
  for (int k = 0; k < 8; ++k) o[k] = xv[k] * bf16_round(sigmoidf_(gv[k]));
  reinterpret_cast<uint4*>(y)[i] = pack8(o);
}

__global__ void __launch_bounds__(256) sigmoid_mul_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                               const __nv_bfloat16* __restrict__ g, __nv_bfloat16* __restrict__ dx,
                                                               __nv_bfloat16* __restrict__ dg, long long n8) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= n8) return;
  float dv[8], xv[8], gv[8], ox[8], og[8];
  unpack8(reinterpret_cast<const uint4*>(dy)[i], dv);
  unpack8(reinterpret_cast<const uint4*>(x)[i], xv);
  unpack8(reinterpret_cast<const uint4*>(g)[i], gv);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float s = sigmoidf_(gv[k]);
    ox[k] = dv[k] * s;
    og[k] = dv[k] * xv[k] * s * (1.f - s);
  }
  reinterpret_cast<uint4*>(dx)[i] = pack8(ox);
  reinterpret_cast<uint4*>(dg)[i] = pack8(og);
}

at::Tensor sigmoid_mul_fwd(const at::Tensor& x, const at::Tensor& g) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && g.scalar_type() == at::kBFloat16 && x.is_contiguous() && g.is_contiguous() &&
                  x.numel() == g.numel() && x.numel() % 8 == 0, "sigmoid_mul_fwd: contiguous bf16 tensors of equal size (a multiple of 8 elements) required");
  const c10::cuda::CUDAGuard guard(x.device());
  auto y = at::empty_like(x);
  const long long n8 = x.numel() / 8;
  if (n8) sigmoid_mul_fwd_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      (const __nv_bfloat16*)x.data_ptr(), (const __nv_bfloat16*)g.data_ptr(), (__nv_bfloat16*)y.data_ptr(), n8);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return y;
}

std::vector<at::Tensor> sigmoid_mul_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& g) {
  TORCH_CHECK(dy.is_cuda() && dy.scalar_type() == at::kBFloat16 && dy.is_contiguous() && dy.numel() == x.numel(), "sigmoid_mul_bwd: bad gradient");
  const c10::cuda::CUDAGuard guard(x.device());
  auto dx = at::empty_like(x), dg = at::empty_like(g);
  const long long n8 = x.numel() / 8;
  if (n8) sigmoid_mul_bwd_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      (const __nv_bfloat16*)dy.data_ptr(), (const __nv_bfloat16*)x.data_ptr(), (const __nv_bfloat16*)g.data_ptr(), (__nv_bfloat16*)dx.data_ptr(),
      (__nv_bfloat16*)dg.data_ptr(), n8);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {dx, dg};
}

// ---- shared-expert merge: out = routed + sigmoid(logit_t) * shared  (one warp per token row, 16-byte accesses) ------------
__global__ void __launch_bounds__(256) gate_add_fwd_kernel(const __nv_bfloat16* __restrict__ routed, const __nv_bfloat16* __restrict__ shared,
                                                            const __nv_bfloat16* __restrict__ logit, __nv_bfloat16* __restrict__ out, int T, int h) {
  const int lane = threadIdx.x & 31;
  const long long t = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= T) return;
  const float s = bf16_round(sigmoidf_(__bfloat162float(logit[t])));
  for (int c = lane; c < h / 8; c += 32) {
    float a[8], b[8], o[8];
    unpack8(reinterpret_cast<const uint4*>(routed + t * h)[c], a);
    unpack8(reinterpret_cast<const uint4*>(shared + t * h)[c], b);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = a[i] + bf16_round(s * b[i]);
    reinterpret_cast<uint4*>(out + t * h)[c] = pack8(o);
  }
}

// d(shared) = dy * sigmoid(logit);  d(logit)_t = sigmoid'(logit) * <dy_t, shared_t>;  d(routed) = dy needs no kernel
__global__ void __launch_bounds__(256) gate_add_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ shared,
                                                            const __nv_bfloat16* __restrict__ logit, __nv_bfloat16* __restrict__ dshared,
                                                            __nv_bfloat16* __restrict__ dlogit, int T, int h) {
  const int lane = threadIdx.x & 31;
  const long long t = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= T) return;
  const float s = bf16_round(sigmoidf_(__bfloat162float(logit[t])));
  float dot = 0.f;
  for (int c = lane; c < h / 8; c += 32) {
    float g[8], b[8], o[8];
    unpack8(reinterpret_cast<const uint4*>(dy + t * h)[c], g);
    unpack8(reinterpret_cast<const uint4*>(shared + t * h)[c], b);
#pragma unroll
    for (int i = 0; i < 8; ++i) { o[i] = g[i] * s; dot += g[i] * b[i]; }
    reinterpret_cast<uint4*>(dshared + t * h)[c] = pack8(o);
  }
  dot = warp_sum(dot);
  if (lane == 0) dlogit[t] = __float2bfloat16_rn(dot * s * (1.f - s));
}

at::Tensor gate_add_fwd(const at::Tensor& routed, const at::Tensor& shared, const at::Tensor& logit) {
  TORCH_CHECK(routed.is_cuda() && routed.scalar_type() == at::kBFloat16 && routed.is_contiguous() && shared.is_contiguous() && logit.is_contiguous() &&
                  routed.dim() == 2 && routed.sizes() == shared.sizes() && logit.numel() == routed.size(0) && routed.size(1) % 8 == 0,
              "gate_add_fwd: contiguous bf16 [T,h] (h a multiple of 8) and [T,1] required");
  const c10::cuda::CUDAGuard guard(routed.device());
  const int T = routed.size(0), h = routed.size(1);
  auto out = at::empty_like(routed);
  if (T) gate_add_fwd_kernel<<<(T + 7) / 8, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      (const __nv_bfloat16*)routed.data_ptr(), (const __nv_bfloat16*)shared.data_ptr(), (const __nv_bfloat16*)logit.data_ptr(), (__nv_bfloat16*)out.data_ptr(), T, h);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return out;
}

std::vector<at::Tensor> gate_add_bwd(const at::Tensor& dy, const at::Tensor& shared, const at::Tensor& logit) {
  TORCH_CHECK(dy.is_cuda() && dy.scalar_type() == at::kBFloat16 && dy.is_contiguous() && shared.is_contiguous() && dy.sizes() == shared.sizes(), "gate_add_bwd: bad inputs");
  const c10::cuda::CUDAGuard guard(dy.device());
  const int T = dy.size(0), h = dy.size(1);
  auto dshared = at::empty_like(shared), dlogit = at::empty_like(logit);
  if (T) gate_add_bwd_kernel<<<(T + 7) / 8, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      (const __nv_bfloat16*)dy.data_ptr(), (const __nv_bfloat16*)shared.data_ptr(), (const __nv_bfloat16*)logit.data_ptr(), (__nv_bfloat16*)dshared.data_ptr(),
      (__nv_bfloat16*)dlogit.data_ptr(), T, h);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {dshared, dlogit};
}

// ---- Gated DeltaNet gates: beta = sigmoid(b), g = -exp(A_log) * softplus(a + dt_bias), per (token, value head) ----------
__global__ void __launch_bounds__(256) gdn_gates_fwd_kernel(const __nv_bfloat16* __restrict__ b_raw, const __nv_bfloat16* __restrict__ a_raw,
                                                             const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                                             __nv_bfloat16* __restrict__ beta, float* __restrict__ g, long long n, int H) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  const int h = i % H;
  beta[i] = __float2bfloat16_rn(sigmoidf_(__bfloat162float(b_raw[i])));
  const float x = __bfloat162float(a_raw[i]) + dt_bias[h];
  const float sp = x > 20.f ? x : log1pf(__expf(x));
  g[i] = -__expf(A_log[h]) * sp;
}

// d(b) = d(beta) beta (1 - beta);  d(a) = d(g) (-exp(A_log)) sigmoid(a + dt_bias);  d(dt_bias)_h = sum_t d(a);  d(A_log)_h = sum_t d(g) g
__global__ void __launch_bounds__(256) gdn_gates_bwd_kernel(const __nv_bfloat16* __restrict__ dbeta, const float* __restrict__ dg,
                                                             const __nv_bfloat16* __restrict__ b_raw, const __nv_bfloat16* __restrict__ a_raw,
                                                             const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                                             __nv_bfloat16* __restrict__ db_raw, __nv_bfloat16* __restrict__ da_raw,
                                                             float* __restrict__ dA_log, float* __restrict__ ddt_bias, long long rows, int H) {
  extern __shared__ float acc[];                     // [2 * H]
  for (int i = threadIdx.x; i < 2 * H; i += blockDim.x) acc[i] = 0.f;
  __syncthreads();
  // thread -> fixed head column, walking rows: a thread's partial sums belong to one head
  const int per_row = H, cols_per_block = (256 / per_row) * per_row;
  if (cols_per_block > 0 && (int)threadIdx.x < cols_per_block) {
    const int h = threadIdx.x % per_row, r0 = threadIdx.x / per_row, rstep = 256 / per_row;
    const float na = -__expf(A_log[h]), bias = dt_bias[h];
    float s_a = 0.f, s_l = 0.f;
    for (long long r = (long long)blockIdx.x * rstep + r0; r < rows; r += (long long)gridDim.x * rstep) {
      const long long i = r * H + h;
      const float be = sigmoidf_(__bfloat162float(b_raw[i]));
      db_raw[i] = __float2bfloat16_rn(__bfloat162float(dbeta[i]) * be * (1.f - be));
      const float x = __bfloat162float(a_raw[i]) + bias;
      const float sp = x > 20.f ? x : log1pf(__expf(x));
      const float dgi = dg[i];
      const float da = dgi * na * (x > 20.f ? 1.f : sigmoidf_(x));
      da_raw[i] = __float2bfloat16_rn(da);
      s_a += da;
      s_l += dgi * na * sp;
    }
    atomicAdd(&acc[h], s_l);
    atomicAdd(&acc[H + h], s_a);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < H; i += blockDim.x) { atomicAdd(&dA_log[i], acc[i]); atomicAdd(&ddt_bias[i], acc[H + i]); }
}

// b_raw, a_raw [T,H] bf16 -> {beta [T,H] bf16, g [T,H] fp32}
std::vector<at::Tensor> gdn_gates_fwd(const at::Tensor& b_raw, const at::Tensor& a_raw, const at::Tensor& A_log, const at::Tensor& dt_bias) {
  TORCH_CHECK(b_raw.is_cuda() && b_raw.scalar_type() == at::kBFloat16 && a_raw.scalar_type() == at::kBFloat16 && b_raw.is_contiguous() && a_raw.is_contiguous() &&
                  b_raw.sizes() == a_raw.sizes() && A_log.scalar_type() == at::kFloat && dt_bias.scalar_type() == at::kFloat && A_log.is_contiguous() &&
                  dt_bias.is_contiguous() && A_log.numel() == b_raw.size(-1) && dt_bias.numel() == b_raw.size(-1) && b_raw.size(-1) <= 256,
              "gdn_gates_fwd: bf16 [..,H] projections and fp32 [H] parameters required (H <= 256)");
  const c10::cuda::CUDAGuard guard(b_raw.device());
  const int H = b_raw.size(-1);
  const long long n = b_raw.numel();
  auto beta = at::empty_like(b_raw);
  auto g = at::empty(b_raw.sizes(), b_raw.options().dtype(at::kFloat));
  if (n) gdn_gates_fwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      (const __nv_bfloat16*)b_raw.data_ptr(), (const __nv_bfloat16*)a_raw.data_ptr(), A_log.data_ptr<float>(), dt_bias.data_ptr<float>(),
      (__nv_bfloat16*)beta.data_ptr(), g.data_ptr<float>(), n, H);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {beta, g};
}

// -> {d(b_raw), d(a_raw) bf16, d(A_log), d(dt_bias) fp32 [H]}
std::vector<at::Tensor> gdn_gates_bwd(const at::Tensor& dbeta, const at::Tensor& dg, const at::Tensor& b_raw, const at::Tensor& a_raw, const at::Tensor& A_log,
                                      const at::Tensor& dt_bias) {
  TORCH_CHECK(dbeta.is_cuda() && dbeta.scalar_type() == at::kBFloat16 && dg.scalar_type() == at::kFloat && dbeta.is_contiguous() && dg.is_contiguous() &&
                  dbeta.sizes() == b_raw.sizes() && dg.sizes() == b_raw.sizes(), "gdn_gates_bwd: bf16 d(beta) and fp32 d(g) shaped like the projections required");
  const c10::cuda::CUDAGuard guard(b_raw.device());
  const int H = b_raw.size(-1);
  const long long rows = b_raw.numel() / H;
  auto db = at::empty_like(b_raw), da = at::empty_like(a_raw);
  auto dA = at::zeros({H}, A_log.options()), dbias = at::zeros({H}, A_log.options());
  if (rows) gdn_gates_bwd_kernel<<<(unsigned)std::min<long long>((rows + 11) / 12, 4 * kNumSMs), 256, 2 * H * sizeof(float), at::cuda::getCurrentCUDAStream()>>>(
      (const __nv_bfloat16*)dbeta.data_ptr(), dg.data_ptr<float>(), (const __nv_bfloat16*)b_raw.data_ptr(), (const __nv_bfloat16*)a_raw.data_ptr(),
      A_log.data_ptr<float>(), dt_bias.data_ptr<float>(), (__nv_bfloat16*)db.data_ptr(), (__nv_bfloat16*)da.data_ptr(), dA.data_ptr<float>(),
      dbias.data_ptr<float>(), rows, H);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {db, da, dA, dbias};
}

at::Tensor gated_rmsnorm_fwd(const at::Tensor& x, const at::Tensor& gate, const at::Tensor& w, double eps) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && gate.scalar_type() == at::kBFloat16 && x.size(-1) == 64 &&
              x.is_contiguous() && gate.is_contiguous() && w.scalar_type() == at::kFloat, "gated_rmsnorm_fwd: bf16 [.., 64] inputs required");
  const c10::cuda::CUDAGuard guard(x.device());
  const int rows = x.numel() / 64;
  auto y = at::empty_like(x);
  if (rows) gated_rmsnorm_fwd_kernel<<<(rows + 31) / 32, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      (const __nv_bfloat16*)x.data_ptr(), (const __nv_bfloat16*)gate.data_ptr(), w.data_ptr<float>(), (__nv_bfloat16*)y.data_ptr(), rows, (float)eps);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return y;
}

std::vector<at::Tensor> gated_rmsnorm_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& gate, const at::Tensor& w, double eps) {
  TORCH_CHECK(dy.is_contiguous() && dy.scalar_type() == at::kBFloat16 && x.size(-1) == 64, "gated_rmsnorm_bwd: bad inputs");
  const c10::cuda::CUDAGuard guard(x.device());
  const int rows = x.numel() / 64;
  auto dx = at::empty_like(x), dgate = at::empty_like(gate);
  auto dw = at::zeros({64}, x.options().dtype(at::kFloat));
  if (rows) gated_rmsnorm_bwd_kernel<<<std::min((rows + 31) / 32, kNumSMs * 8), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      (const __nv_bfloat16*)dy.data_ptr(), (const __nv_bfloat16*)x.data_ptr(), (const __nv_bfloat16*)gate.data_ptr(), w.data_ptr<float>(),
      (__nv_bfloat16*)dx.data_ptr(), (__nv_bfloat16*)dgate.data_ptr(), dw.data_ptr<float>(), rows, (float)eps);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {dx, dgate, dw};
}

// ---- flat AdamW (decoupled decay first, torch.optim.AdamW arithmetic), optional bf16 shadow write --------------------
__global__ void __launch_bounds__(256) adamw_flat_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                                                          float* __restrict__ v, __nv_bfloat16* __restrict__ shadow,
                                                          const float* __restrict__ grad_scale, size_t n, float lr, float wd, float b1,
                                                          float b2, float eps, float inv_bc1, float inv_sqrt_bc2,
                                                          const float* __restrict__ hyper, const int* __restrict__ err) {
  if (err != nullptr && *reinterpret_cast<const volatile int*>(err) != 0) return;   // a peer missed a barrier: leave parameters and moments untouched
  const float gs = grad_scale ? *grad_scale : 1.f;
  if (hyper) { lr = hyper[0]; inv_bc1 = hyper[1]; inv_sqrt_bc2 = hyper[2]; }   // step-dependent scalars from device memory (CUDA-graph replay)
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float gi = g[i] * gs;
    float pi = p[i] * (1.f - lr * wd);
    const float mi = m[i] + (gi - m[i]) * (1.f - b1);
    const float vi = v[i] * b2 + gi * gi * (1.f - b2);
    pi -= lr * inv_bc1 * mi / (sqrtf(vi) * inv_sqrt_bc2 + eps);
    p[i] = pi; m[i] = mi; v[i] = vi;
    if (shadow) shadow[i] = __float2bfloat16_rn(pi);
  }
}

void adamw_flat(at::Tensor& p, const at::Tensor& g, at::Tensor& m, at::Tensor& v, c10::optional<at::Tensor> shadow,
                c10::optional<at::Tensor> grad_scale, int64_t step, double lr, double wd, double beta1, double beta2, double eps,
                c10::optional<at::Tensor> hyper, c10::optional<at::Tensor> err) {
  TORCH_CHECK(!hyper.has_value() || (hyper->is_cuda() && hyper->scalar_type() == at::kFloat && hyper->is_contiguous() && hyper->numel() >= 3),
              "adamw_flat: hyper must be a CUDA fp32 tensor {lr, 1/(1-b1^t), 1/sqrt(1-b2^t)}");
  TORCH_CHECK(p.is_cuda() && p.scalar_type() == at::kFloat && p.is_contiguous() && g.is_contiguous() && m.is_contiguous() && v.is_contiguous(),
              "adamw_flat: contiguous fp32 CUDA tensors required");
  const c10::cuda::CUDAGuard guard(p.device());
  const size_t n = p.numel();
  if (!n) return;
  const double bc1 = 1.0 - std::pow(beta1, (double)step), bc2 = 1.0 - std::pow(beta2, (double)step);
  const int grid = (int)std::min<size_t>((n + 255) / 256, (size_t)kNumSMs * 16);
  adamw_flat_kernel<<<grid, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      p.data_ptr<float>(), g.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(),
      shadow.has_value() ? (__nv_bfloat16*)shadow->data_ptr() : nullptr, grad_scale.has_value() ? grad_scale->data_ptr<float>() : nullptr,
      n, (float)lr, (float)wd, (float)beta1, (float)beta2, (float)eps, (float)(1.0 / bc1), (float)(1.0 / std::sqrt(bc2)),
      hyper.has_value() ? hyper->data_ptr<float>() : nullptr, err.has_value() ? err->data_ptr<int>() : nullptr);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

// ---- sum of squares of a flat fp32 tensor -> one fp32 scalar (double accumulation across CTAs) ------------------------
__global__ void __launch_bounds__(256) sum_squares_kernel(const float* __restrict__ x, size_t n, double* __restrict__ out) {
  __shared__ float scratch[32];
  float acc = 0.f;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) acc += x[i] * x[i];
  acc = block_sum(acc, scratch);
  if (threadIdx.x == 0) atomicAdd(out, (double)acc);
}

at::Tensor sum_squares(const at::Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kFloat && x.is_contiguous(), "sum_squares: contiguous fp32 CUDA tensor required");
  const c10::cuda::CUDAGuard guard(x.device());
  auto out = at::zeros({}, x.options().dtype(at::kDouble));
  const size_t n = x.numel();
  if (n) {
    const int grid = (int)std::min<size_t>((n + 255) / 256, (size_t)kNumSMs * 8);
    sum_squares_kernel<<<grid, 256, 0, at::cuda::getCurrentCUDAStream()>>>(x.data_ptr<float>(), n, out.data_ptr<double>());
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  }
  return out;
}

}  // namespace q38
