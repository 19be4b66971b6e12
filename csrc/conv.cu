// Depthwise causal convolution (kernel 4, left padding 3) fused with SiLU on the [B, S, C] layout, forward and backward.
// Every thread owns two adjacent channels and a run of RUN tokens, sliding a 4-token window through registers, so x is
// read once and y written once with fully coalesced 4-byte accesses across channels.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"
#include "host.h"

namespace q38 {

constexpr int RUN = 32, RUN_BWD = 128, KW = 4;   // tokens per thread: the backward uses longer runs (fewer atomics per weight-gradient element)
using bf16 = __nv_bfloat16;

__device__ __forceinline__ float2 ld2(const bf16* p) { const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(p); return make_float2(__low2float(v), __high2float(v)); }

// y[b,t,c] = silu( sum_j w[c,j] * x[b,t-3+j,c] ),  x out of range = 0
__global__ void __launch_bounds__(128) conv_silu_fwd_kernel(const bf16* __restrict__ x, const float* __restrict__ w, bf16* __restrict__ y, int S, int C) {
  const int c = 2 * (blockIdx.x * 128 + threadIdx.x);
  if (c >= C) return;
  const int t0 = blockIdx.y * RUN, b = blockIdx.z;
  const bf16* xb = x + ((size_t)b * S) * C + c;
  bf16* yb = y + ((size_t)b * S) * C + c;
  float w0[KW], w1[KW];
#pragma unroll
  for (int j = 0; j < KW; ++j) { w0[j] = bf16_round(w[c * KW + j]); w1[j] = bf16_round(w[(c + 1) * KW + j]); }
  float2 win[KW];
#pragma unroll
  for (int j = 0; j < KW - 1; ++j) { const int t = t0 - 3 + j; win[j + 1] = t >= 0 ? ld2(xb + (size_t)t * C) : make_float2(0.f, 0.f); }
  for (int i = 0; i < RUN && t0 + i < S; ++i) {
#pragma unroll
    for (int j = 0; j < KW - 1; ++j) win[j] = win[j + 1];
    win[KW - 1] = ld2(xb + (size_t)(t0 + i) * C);
    float a0 = 0.f, a1 = 0.f;
#pragma unroll
    for (int j = 0; j < KW; ++j) { a0 += w0[j] * win[j].x; a1 += w1[j] * win[j].y; }
    a0 = bf16_round(a0); a1 = bf16_round(a1);                       // the convolution output is bf16 before the activation
    *reinterpret_cast<__nv_bfloat162*>(yb + (size_t)(t0 + i) * C) = __floats2bfloat162_rn(siluf_(a0), siluf_(a1));
  }
}

// dpre[t] = dy[t] * silu'(pre[t]);  dx[t] = sum_j w[j] * dpre[t+3-j];  dw[j] += sum_t dpre[t] * x[t-3+j]
__global__ void __launch_bounds__(128) conv_silu_bwd_kernel(const bf16* __restrict__ x, const float* __restrict__ w, const bf16* __restrict__ dy,
                                                            bf16* __restrict__ dx, float* __restrict__ dw, int S, int C) {
  const int c = 2 * (blockIdx.x * 128 + threadIdx.x);
  if (c >= C) return;
  const int t0 = blockIdx.y * RUN_BWD, b = blockIdx.z;
  const bf16* xb = x + ((size_t)b * S) * C + c;
  const bf16* gb = dy + ((size_t)b * S) * C + c;
  bf16* dxb = dx + ((size_t)b * S) * C + c;
  float w0[KW], w1[KW], g0[KW] = {0.f, 0.f, 0.f, 0.f}, g1[KW] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < KW; ++j) { w0[j] = bf16_round(w[c * KW + j]); w1[j] = bf16_round(w[(c + 1) * KW + j]); }
  // token t needs dpre[t .. t+3]; walk tokens t0 .. t0+RUN+2 and emit dx for token (cursor - 3)
  float2 win[KW];                                         // x[t-3 .. t]
  float2 dpre_win[KW] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};   // dpre[t-3 .. t]
#pragma unroll
  for (int j = 0; j < KW - 1; ++j) { const int t = t0 - 3 + j; win[j + 1] = t >= 0 ? ld2(xb + (size_t)t * C) : make_float2(0.f, 0.f); }
  // Tokens are walked in groups of eight whose x and dy values are fetched up front (sixteen independent loads in flight per
  // thread); the recurrence over the window is then evaluated from registers.
  constexpr int STEPS = RUN_BWD + KW - 1, GROUP = 8;
  for (int i0 = 0; i0 < STEPS; i0 += GROUP) {
    float2 xs[GROUP], gs[GROUP];
#pragma unroll
    for (int u = 0; u < GROUP; ++u) {
      const int t = t0 + i0 + u;
      const bool ok = i0 + u < STEPS && t < S;
      xs[u] = ok ? ld2(xb + (size_t)t * C) : make_float2(0.f, 0.f);
      gs[u] = ok ? ld2(gb + (size_t)t * C) : make_float2(0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < GROUP; ++u) {
      const int i = i0 + u, t = t0 + i;
      if (i >= STEPS) break;
#pragma unroll
      for (int j = 0; j < KW - 1; ++j) { win[j] = win[j + 1]; dpre_win[j] = dpre_win[j + 1]; }
      float2 dp = make_float2(0.f, 0.f);
      win[KW - 1] = xs[u];                                  // zero beyond the sequence end
      if (t < S) {
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int j = 0; j < KW; ++j) { a0 += w0[j] * win[j].x; a1 += w1[j] * win[j].y; }
        a0 = bf16_round(a0); a1 = bf16_round(a1);
        const float2 g = gs[u];
        const float s0 = sigmoidf_(a0), s1 = sigmoidf_(a1);
        dp = make_float2(g.x * s0 * (1.f + a0 * (1.f - s0)), g.y * s1 * (1.f + a1 * (1.f - s1)));
        if (i < RUN_BWD) {                                      // weight gradient: only tokens owned by this run
#pragma unroll
          for (int j = 0; j < KW; ++j) { g0[j] += dp.x * win[j].x; g1[j] += dp.y * win[j].y; }
        }
      }
      dpre_win[KW - 1] = dp;
      const int to = t - (KW - 1);                          // dx[to] = sum_j w[j] dpre[to+3-j] = sum_j w[j] dpre_win[3-j]
      if (i >= KW - 1 && to < S) {
        float d0 = 0.f, d1 = 0.f;
#pragma unroll
        for (int j = 0; j < KW; ++j) { d0 += w0[j] * dpre_win[KW - 1 - j].x; d1 += w1[j] * dpre_win[KW - 1 - j].y; }
        *reinterpret_cast<__nv_bfloat162*>(dxb + (size_t)to * C) = __floats2bfloat162_rn(d0, d1);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < KW; ++j) { atomicAdd(&dw[c * KW + j], g0[j]); atomicAdd(&dw[(c + 1) * KW + j], g1[j]); }
}

at::Tensor conv_silu_fwd(const at::Tensor& x, const at::Tensor& w) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.is_contiguous() && x.dim() == 3 && x.size(2) % 2 == 0, "conv_silu_fwd: contiguous bf16 [B,S,C] with even C required");
  TORCH_CHECK(w.scalar_type() == at::kFloat && w.is_contiguous() && w.numel() == x.size(2) * KW, "conv_silu_fwd: weight must be fp32 [C,4]");
  const c10::cuda::CUDAGuard guard(x.device());
  const int B = x.size(0), S = x.size(1), C = x.size(2);
  auto y = at::empty_like(x);
  dim3 grid((C / 2 + 127) / 128, (S + RUN - 1) / RUN, B);
  conv_silu_fwd_kernel<<<grid, 128, 0, at::cuda::getCurrentCUDAStream()>>>((const bf16*)x.data_ptr(), w.data_ptr<float>(), (bf16*)y.data_ptr(), S, C);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return y;
}

std::vector<at::Tensor> conv_silu_bwd(const at::Tensor& x, const at::Tensor& w, const at::Tensor& dy) {
  TORCH_CHECK(dy.is_cuda() && dy.scalar_type() == at::kBFloat16 && dy.is_contiguous() && x.is_contiguous(), "conv_silu_bwd: contiguous bf16 tensors required");
  const c10::cuda::CUDAGuard guard(x.device());
  const int B = x.size(0), S = x.size(1), C = x.size(2);
  auto dx = at::empty_like(x);
  auto dw = at::zeros({C, KW}, x.options().dtype(at::kFloat));
  dim3 grid((C / 2 + 127) / 128, (S + RUN_BWD - 1) / RUN_BWD, B);
  conv_silu_bwd_kernel<<<grid, 128, 0, at::cuda::getCurrentCUDAStream()>>>((const bf16*)x.data_ptr(), w.data_ptr<float>(), (const bf16*)dy.data_ptr(),
                                                                           (bf16*)dx.data_ptr(), dw.data_ptr<float>(), S, C);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {dx, dw};
}

}  // namespace q38
