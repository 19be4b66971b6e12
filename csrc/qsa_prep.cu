// Head preparation for the QSA layer and its indexer: per (token, head) optional zero-centred RMSNorm over the 64 head dims,
// rotary embedding on the first 16 dims (rotate-half pairs d <-> d + 8), and the move from token-major [B,S,H,*] projection
// output to the head-major [B,H,S,64] layout of the attention kernels, in one pass.  For the query projection, whose rows hold
// q and the output gate interleaved per head ([.., H, 128]), the gate half is copied out to [B,S,H*64] in the same pass.
// The backward kernel undoes all of it and writes the gradient of the projection output (both halves) directly.
//
// One warp per (b, s, h) row, lane l owns dims 2l, 2l+1, so the rotary partner of lanes 0..3 is lane + 4.
// cos/sin: fp32 [Bc, S, 16] with Bc in {1, B}; they are rounded to bf16 as the PyTorch path does before use.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"
#include "host.h"

namespace q38 {

constexpr int HP_WARPS = 8;
using bf16 = __nv_bfloat16;

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__global__ void __launch_bounds__(32 * HP_WARPS) qsa_headprep_fwd_kernel(const bf16* __restrict__ src, long long src_row, const float* __restrict__ w,
                                                                         const float* __restrict__ cosv, const float* __restrict__ sinv, int Bc,
                                                                         bf16* __restrict__ out, bf16* __restrict__ gate, float* __restrict__ rstd_out,
                                                                         int B, int S, int H, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * HP_WARPS + warp;            // (b, s, h)
  if (row >= (long long)B * S * H) return;
  const int h = row % H, s = (row / H) % S, b = row / ((long long)H * S);
  const bf16* p = src + row * src_row;
  const __nv_bfloat162 raw = *reinterpret_cast<const __nv_bfloat162*>(p + 2 * lane);
  float x0 = __low2float(raw), x1 = __high2float(raw);
  if (gate != nullptr) *reinterpret_cast<__nv_bfloat162*>(gate + row * 64 + 2 * lane) = *reinterpret_cast<const __nv_bfloat162*>(p + 64 + 2 * lane);
  if (w != nullptr) {
    const float ss = warp_sum(x0 * x0 + x1 * x1);
    const float rstd = rsqrtf(ss / 64.f + eps);
    if (lane == 0) rstd_out[row] = rstd;
    x0 = bf16r(x0 * rstd * (1.f + w[2 * lane]));
    x1 = bf16r(x1 * rstd * (1.f + w[2 * lane + 1]));
  }
  const float o0 = __shfl_xor_sync(0xffffffffu, x0, 4), o1 = __shfl_xor_sync(0xffffffffu, x1, 4);
  if (lane < 8) {
    const float* c = cosv + ((long long)(Bc == 1 ? 0 : b) * S + s) * 16 + 2 * lane;
    const float* sn = sinv + ((long long)(Bc == 1 ? 0 : b) * S + s) * 16 + 2 * lane;
    const float c0 = bf16r(c[0]), c1 = bf16r(c[1]), s0 = bf16r(sn[0]), s1 = bf16r(sn[1]);
    const float sign = lane < 4 ? -1.f : 1.f;
    x0 = x0 * c0 + sign * o0 * s0;
    x1 = x1 * c1 + sign * o1 * s1;
  }
  *reinterpret_cast<__nv_bfloat162*>(out + (((long long)b * H + h) * S + s) * 64 + 2 * lane) = __floats2bfloat162_rn(x0, x1);
}

__global__ void __launch_bounds__(32 * HP_WARPS) qsa_headprep_bwd_kernel(const bf16* __restrict__ dout, const bf16* __restrict__ dgate,
                                                                         const bf16* __restrict__ src, long long src_row, const float* __restrict__ w,
                                                                         const float* __restrict__ cosv, const float* __restrict__ sinv, int Bc,
                                                                         const float* __restrict__ rstd_in, bf16* __restrict__ dsrc, float* __restrict__ dw,
                                                                         int B, int S, int H) {
  __shared__ float dw_s[64];
  if (threadIdx.x < 64) dw_s[threadIdx.x] = 0.f;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * HP_WARPS + warp;
  if (row < (long long)B * S * H) {
    const int h = row % H, s = (row / H) % S, b = row / ((long long)H * S);
    const __nv_bfloat162 graw = *reinterpret_cast<const __nv_bfloat162*>(dout + (((long long)b * H + h) * S + s) * 64 + 2 * lane);
    float g0 = __low2float(graw), g1 = __high2float(graw);
    // rotary backward: dx_d = dy_d c_d + dy_{d+8} s_{d+8} (d < 8),  dx_{d+8} = dy_{d+8} c_{d+8} - dy_d s_d
    const float o0 = __shfl_xor_sync(0xffffffffu, g0, 4), o1 = __shfl_xor_sync(0xffffffffu, g1, 4);
    if (lane < 8) {
      const float* c = cosv + ((long long)(Bc == 1 ? 0 : b) * S + s) * 16 + 2 * lane;
      const float* sn = sinv + ((long long)(Bc == 1 ? 0 : b) * S + s) * 16 + 2 * lane;
      const float c0 = bf16r(c[0]), c1 = bf16r(c[1]), s0 = bf16r(sn[0]), s1 = bf16r(sn[1]);   // tables repeat: entry d + 8 equals entry d
      const float sign = lane < 4 ? 1.f : -1.f;
      g0 = g0 * c0 + sign * o0 * s0;
      g1 = g1 * c1 + sign * o1 * s1;
    }
    bf16* dp = dsrc + row * src_row;
    if (w != nullptr) {
      const bf16* p = src + row * src_row;
      const __nv_bfloat162 raw = *reinterpret_cast<const __nv_bfloat162*>(p + 2 * lane);
      const float rstd = rstd_in[row];
      const float xh0 = __low2float(raw) * rstd, xh1 = __high2float(raw) * rstd;
      atomicAdd(&dw_s[2 * lane], g0 * xh0);
      atomicAdd(&dw_s[2 * lane + 1], g1 * xh1);
      g0 *= 1.f + w[2 * lane];
      g1 *= 1.f + w[2 * lane + 1];
      const float dot = warp_sum(g0 * xh0 + g1 * xh1) / 64.f;
      g0 = rstd * (g0 - xh0 * dot);
      g1 = rstd * (g1 - xh1 * dot);
    }
    *reinterpret_cast<__nv_bfloat162*>(dp + 2 * lane) = __floats2bfloat162_rn(g0, g1);
    if (dgate != nullptr) *reinterpret_cast<__nv_bfloat162*>(dp + 64 + 2 * lane) = *reinterpret_cast<const __nv_bfloat162*>(dgate + row * 64 + 2 * lane);
  }
  __syncthreads();
  if (w != nullptr && threadIdx.x < 64) atomicAdd(&dw[threadIdx.x], dw_s[threadIdx.x]);
}

static void check_tables(const at::Tensor& cosv, const at::Tensor& sinv, int B, int S) {
  TORCH_CHECK(cosv.scalar_type() == at::kFloat && sinv.scalar_type() == at::kFloat && cosv.is_contiguous() && sinv.is_contiguous() && cosv.dim() == 3 &&
                  cosv.sizes() == sinv.sizes() && cosv.size(2) == 16 && cosv.size(1) == S && (cosv.size(0) == 1 || cosv.size(0) == B),
              "qsa_headprep: cos/sin must be contiguous fp32 [1 or B, S, 16]");
}

// src [B,S,H,64] or, with split_gate, [B,S,H,128] (q | gate) bf16 contiguous -> {out [B,H,S,64], gate [B,S,H*64] or empty, rstd [B,S,H] or empty}
std::vector<at::Tensor> qsa_headprep_fwd(const at::Tensor& src, const c10::optional<at::Tensor>& w, const at::Tensor& cosv, const at::Tensor& sinv, double eps,
                                         bool split_gate) {
  TORCH_CHECK(src.is_cuda() && src.scalar_type() == at::kBFloat16 && src.is_contiguous() && src.dim() == 4 && src.size(3) == (split_gate ? 128 : 64),
              "qsa_headprep_fwd: contiguous bf16 [B,S,H,64] (or [B,S,H,128] with the gate) required");
  TORCH_CHECK(!w.has_value() || (w->scalar_type() == at::kFloat && w->is_contiguous() && w->numel() == 64), "qsa_headprep_fwd: norm weight must be fp32 [64]");
  const c10::cuda::CUDAGuard guard(src.device());
  const int B = src.size(0), S = src.size(1), H = src.size(2);
  check_tables(cosv, sinv, B, S);
  auto out = at::empty({B, H, S, 64}, src.options());
  auto gate = at::empty({split_gate ? B : 0, S, H * 64}, src.options());
  auto rstd = at::empty({w.has_value() ? B : 0, S, H}, src.options().dtype(at::kFloat));
  const long long rows = (long long)B * S * H;
  qsa_headprep_fwd_kernel<<<(unsigned)((rows + HP_WARPS - 1) / HP_WARPS), 32 * HP_WARPS, 0, at::cuda::getCurrentCUDAStream()>>>(
      (const bf16*)src.data_ptr(), src.size(3), w.has_value() ? w->data_ptr<float>() : nullptr, cosv.data_ptr<float>(), sinv.data_ptr<float>(), (int)cosv.size(0),
      (bf16*)out.data_ptr(), split_gate ? (bf16*)gate.data_ptr() : nullptr, w.has_value() ? rstd.data_ptr<float>() : nullptr, B, S, H, (float)eps);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {out, gate, rstd};
}

// dout [B,H,S,64], dgate [B,S,H*64] (with split_gate) -> {dsrc like src, dw [64] (zeros without a norm)}
std::vector<at::Tensor> qsa_headprep_bwd(const at::Tensor& dout, const c10::optional<at::Tensor>& dgate, const at::Tensor& src, const c10::optional<at::Tensor>& w,
                                         const at::Tensor& cosv, const at::Tensor& sinv, const at::Tensor& rstd) {
  TORCH_CHECK(dout.is_cuda() && dout.scalar_type() == at::kBFloat16 && dout.is_contiguous() && src.is_contiguous() && src.dim() == 4, "qsa_headprep_bwd: bad inputs");
  const c10::cuda::CUDAGuard guard(src.device());
  const int B = src.size(0), S = src.size(1), H = src.size(2);
  const bool split = src.size(3) == 128;
  TORCH_CHECK(dout.size(0) == B && dout.size(1) == H && dout.size(2) == S && dout.size(3) == 64 && split == dgate.has_value(), "qsa_headprep_bwd: shape mismatch");
  TORCH_CHECK(!split || (dgate->scalar_type() == at::kBFloat16 && dgate->is_contiguous() && dgate->numel() == (long long)B * S * H * 64), "qsa_headprep_bwd: bad gate gradient");
  check_tables(cosv, sinv, B, S);
  auto dsrc = at::empty_like(src);
  auto dw = at::zeros({64}, src.options().dtype(at::kFloat));
  const long long rows = (long long)B * S * H;
  qsa_headprep_bwd_kernel<<<(unsigned)((rows + HP_WARPS - 1) / HP_WARPS), 32 * HP_WARPS, 0, at::cuda::getCurrentCUDAStream()>>>(
      (const bf16*)dout.data_ptr(), split ? (const bf16*)dgate->data_ptr() : nullptr, (const bf16*)src.data_ptr(), src.size(3),
      w.has_value() ? w->data_ptr<float>() : nullptr, cosv.data_ptr<float>(), sinv.data_ptr<float>(), (int)cosv.size(0),
      w.has_value() ? rstd.data_ptr<float>() : nullptr, (bf16*)dsrc.data_ptr(), dw.data_ptr<float>(), B, S, H);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {dsrc, dw};
}

}  // namespace q38
