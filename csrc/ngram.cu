// Hashed bigram / trigram embeddings: row hash, two-table gather, RMSNorm, and the backward scatter-add.
//
//   ngram_fwd   one warp per token: the predecessors a = ids[t-1], c = ids[t-2] are replaced by the placeholder id `vocab`
//               when they lie before the latest EOS at or before t, which reduces to a local rule (a is hidden when ids[t] is
//               the EOS, c when ids[t] or ids[t-1] is); rows i2, i3 from the wrapping 64-bit hashes; e = rmsnorm(emb2[i2] +
//               emb3[i3]) * w in fp32 -> bf16, 1/rms kept for the backward.
//   ngram_bwd   one warp per token: the RMSNorm backward of d(e) gives the gradient of the summed row, which is added with fp32
//               atomics to row i2 of the first table's gradient and row i3 of the second's (the gradient buffers of the
//               parameters themselves), and d(norm weight) is reduced per CTA.
// The hash is (a P2_0) ^ (b P2_1), resp. (c P3_0) ^ (a P3_1) ^ (b P3_2), then h ^= h >> 17 (arithmetic), h *= MIX, all in
// wrapping int64, and the row is the non-negative remainder mod `rows`.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"
#include "host.h"

namespace q38 {

constexpr int NG_WARPS = 8;

__device__ __forceinline__ long long wrap_mul(long long a, long long b) {
  return static_cast<long long>(static_cast<unsigned long long>(a) * static_cast<unsigned long long>(b));
}
__device__ __forceinline__ int hash_row(long long h, long long rows) {
  h = wrap_mul(h ^ (h >> 17), 2654435761LL);
  long long r = h % rows;
  if (r < 0) r += rows;
  return static_cast<int>(r);
}

__global__ void __launch_bounds__(32 * NG_WARPS) ngram_fwd_kernel(const long long* __restrict__ ids, const float* __restrict__ emb2,
                                                                  const float* __restrict__ emb3, const float* __restrict__ norm_w,
                                                                  __nv_bfloat16* __restrict__ e, float* __restrict__ rstd_out, int* __restrict__ rows_out,
                                                                  int B, int T, int h, long long vocab, long long eos, long long rows, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long tok = (long long)blockIdx.x * NG_WARPS + warp;
  if (tok >= (long long)B * T) return;
  const int t = tok % T;
  const long long b = ids[tok];
  const long long prev1 = t >= 1 ? ids[tok - 1] : vocab, prev2 = t >= 2 ? ids[tok - 2] : vocab;
  const bool own_eos = b == eos;
  const long long a = (t >= 1 && !own_eos) ? prev1 : vocab;
  const long long c = (t >= 2 && !own_eos && prev1 != eos) ? prev2 : vocab;
  const int i2 = hash_row(wrap_mul(a, 1000003LL) ^ wrap_mul(b, 998244353LL), rows);
  const int i3 = hash_row(wrap_mul(c, 1000033LL) ^ wrap_mul(a, 998244353LL) ^ wrap_mul(b, 1000000007LL), rows);
  if (lane == 0) { rows_out[2 * tok] = i2; rows_out[2 * tok + 1] = i3; }
  const float4* r2 = reinterpret_cast<const float4*>(emb2 + (long long)i2 * h);
  const float4* r3 = reinterpret_cast<const float4*>(emb3 + (long long)i3 * h);
  const int h4 = h >> 2;
  float ss = 0.f;
  for (int q = lane; q < h4; q += 32) {
    const float4 x = r2[q], y = r3[q];
    const float4 s = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
    ss += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / h + eps);
  if (lane == 0) rstd_out[tok] = rstd;
  for (int q = lane; q < h4; q += 32) {
    const float4 x = r2[q], y = r3[q], w = reinterpret_cast<const float4*>(norm_w)[q];
    __nv_bfloat162 lo = __floats2bfloat162_rn((x.x + y.x) * rstd * w.x, (x.y + y.y) * rstd * w.y);
    __nv_bfloat162 hi = __floats2bfloat162_rn((x.z + y.z) * rstd * w.z, (x.w + y.w) * rstd * w.w);
    *reinterpret_cast<uint2*>(e + tok * h + 4 * q) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
  }
}

__global__ void __launch_bounds__(32 * NG_WARPS) ngram_bwd_kernel(const __nv_bfloat16* __restrict__ de, const int* __restrict__ rows_in,
                                                                  const float* __restrict__ emb2, const float* __restrict__ emb3,
                                                                  const float* __restrict__ norm_w, const float* __restrict__ rstd_in,
                                                                  float* __restrict__ g2, float* __restrict__ g3, float* __restrict__ dnorm_w,
                                                                  long long tokens, int h) {
  extern __shared__ float dw_s[];                   // [h]
  for (int i = threadIdx.x; i < h; i += blockDim.x) dw_s[i] = 0.f;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long tok = (long long)blockIdx.x * NG_WARPS + warp;
  if (tok < tokens) {
    const int i2 = rows_in[2 * tok], i3 = rows_in[2 * tok + 1];
    const float rstd = rstd_in[tok];
    const float* r2 = emb2 + (long long)i2 * h;
    const float* r3 = emb3 + (long long)i3 * h;
    float dot = 0.f;
    for (int i = lane; i < h; i += 32) {
      const float xhat = (r2[i] + r3[i]) * rstd, g = __bfloat162float(de[tok * h + i]);
      dot += g * norm_w[i] * xhat;
      atomicAdd(&dw_s[i], g * xhat);
    }
    dot = warp_sum(dot) / h;
    for (int i = lane; i < h; i += 32) {
      const float xhat = (r2[i] + r3[i]) * rstd, g = __bfloat162float(de[tok * h + i]) * norm_w[i];
      const float dx = rstd * (g - xhat * dot);
      atomicAdd(g2 + (long long)i2 * h + i, dx);
      atomicAdd(g3 + (long long)i3 * h + i, dx);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < h; i += blockDim.x) atomicAdd(&dnorm_w[i], dw_s[i]);
}

// Token-embedding backward: grad[ids[t], :] += dout[t, :] with fp32 atomics, one warp per token.
__global__ void __launch_bounds__(32 * NG_WARPS) embed_bwd_kernel(const long long* __restrict__ ids, const float* __restrict__ dout, float* __restrict__ grad,
                                                                  long long tokens, int h, long long vocab) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long tok = (long long)blockIdx.x * NG_WARPS + warp;
  if (tok >= tokens) return;
  const long long id = ids[tok];
  if (id < 0 || id >= vocab) return;
  const float* src = dout + tok * h;
  float* dst = grad + id * h;
  for (int i = lane; i < h; i += 32) atomicAdd(dst + i, src[i]);
}

void embed_bwd(const at::Tensor& ids, const at::Tensor& dout, at::Tensor& grad) {
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous() && dout.scalar_type() == at::kFloat && dout.is_contiguous() &&
                  grad.scalar_type() == at::kFloat && grad.is_contiguous() && grad.dim() == 2 && dout.numel() == ids.numel() * grad.size(1),
              "embed_bwd: int64 ids, fp32 gradient rows and an fp32 [vocab,h] gradient table required");
  const c10::cuda::CUDAGuard guard(ids.device());
  const long long tokens = ids.numel();
  if (tokens) embed_bwd_kernel<<<(unsigned)((tokens + NG_WARPS - 1) / NG_WARPS), 32 * NG_WARPS, 0, at::cuda::getCurrentCUDAStream()>>>(
      (const long long*)ids.data_ptr<int64_t>(), dout.data_ptr<float>(), grad.data_ptr<float>(), tokens, (int)grad.size(1), (long long)grad.size(0));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

// ids [B,T] int64, tables [rows,h] fp32 -> {e [B,T,h] bf16, rstd [B,T] fp32, rows [B,T,2] int32}
std::vector<at::Tensor> ngram_fwd(const at::Tensor& ids, const at::Tensor& emb2, const at::Tensor& emb3, const at::Tensor& norm_w, int64_t vocab,
                                  int64_t eos, double eps) {
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous() && ids.dim() == 2, "ngram_fwd: contiguous int64 ids [B,T] required");
  TORCH_CHECK(emb2.scalar_type() == at::kFloat && emb2.is_contiguous() && emb3.scalar_type() == at::kFloat && emb3.is_contiguous() && emb2.sizes() == emb3.sizes() &&
                  norm_w.scalar_type() == at::kFloat && norm_w.is_contiguous() && emb2.size(1) % 4 == 0,
              "ngram_fwd: fp32 tables [rows,h] with h a multiple of 4 required");
  const c10::cuda::CUDAGuard guard(ids.device());
  const int B = ids.size(0), T = ids.size(1), h = emb2.size(1);
  auto e = at::empty({B, T, h}, emb2.options().dtype(at::kBFloat16));
  auto rstd = at::empty({B, T}, emb2.options());
  auto rows = at::empty({B, T, 2}, emb2.options().dtype(at::kInt));
  const long long tokens = (long long)B * T;
  ngram_fwd_kernel<<<(unsigned)((tokens + NG_WARPS - 1) / NG_WARPS), 32 * NG_WARPS, 0, at::cuda::getCurrentCUDAStream()>>>(
      (const long long*)ids.data_ptr<int64_t>(), emb2.data_ptr<float>(), emb3.data_ptr<float>(), norm_w.data_ptr<float>(), (__nv_bfloat16*)e.data_ptr(),
      rstd.data_ptr<float>(), rows.data_ptr<int>(), B, T, h, (long long)vocab, (long long)eos, (long long)emb2.size(0), (float)eps);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {e, rstd, rows};
}

// Adds the table gradients into g2, g3 [rows,h] fp32 and returns d(norm weight) [h].
at::Tensor ngram_bwd(const at::Tensor& de, const at::Tensor& rows, const at::Tensor& emb2, const at::Tensor& emb3, const at::Tensor& norm_w,
                     const at::Tensor& rstd, at::Tensor& g2, at::Tensor& g3) {
  TORCH_CHECK(de.is_cuda() && de.scalar_type() == at::kBFloat16 && de.is_contiguous() && g2.scalar_type() == at::kFloat && g2.is_contiguous() &&
                  g3.scalar_type() == at::kFloat && g3.is_contiguous() && g2.sizes() == emb2.sizes() && g3.sizes() == emb3.sizes(),
              "ngram_bwd: bf16 gradient and fp32 gradient tables required");
  const c10::cuda::CUDAGuard guard(de.device());
  const int h = emb2.size(1);
  const long long tokens = de.numel() / h;
  auto dw = at::zeros({h}, emb2.options());
  ngram_bwd_kernel<<<(unsigned)((tokens + NG_WARPS - 1) / NG_WARPS), 32 * NG_WARPS, h * sizeof(float), at::cuda::getCurrentCUDAStream()>>>(
      (const __nv_bfloat16*)de.data_ptr(), rows.data_ptr<int>(), emb2.data_ptr<float>(), emb3.data_ptr<float>(), norm_w.data_ptr<float>(), rstd.data_ptr<float>(),
      g2.data_ptr<float>(), g3.data_ptr<float>(), dw.data_ptr<float>(), tokens, h);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return dw;
}

}  // namespace q38
