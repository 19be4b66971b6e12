// Indexer block log-probabilities for block selection only (evaluation, and training steps that take no KL term): selection
// looks at the first query of every 64-token block, so only those S/64 queries are scored.  One CTA per (query block, batch):
//     I[s]      = sum_h w_h relu(bf16(q_h . k_s)) * scale          for the keys s <= 64 i  (causal for the query at 64 i)
//     lp_blk[j] = logsumexp_{s in block j} I[s] - logsumexp_s I[s]  for j <= i, a large negative number for j > i
// The same rounding points as the full indexer kernel (qsa_index.cu) and the PyTorch specification: q.k is rounded to bf16 before
// the relu.  (Reference: modeling_qwen3_8_moe.py:1126-1131 scores these queries with eager matmul / einsum / log_softmax /
// logsumexp calls.)
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"
#include "host.h"

namespace q38 {

constexpr int QF_THREADS = 128, QF_HEADS_MAX = 4;
constexpr float QF_MASKED = -1e9f;

__global__ void __launch_bounds__(QF_THREADS) qsa_first_query_lp_kernel(const __nv_bfloat16* __restrict__ q_first, const __nv_bfloat16* __restrict__ ki,
                                                                        const float* __restrict__ w_first, float* __restrict__ lp_blk, int S, int NI,
                                                                        float scale) {
  extern __shared__ __align__(16) float qf_smem[];
  float* qs = qf_smem;                       // [NI][64]
  float* ws = qs + QF_HEADS_MAX * 64;        // [NI]
  float* red = ws + 4;                       // [8]
  float* scores = red + 8;                   // [S]
  const int i = blockIdx.x, b = blockIdx.y, nb = S / 64, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nkeys = 64 * i + 1;
  for (int e = tid; e < NI * 64; e += QF_THREADS) {
    const int h = e >> 6, d = e & 63;
    qs[e] = __bfloat162float(q_first[(((long long)b * NI + h) * nb + i) * 64 + d]);
  }
  if (tid < NI) ws[tid] = w_first[((long long)b * nb + i) * NI + tid];
  __syncthreads();
  float m = -INFINITY;
  for (int s = tid; s < nkeys; s += QF_THREADS) {
    const uint4* krow = reinterpret_cast<const uint4*>(ki + ((long long)b * S + s) * 64);
    float dot[QF_HEADS_MAX] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint4 raw = krow[c];
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
      float kv[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) { kv[2 * e] = __low2float(h2[e]); kv[2 * e + 1] = __high2float(h2[e]); }
#pragma unroll
      for (int h = 0; h < QF_HEADS_MAX; ++h) {
        if (h >= NI) break;
        const float4 qa = *reinterpret_cast<const float4*>(qs + h * 64 + 8 * c), qb = *reinterpret_cast<const float4*>(qs + h * 64 + 8 * c + 4);
        dot[h] += qa.x * kv[0] + qa.y * kv[1] + qa.z * kv[2] + qa.w * kv[3] + qb.x * kv[4] + qb.y * kv[5] + qb.z * kv[6] + qb.w * kv[7];
      }
    }
    float score = 0.f;
#pragma unroll
    for (int h = 0; h < QF_HEADS_MAX; ++h) if (h < NI) score += ws[h] * (fmaxf(bf16_round(dot[h]), 0.f) * scale);
    scores[s] = score;
    m = fmaxf(m, score);
  }
  m = warp_max(m);
  if (lane == 0) red[warp] = m;
  __syncthreads();
  m = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  float sum = 0.f;
  for (int s = tid; s < nkeys; s += QF_THREADS) sum += __expf(scores[s] - m);
  sum = warp_sum(sum);
  __syncthreads();
  if (lane == 0) red[4 + warp] = sum;
  __syncthreads();
  const float lse_all = m + __logf(red[4] + red[5] + red[6] + red[7]);
  float* out = lp_blk + ((long long)b * nb + i) * nb;
  for (int j = warp; j < nb; j += QF_THREADS / 32) {
    if (j > i) { if (lane == 0) out[j] = QF_MASKED; continue; }
    const int s0 = 64 * j + lane, s1 = s0 + 32;
    const float a = s0 < nkeys ? scores[s0] : -INFINITY, c = s1 < nkeys ? scores[s1] : -INFINITY;
    const float bm = warp_max(fmaxf(a, c));
    const float bs = warp_sum((s0 < nkeys ? __expf(a - bm) : 0.f) + (s1 < nkeys ? __expf(c - bm) : 0.f));
    if (lane == 0) out[j] = bm + __logf(bs) - lse_all;
  }
}

// q_first [B, NI, S/64, 64] bf16 (the first query of every block), ki [B, S, 64] bf16, w_first [B, S/64, NI] fp32 -> lp_blk [B, S/64, S/64]
at::Tensor qsa_first_query_lp(const at::Tensor& q_first, const at::Tensor& ki, const at::Tensor& w_first, double scale) {
  TORCH_CHECK(q_first.is_cuda() && q_first.scalar_type() == at::kBFloat16 && q_first.dim() == 4 && q_first.is_contiguous() && q_first.size(3) == 64,
              "qsa_first_query_lp: contiguous bf16 queries [B,NI,nb,64] required");
  TORCH_CHECK(ki.scalar_type() == at::kBFloat16 && ki.dim() == 3 && ki.is_contiguous() && ki.size(2) == 64 && ki.size(0) == q_first.size(0),
              "qsa_first_query_lp: contiguous bf16 keys [B,S,64] required");
  const int B = q_first.size(0), NI = q_first.size(1), nb = q_first.size(2), S = ki.size(1);
  TORCH_CHECK(NI <= QF_HEADS_MAX && S == 64 * nb && S <= 8192 && w_first.scalar_type() == at::kFloat && w_first.is_contiguous() && w_first.numel() == (int64_t)B * nb * NI,
              "qsa_first_query_lp: at most 4 heads, S = 64 nb <= 8192, fp32 weights [B,nb,NI]");
  const c10::cuda::CUDAGuard guard(q_first.device());
  auto lp = at::empty({B, nb, nb}, q_first.options().dtype(at::kFloat));
  const int smem = (QF_HEADS_MAX * 64 + 4 + 8 + S) * 4;
  qsa_first_query_lp_kernel<<<dim3(nb, B), QF_THREADS, smem, at::cuda::getCurrentCUDAStream()>>>(
      (const __nv_bfloat16*)q_first.data_ptr(), (const __nv_bfloat16*)ki.data_ptr(), w_first.data_ptr<float>(), lp.data_ptr<float>(), S, NI, (float)scale);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return lp;
}

}  // namespace q38
