// mHC (manifold hyper-connections): the 4-branch fp32 residual stream X[T,4,h] around every sub-layer.
//
// Forward of one sub-layer, given L_raw = X_flat . A^T (a tensor-core GEMM done by the caller):
//   mhc_coef_fwd   one warp per token: inv = rsqrt(mean(X^2)+1e-6); z = tanh(B (inv L_raw)); pre/post/res coefficients
//                  (Sinkhorn on the 4x4 residual mix, one matrix entry per lane); xin = sum_n pre_n X_n; then the
//                  sub-layer's zero-centred RMSNorm, written as bf16/fp32 -> the GEMM input.  X is read once from HBM.
//   mhc_post_fwd   X'_m = sum_n res[m,n] X_n + post_m y          (one pass over X, one write of X')
// Backward:
//   mhc_post_bwd   dy = sum_m post_m dX'_m; dpost_m = <dX'_m, y>; dres[m,n] = <dX'_m, X_n>
//   mhc_pre_bwd_a  norm backward, dpre, coefficient/Sinkhorn/tanh backward -> dL_raw, the scalar c1 of the rms path,
//                  dxin, and the parameter gradients (B, biases, alphas, norm weight)
//   mhc_pre_bwd_c  dX_n = G_n + c1 X_n + pre_n dxin + sum_m res[m,n] dX'_m   with G = dL_raw . A from a GEMM
// Coefficient row layout: [0,4) pre, [4,8) post, [8,24) res (row m, column n).  n_branch is fixed at 4.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"
#include "host.h"

namespace q38 {

constexpr int NB = 4, NCOEF = 24, MAX_SINKHORN = 32, WARPS = 8;

struct MhcParams {
  const float* Bw;      // [24, r]
  const float* b_pre;   // [4]
  const float* b_post;  // [4]
  const float* b_res;   // [16]
  const float* alphas;  // [3]
};

// Sinkhorn forward on lanes 0..15 (lane = 4 m + n).  Stores every normalised iterate and divisor for the backward.
__device__ __forceinline__ float sinkhorn_fwd(float logit, int iters, float* Y, float* S, bool keep) {
  float mx = logit;
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0x0000ffffu, mx, o));
  float p = __expf(logit - mx);
  for (int it = 0; it < iters; ++it) {
    float s = p + __shfl_xor_sync(0x0000ffffu, p, 1);
    s += __shfl_xor_sync(0x0000ffffu, s, 2);                  // row sum (over n)
    s = fmaxf(s, 1e-9f);
    p = p / s;
    if (keep) { Y[2 * it] = p; S[2 * it] = s; }
    float c = p + __shfl_xor_sync(0x0000ffffu, p, 4);
    c += __shfl_xor_sync(0x0000ffffu, c, 8);                  // column sum (over m)
    c = fmaxf(c, 1e-9f);
    p = p / c;
    if (keep) { Y[2 * it + 1] = p; S[2 * it + 1] = c; }
  }
  return p;
}

// Forward + backward with a compile-time iteration count: the loops unroll completely, so the saved iterates live in
// registers instead of a per-thread local-memory array.  Lanes 0..15 (lane = 4 m + n); returns d(logit) given d(result).
template <int ITERS>
__device__ __forceinline__ float sinkhorn_fwd_bwd_unrolled(float logit, float dres) {
  float Y[2 * ITERS], S[2 * ITERS];
  float mx = logit;
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0x0000ffffu, mx, o));
  const float p0 = __expf(logit - mx);
  float p = p0;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    float s = p + __shfl_xor_sync(0x0000ffffu, p, 1);
    s += __shfl_xor_sync(0x0000ffffu, s, 2);
    s = fmaxf(s, 1e-9f);
    p = p / s;
    Y[2 * it] = p; S[2 * it] = s;
    float c = p + __shfl_xor_sync(0x0000ffffu, p, 4);
    c += __shfl_xor_sync(0x0000ffffu, c, 8);
    c = fmaxf(c, 1e-9f);
    p = p / c;
    Y[2 * it + 1] = p; S[2 * it + 1] = c;
  }
  float d = dres;
#pragma unroll
  for (int it = ITERS - 1; it >= 0; --it) {
    float t = d * Y[2 * it + 1];
    t += __shfl_xor_sync(0x0000ffffu, t, 4);
    t += __shfl_xor_sync(0x0000ffffu, t, 8);
    d = (d - t) / S[2 * it + 1];
    t = d * Y[2 * it];
    t += __shfl_xor_sync(0x0000ffffu, t, 1);
    t += __shfl_xor_sync(0x0000ffffu, t, 2);
    d = (d - t) / S[2 * it];
  }
  return d * p0;
}

// d(logit) given d(result); y = p / sum(p)  =>  dp = (dy - sum(dy * y)) / s
__device__ __forceinline__ float sinkhorn_bwd(float dres, float logit, int iters, const float* Y, const float* S) {
  float d = dres;
  for (int it = iters - 1; it >= 0; --it) {
    float t = d * Y[2 * it + 1];
    t += __shfl_xor_sync(0x0000ffffu, t, 4);
    t += __shfl_xor_sync(0x0000ffffu, t, 8);
    d = (d - t) / S[2 * it + 1];
    t = d * Y[2 * it];
    t += __shfl_xor_sync(0x0000ffffu, t, 1);
    t += __shfl_xor_sync(0x0000ffffu, t, 2);
    d = (d - t) / S[2 * it];
  }
  // p0 = exp(logit - max): the shift cancels in the normalisations, so d(logit) = d(p0) * p0
  float mx = logit;
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0x0000ffffu, mx, o));
  return d * __expf(logit - mx);
}

template <typename OutT>
__global__ void __launch_bounds__(32 * WARPS) mhc_coef_fwd_kernel(const float* __restrict__ X, const float* __restrict__ Lraw, MhcParams P,
                                                                  const float* __restrict__ norm_w, OutT* __restrict__ xout,
                                                                  float* __restrict__ coef, float* __restrict__ zsave,
                                                                  float* __restrict__ inv_save, float* __restrict__ rstd_save, int T, int h,
                                                                  int r, int iters, float norm_eps) {
  extern __shared__ float sm[];
  float* Bs = sm;                               // [24 * r]
  float* xin_s = sm + NCOEF * r;                // [WARPS * h]
  for (int i = threadIdx.x; i < NCOEF * r; i += blockDim.x) Bs[i] = P.Bw[i];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * WARPS + warp;
  if (t >= T) return;
  const float* Xt = X + (size_t)t * NB * h;
  const int n4 = NB * h / 4;
  float ss = 0.f;
  for (int i = lane; i < n4; i += 32) {
    const float4 v = reinterpret_cast<const float4*>(Xt)[i];
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (NB * h) + 1e-6f);
  // z_j for j = lane < 24
  float z = 0.f;
  if (lane < NCOEF) {
    const float* Lt = Lraw + (size_t)t * r;
    float acc = 0.f;
    for (int i = 0; i < r; ++i) acc += Bs[lane * r + i] * Lt[i];
    z = tanhf(acc * inv);
    zsave[(size_t)t * NCOEF + lane] = z;
  }
  // coefficients: lanes 0..3 pre, 4..7 post; residual logits are moved to lanes 0..15 for the Sinkhorn
  float c = 0.f;
  if (lane < 4) c = sigmoidf_(P.b_pre[lane] + P.alphas[0] * z);
  else if (lane < 8) c = 2.f * sigmoidf_(P.b_post[lane - 4] + P.alphas[1] * z);
  const float zr = __shfl_sync(0xffffffffu, z, (lane & 15) + 8);
  float res = 0.f;
  if (lane < 16) {
    const float logit = P.b_res[lane] + P.alphas[2] * zr;
    res = sinkhorn_fwd(logit, iters, nullptr, nullptr, false);
  }
  if (lane < 8) coef[(size_t)t * NCOEF + lane] = c;
  if (lane < 16) coef[(size_t)t * NCOEF + 8 + lane] = res;
  const float p0 = __shfl_sync(0xffffffffu, c, 0), p1 = __shfl_sync(0xffffffffu, c, 1), p2 = __shfl_sync(0xffffffffu, c, 2),
              p3 = __shfl_sync(0xffffffffu, c, 3);
  float* xs = xin_s + warp * h;
  float ss2 = 0.f;
  for (int i = lane; i < h; i += 32) {
    const float v = p0 * Xt[i] + p1 * Xt[h + i] + p2 * Xt[2 * h + i] + p3 * Xt[3 * h + i];
    xs[i] = v;
    ss2 += v * v;
  }
  ss2 = warp_sum(ss2);
  const float rstd = rsqrtf(ss2 / h + norm_eps);
  if (lane == 0) { inv_save[t] = inv; rstd_save[t] = rstd; }
  __syncwarp();
  OutT* xo = xout + (size_t)t * h;
  for (int i = lane; i < h; i += 32) xo[i] = from_float<OutT>(xs[i] * rstd * (1.f + norm_w[i]));
}

// X'_m = sum_n res[m,n] X_n + post_m y, four columns per thread (16-byte accesses; h is a multiple of 4).
template <typename YT>
__global__ void __launch_bounds__(256) mhc_post_fwd_kernel(const float* __restrict__ X, const YT* __restrict__ y,
                                                           const float* __restrict__ coef, float* __restrict__ Xout, int T, int h) {
  const int h4 = h >> 2;
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)T * h4) return;
  const int t = idx / h4, q = idx % h4;
  const float* c = coef + (size_t)t * NCOEF;
  const size_t base = (size_t)t * NB * h + 4 * q;
  float4 x[NB];
#pragma unroll
  for (int n = 0; n < NB; ++n) x[n] = __ldcs(reinterpret_cast<const float4*>(X + base + (size_t)n * h));
  float4 yv;
  if constexpr (sizeof(YT) == 2) {
    const uint2 raw = *reinterpret_cast<const uint2*>(y + (size_t)t * h + 4 * q);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x)), hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    yv = make_float4(lo.x, lo.y, hi.x, hi.y);
  } else {
    yv = *reinterpret_cast<const float4*>(y + (size_t)t * h + 4 * q);
  }
#pragma unroll
  for (int m = 0; m < NB; ++m) {
    const float r0 = c[8 + 4 * m], r1 = c[8 + 4 * m + 1], r2 = c[8 + 4 * m + 2], r3 = c[8 + 4 * m + 3], pm = c[4 + m];
    float4 o;
    o.x = r0 * x[0].x + r1 * x[1].x + r2 * x[2].x + r3 * x[3].x + pm * yv.x;
    o.y = r0 * x[0].y + r1 * x[1].y + r2 * x[2].y + r3 * x[3].y + pm * yv.y;
    o.z = r0 * x[0].z + r1 * x[1].z + r2 * x[2].z + r3 * x[3].z + pm * yv.z;
    o.w = r0 * x[0].w + r1 * x[1].w + r2 * x[2].w + r3 * x[3].w + pm * yv.w;
    *reinterpret_cast<float4*>(Xout + base + (size_t)m * h) = o;
  }
}

template <typename YT>
__global__ void __launch_bounds__(32 * WARPS) mhc_post_bwd_kernel(const float* __restrict__ dXo, const float* __restrict__ X,
                                                                  const YT* __restrict__ y, const float* __restrict__ coef,
                                                                  YT* __restrict__ dy, float* __restrict__ dcoef, int T, int h) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * WARPS + warp;
  if (t >= T) return;
  const float* c = coef + (size_t)t * NCOEF;
  const float q0 = c[4], q1 = c[5], q2 = c[6], q3 = c[7];
  const float* D = dXo + (size_t)t * NB * h;
  const float* Xt = X + (size_t)t * NB * h;
  float dpost[NB] = {0.f, 0.f, 0.f, 0.f};
  float dres[16];
#pragma unroll
  for (int k = 0; k < 16; ++k) dres[k] = 0.f;
  for (int i = lane; i < h; i += 32) {
    const float d[NB] = {D[i], D[h + i], D[2 * h + i], D[3 * h + i]};
    const float x[NB] = {Xt[i], Xt[h + i], Xt[2 * h + i], Xt[3 * h + i]};
    const float yv = to_float(y[(size_t)t * h + i]);
    dy[(size_t)t * h + i] = from_float<YT>(q0 * d[0] + q1 * d[1] + q2 * d[2] + q3 * d[3]);
#pragma unroll
    for (int m = 0; m < NB; ++m) {
      dpost[m] += d[m] * yv;
#pragma unroll
      for (int n = 0; n < NB; ++n) dres[4 * m + n] += d[m] * x[n];
    }
  }
#pragma unroll
  for (int m = 0; m < NB; ++m) dpost[m] = warp_sum(dpost[m]);
#pragma unroll
  for (int k = 0; k < 16; ++k) dres[k] = warp_sum(dres[k]);
  if (lane == 0) {
    float* o = dcoef + (size_t)t * NCOEF;
#pragma unroll
    for (int m = 0; m < NB; ++m) { o[m] = 0.f; o[4 + m] = dpost[m]; }
#pragma unroll
    for (int k = 0; k < 16; ++k) o[8 + k] = dres[k];
  }
}

// Part A of the pre backward.  dcoef holds dpost/dres from mhc_post_bwd in its [4,24) entries; this kernel fills [0,4).
template <typename GT>
__global__ void __launch_bounds__(32 * WARPS) mhc_pre_bwd_a_kernel(const GT* __restrict__ dxout, const float* __restrict__ X,
                                                                   const float* __restrict__ Lraw, MhcParams P, const float* __restrict__ norm_w,
                                                                   const float* __restrict__ coef, const float* __restrict__ zsave,
                                                                   const float* __restrict__ inv_save, const float* __restrict__ rstd_save,
                                                                   float* __restrict__ dcoef, float* __restrict__ dLraw, float* __restrict__ c1_out,
                                                                   float* __restrict__ dxin_out, float* __restrict__ dBw, float* __restrict__ dbias,
                                                                   float* __restrict__ dnorm_w, int T, int h, int r, int iters) {
  extern __shared__ float sm[];
  float* Bs = sm;                      // [24 * r]
  float* dB_s = Bs + NCOEF * r;        // [24 * r]   CTA-level accumulation of dB
  float* dnw_s = dB_s + NCOEF * r;     // [h]        CTA-level accumulation of d(norm weight)
  float* dbias_s = dnw_s + h;          // [27]       b_pre(4) b_post(4) b_res(16) alphas(3)
  float* xin_s = dbias_s + 32;         // [WARPS * h]
  float* dl_s = xin_s + WARPS * h;     // [WARPS * 24]
  for (int i = threadIdx.x; i < NCOEF * r; i += blockDim.x) { Bs[i] = P.Bw[i]; dB_s[i] = 0.f; }
  for (int i = threadIdx.x; i < h; i += blockDim.x) dnw_s[i] = 0.f;
  if (threadIdx.x < 32) dbias_s[threadIdx.x] = 0.f;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * WARPS + warp;
  if (t < T) {
    const float* Xt = X + (size_t)t * NB * h;
    const float* c = coef + (size_t)t * NCOEF;
    const float p[NB] = {c[0], c[1], c[2], c[3]};
    const float rstd = rstd_save[t], inv = inv_save[t];
    float* xs = xin_s + warp * h;
    // norm backward: g = dx (1 + w); dxin = rstd (g - xhat mean(g xhat))
    float dot = 0.f;
    for (int i = lane; i < h; i += 32) {
      const float xin = p[0] * Xt[i] + p[1] * Xt[h + i] + p[2] * Xt[2 * h + i] + p[3] * Xt[3 * h + i];
      const float xhat = xin * rstd, g = to_float(dxout[(size_t)t * h + i]);
      xs[i] = xhat;
      dot += g * (1.f + norm_w[i]) * xhat;
      atomicAdd(&dnw_s[i], g * xhat);
    }
    dot = warp_sum(dot) / h;
    float dpre[NB] = {0.f, 0.f, 0.f, 0.f};
    for (int i = lane; i < h; i += 32) {
      const float g = to_float(dxout[(size_t)t * h + i]) * (1.f + norm_w[i]);
      const float dxin = rstd * (g - xs[i] * dot);
      dxin_out[(size_t)t * h + i] = dxin;
#pragma unroll
      for (int n = 0; n < NB; ++n) dpre[n] += dxin * Xt[n * h + i];
    }
#pragma unroll
    for (int n = 0; n < NB; ++n) dpre[n] = warp_sum(dpre[n]);
    // coefficient backward, lane j < 24 owns logit j
    const float z = lane < NCOEF ? zsave[(size_t)t * NCOEF + lane] : 0.f;
    float dlogit = 0.f;
    if (lane < 4) {
      const float dp = lane == 0 ? dpre[0] : lane == 1 ? dpre[1] : lane == 2 ? dpre[2] : dpre[3];
      dcoef[(size_t)t * NCOEF + lane] = dp;
      dlogit = dp * c[lane] * (1.f - c[lane]);
    } else if (lane < 8) {
      const float q = c[lane];                             // post = 2 sigmoid  =>  d/dlogit = q (1 - q/2)
      dlogit = dcoef[(size_t)t * NCOEF + lane] * q * (1.f - 0.5f * q);
    }
    // Sinkhorn backward on lanes 0..15, result moved to lanes 8..23
    float dres_logit = 0.f;
    {
      const float zr = __shfl_sync(0xffffffffu, z, (lane & 15) + 8);
      float Y[2 * MAX_SINKHORN], S[2 * MAX_SINKHORN];
      if (lane < 16) {
        const float logit = P.b_res[lane] + P.alphas[2] * zr;
        sinkhorn_fwd(logit, iters, Y, S, true);
        dres_logit = sinkhorn_bwd(dcoef[(size_t)t * NCOEF + 8 + lane], logit, iters, Y, S);
      }
    }
    const float moved = __shfl_sync(0xffffffffu, dres_logit, (lane + 24) & 31);   // lane j gets lane j-8
    if (lane >= 8 && lane < NCOEF) dlogit = moved;
    // biases and alphas
    if (lane < NCOEF) {
      atomicAdd(&dbias_s[lane], dlogit);
      const int a = lane < 4 ? 0 : lane < 8 ? 1 : 2;
      atomicAdd(&dbias_s[24 + a], dlogit * z);
    }
    const float alpha = lane < 4 ? P.alphas[0] : lane < 8 ? P.alphas[1] : P.alphas[2];
    const float dlin = lane < NCOEF ? dlogit * alpha * (1.f - z * z) : 0.f;       // grad of B (inv L_raw) row j
    float* dls = dl_s + warp * NCOEF;
    if (lane < NCOEF) dls[lane] = dlin;
    __syncwarp();
    // dB[j,i] += dlin_j * inv * Lraw_i ;  dL_i = sum_j B[j,i] dlin_j ;  dLraw_i = inv dL_i ;  dinv = sum_i dL_i Lraw_i
    const float* Lt = Lraw + (size_t)t * r;
    float dinv = 0.f;
    for (int i = lane; i < r; i += 32) {
      const float li = Lt[i];
      float dl = 0.f;
#pragma unroll
      for (int j = 0; j < NCOEF; ++j) {
        dl += Bs[j * r + i] * dls[j];
        atomicAdd(&dB_s[j * r + i], dls[j] * inv * li);
      }
      dLraw[(size_t)t * r + i] = inv * dl;
      dinv += dl * li;
    }
    dinv = warp_sum(dinv);
    if (lane == 0) c1_out[t] = -dinv * inv * inv * inv / (NB * h);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < NCOEF * r; i += blockDim.x) atomicAdd(&dBw[i], dB_s[i]);
  for (int i = threadIdx.x; i < h; i += blockDim.x) atomicAdd(&dnorm_w[i], dnw_s[i]);
  if (threadIdx.x < 27) atomicAdd(&dbias[threadIdx.x], dbias_s[threadIdx.x]);
}

// dX_n = G_n + c1 X_n + pre_n dxin + sum_m res[m,n] dX'_m, four columns per thread.  G (= dL_raw . A from the GEMM) may be bf16:
// it is the low-rank correction to the stream gradient, whose other terms stay fp32.
template <typename GT>
__global__ void __launch_bounds__(256) mhc_pre_bwd_c_kernel(float* __restrict__ dX, const GT* __restrict__ G, const float* __restrict__ dXo,
                                                            const float* __restrict__ X, const float* __restrict__ dxin, const float* __restrict__ coef,
                                                            const float* __restrict__ c1, int T, int h) {
  const int h4 = h >> 2;
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)T * h4) return;
  const int t = idx / h4, q = idx % h4;
  const float* c = coef + (size_t)t * NCOEF;
  const size_t base = (size_t)t * NB * h + 4 * q;
  float4 d[NB];
#pragma unroll
  for (int m = 0; m < NB; ++m) d[m] = __ldcs(reinterpret_cast<const float4*>(dXo + base + (size_t)m * h));
  const float k1 = c1[t];
  const float4 di = *reinterpret_cast<const float4*>(dxin + (size_t)t * h + 4 * q);
#pragma unroll
  for (int n = 0; n < NB; ++n) {
    const size_t o = base + (size_t)n * h;
    const float4 x = __ldcs(reinterpret_cast<const float4*>(X + o));
    float4 g;
    if constexpr (sizeof(GT) == 2) {
      const uint2 raw = *reinterpret_cast<const uint2*>(G + o);
      const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x)), hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
      g = make_float4(lo.x, lo.y, hi.x, hi.y);
    } else {
      g = *reinterpret_cast<const float4*>(G + o);
    }
    const float pn = c[n], r0 = c[8 + n], r1 = c[12 + n], r2 = c[16 + n], r3 = c[20 + n];
    float4 out;
    out.x = g.x + k1 * x.x + pn * di.x + r0 * d[0].x + r1 * d[1].x + r2 * d[2].x + r3 * d[3].x;
    out.y = g.y + k1 * x.y + pn * di.y + r0 * d[0].y + r1 * d[1].y + r2 * d[2].y + r3 * d[3].y;
    out.z = g.z + k1 * x.z + pn * di.z + r0 * d[0].z + r1 * d[1].z + r2 * d[2].z + r3 * d[3].z;
    out.w = g.w + k1 * x.w + pn * di.w + r0 * d[0].w + r1 * d[1].w + r2 * d[2].w + r3 * d[3].w;
    *reinterpret_cast<float4*>(dX + o) = out;
  }
}

// ---- row-in-registers variants ---------------------------------------------------------------------------------------
// One warp per token, looping over tokens.  A lane owns the float4 columns q = lane + 32 jj (jj < NQ) of all four branches,
// so the token's 4 x h row is loaded once with 4 NQ independent 16-byte loads per lane and every later use (mean square,
// branch mix, gradient dot products) comes from registers.  B is kept in shared memory with a padded row (r + 1 words) so
// that lane j reading row j is conflict free.  Used when h / 4 <= 32 NQ and r <= 96.
constexpr int RW = 4;      // warps per CTA

template <typename T> __device__ __forceinline__ float4 load4(const T* p);
template <> __device__ __forceinline__ float4 load4<float>(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
template <> __device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p));
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x)), b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
}
__device__ __forceinline__ float dot4(float4 a, float4 b) { return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w; }

template <int NQ>
__device__ __forceinline__ void load_row(const float* __restrict__ Xt, int h, int h4, int lane, float4 (&x)[NB][NQ]) {
#pragma unroll
  for (int jj = 0; jj < NQ; ++jj) {
    const int q = lane + 32 * jj;
#pragma unroll
    for (int n = 0; n < NB; ++n) x[n][jj] = q < h4 ? __ldcs(reinterpret_cast<const float4*>(Xt + n * h) + q) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// value of element i (< 96) of a vector spread as l0 = v[lane], l1 = v[lane + 32], l2 = v[lane + 64]
__device__ __forceinline__ float spread_get(float l0, float l1, float l2, int i) {
  return __shfl_sync(0xffffffffu, i < 32 ? l0 : (i < 64 ? l1 : l2), i & 31);
}

template <typename OutT, int NQ>
__global__ void __launch_bounds__(32 * RW, 4) mhc_coef_fwd_rows_kernel(const float* __restrict__ X, const float* __restrict__ Lraw, MhcParams P,
                                                                       const float* __restrict__ norm_w, OutT* __restrict__ xout,
                                                                       float* __restrict__ coef, float* __restrict__ zsave,
                                                                       float* __restrict__ inv_save, float* __restrict__ rstd_save, int T, int h,
                                                                       int r, int iters, float norm_eps) {
  extern __shared__ float sm[];
  const int RP = r + 1;
  float* Bs = sm;                               // [24][r + 1]
  for (int i = threadIdx.x; i < NCOEF * r; i += blockDim.x) Bs[(i / r) * RP + i % r] = P.Bw[i];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, h4 = h >> 2;
  const float* Brow = Bs + min(lane, NCOEF - 1) * RP;
  for (int t = blockIdx.x * RW + warp; t < T; t += gridDim.x * RW) {
    const float* Xt = X + (size_t)t * NB * h;
    float4 x[NB][NQ];
    load_row<NQ>(Xt, h, h4, lane, x);
    const float* Lt = Lraw + (size_t)t * r;
    const float l0 = lane < r ? Lt[lane] : 0.f, l1 = lane + 32 < r ? Lt[lane + 32] : 0.f, l2 = lane + 64 < r ? Lt[lane + 64] : 0.f;
    float ss = 0.f;
#pragma unroll
    for (int jj = 0; jj < NQ; ++jj)
#pragma unroll
      for (int n = 0; n < NB; ++n) ss += dot4(x[n][jj], x[n][jj]);
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (NB * h) + 1e-6f);
    float acc = 0.f;
    for (int i = 0; i < r; ++i) acc += Brow[i] * spread_get(l0, l1, l2, i);
    float z = 0.f;
    if (lane < NCOEF) {
      z = tanhf(acc * inv);
      zsave[(size_t)t * NCOEF + lane] = z;
    }
    float c = 0.f;
    if (lane < 4) c = sigmoidf_(P.b_pre[lane] + P.alphas[0] * z);
    else if (lane < 8) c = 2.f * sigmoidf_(P.b_post[lane - 4] + P.alphas[1] * z);
    const float zr = __shfl_sync(0xffffffffu, z, (lane & 15) + 8);
    float res = 0.f;
    if (lane < 16) res = sinkhorn_fwd(P.b_res[lane] + P.alphas[2] * zr, iters, nullptr, nullptr, false);
    if (lane < 8) coef[(size_t)t * NCOEF + lane] = c;
    if (lane < 16) coef[(size_t)t * NCOEF + 8 + lane] = res;
    const float p0 = __shfl_sync(0xffffffffu, c, 0), p1 = __shfl_sync(0xffffffffu, c, 1), p2 = __shfl_sync(0xffffffffu, c, 2),
                p3 = __shfl_sync(0xffffffffu, c, 3);
    float4 v[NQ];
    float ss2 = 0.f;
#pragma unroll
    for (int jj = 0; jj < NQ; ++jj) {
      v[jj] = make_float4(p0 * x[0][jj].x + p1 * x[1][jj].x + p2 * x[2][jj].x + p3 * x[3][jj].x,
                          p0 * x[0][jj].y + p1 * x[1][jj].y + p2 * x[2][jj].y + p3 * x[3][jj].y,
                          p0 * x[0][jj].z + p1 * x[1][jj].z + p2 * x[2][jj].z + p3 * x[3][jj].z,
                          p0 * x[0][jj].w + p1 * x[1][jj].w + p2 * x[2][jj].w + p3 * x[3][jj].w);
      ss2 += dot4(v[jj], v[jj]);
    }
    ss2 = warp_sum(ss2);
    const float rstd = rsqrtf(ss2 / h + norm_eps);
    if (lane == 0) { inv_save[t] = inv; rstd_save[t] = rstd; }
    OutT* xo = xout + (size_t)t * h;
#pragma unroll
    for (int jj = 0; jj < NQ; ++jj) {
      const int q = lane + 32 * jj;
      if (q < h4) {
        const float4 nw = load4<float>(norm_w + 4 * q);
        store4(xo + 4 * q, make_float4(v[jj].x * rstd * (1.f + nw.x), v[jj].y * rstd * (1.f + nw.y), v[jj].z * rstd * (1.f + nw.z), v[jj].w * rstd * (1.f + nw.w)));
      }
    }
  }
}

// Part A of the pre backward on register rows, in two kernels.
//   mhc_pre_bwd_rows_kernel   streaming part: norm backward (dxin), dpre_n = <dxin, X_n> (written to dcoef[0,4)), d(norm weight)
//                             accumulated per lane across the warp's tokens.  No long dependent chain, so the loads of the next
//                             token are issued while the current one is reduced.
//   mhc_coef_bwd_kernel       per-token coefficient backward on [T,24] data only (sigmoid / Sinkhorn / tanh backward, dL_raw,
//                             c1, bias and alpha gradients); it writes dlin [T,24], and dB = dlin^T (inv L_raw) is formed by
//                             mhc_dB_kernel.  Few registers, so enough warps are resident to hide the Sinkhorn chain.
template <typename GT, int NQ>
__global__ void __launch_bounds__(32 * RW, 3) mhc_pre_bwd_rows_kernel(const GT* __restrict__ dxout, const float* __restrict__ X,
                                                                      const float* __restrict__ norm_w, const float* __restrict__ coef,
                                                                      const float* __restrict__ rstd_save, float* __restrict__ dcoef,
                                                                      float* __restrict__ dxin_out, float* __restrict__ dnorm_w,
                                                                      __nv_bfloat16* __restrict__ xbf, int T, int h) {
  extern __shared__ float sm[];
  float* dnw_s = sm;                   // [h]
  for (int i = threadIdx.x; i < h; i += blockDim.x) dnw_s[i] = 0.f;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, h4 = h >> 2;
  float4 dnw[NQ];
#pragma unroll
  for (int jj = 0; jj < NQ; ++jj) dnw[jj] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int t = blockIdx.x * RW + warp; t < T; t += gridDim.x * RW) {
    const float* Xt = X + (size_t)t * NB * h;
    float4 x[NB][NQ];
    load_row<NQ>(Xt, h, h4, lane, x);
    // bf16 copy of the row: the operand of the weight-gradient GEMM dA = dL^T X (saves a separate conversion pass over X)
#pragma unroll
    for (int jj = 0; jj < NQ; ++jj) {
      const int q = lane + 32 * jj;
      if (q < h4) {
#pragma unroll
        for (int n = 0; n < NB; ++n) store4(xbf + ((size_t)t * NB + n) * h + 4 * q, x[n][jj]);
      }
    }
    const float cv = lane < 4 ? coef[(size_t)t * NCOEF + lane] : 0.f;
    const float p0 = __shfl_sync(0xffffffffu, cv, 0), p1 = __shfl_sync(0xffffffffu, cv, 1), p2 = __shfl_sync(0xffffffffu, cv, 2),
                p3 = __shfl_sync(0xffffffffu, cv, 3);
    const float rstd = rstd_save[t];
    const GT* gt = dxout + (size_t)t * h;
    float4 g[NQ], xh[NQ];          // dxout (1 + w), normalised sub-layer input
    float dot = 0.f;
#pragma unroll
    for (int jj = 0; jj < NQ; ++jj) {
      const int q = lane + 32 * jj;
      g[jj] = make_float4(0.f, 0.f, 0.f, 0.f);
      xh[jj] = g[jj];
      if (q < h4) {
        const float4 gv = load4<GT>(gt + 4 * q), nw = load4<float>(norm_w + 4 * q);
        xh[jj] = make_float4(rstd * (p0 * x[0][jj].x + p1 * x[1][jj].x + p2 * x[2][jj].x + p3 * x[3][jj].x),
                             rstd * (p0 * x[0][jj].y + p1 * x[1][jj].y + p2 * x[2][jj].y + p3 * x[3][jj].y),
                             rstd * (p0 * x[0][jj].z + p1 * x[1][jj].z + p2 * x[2][jj].z + p3 * x[3][jj].z),
                             rstd * (p0 * x[0][jj].w + p1 * x[1][jj].w + p2 * x[2][jj].w + p3 * x[3][jj].w));
        dnw[jj].x += gv.x * xh[jj].x; dnw[jj].y += gv.y * xh[jj].y; dnw[jj].z += gv.z * xh[jj].z; dnw[jj].w += gv.w * xh[jj].w;
        g[jj] = make_float4(gv.x * (1.f + nw.x), gv.y * (1.f + nw.y), gv.z * (1.f + nw.z), gv.w * (1.f + nw.w));
        dot += dot4(g[jj], xh[jj]);
      }
    }
    dot = warp_sum(dot) / h;
    float dpre[NB] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int jj = 0; jj < NQ; ++jj) {
      const int q = lane + 32 * jj;
      if (q < h4) {
        const float4 dxin = make_float4(rstd * (g[jj].x - xh[jj].x * dot), rstd * (g[jj].y - xh[jj].y * dot), rstd * (g[jj].z - xh[jj].z * dot),
                                        rstd * (g[jj].w - xh[jj].w * dot));
        store4(dxin_out + (size_t)t * h + 4 * q, dxin);
#pragma unroll
        for (int n = 0; n < NB; ++n) dpre[n] += dot4(dxin, x[n][jj]);
      }
    }
#pragma unroll
    for (int n = 0; n < NB; ++n) dpre[n] = warp_sum(dpre[n]);
    if (lane < 4) dcoef[(size_t)t * NCOEF + lane] = lane == 0 ? dpre[0] : lane == 1 ? dpre[1] : lane == 2 ? dpre[2] : dpre[3];
  }
#pragma unroll
  for (int jj = 0; jj < NQ; ++jj) {
    const int q = lane + 32 * jj;
    if (q < h4) {
      atomicAdd(&dnw_s[4 * q], dnw[jj].x); atomicAdd(&dnw_s[4 * q + 1], dnw[jj].y);
      atomicAdd(&dnw_s[4 * q + 2], dnw[jj].z); atomicAdd(&dnw_s[4 * q + 3], dnw[jj].w);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < h; i += blockDim.x) atomicAdd(&dnorm_w[i], dnw_s[i]);
}

constexpr int CW = 8;      // warps per CTA of the coefficient backward
__global__ void __launch_bounds__(32 * CW) mhc_coef_bwd_kernel(const float* __restrict__ Lraw, MhcParams P, const float* __restrict__ coef,
                                                               const float* __restrict__ zsave, const float* __restrict__ inv_save,
                                                               const float* __restrict__ dcoef, float* __restrict__ dLraw, float* __restrict__ c1_out,
                                                               float* __restrict__ dlin_out, float* __restrict__ dbias, int T, int h, int r, int iters) {
  extern __shared__ float sm[];
  const int RP = r + 1;
  float* Bs = sm;                      // [24][r + 1]
  float* dbias_s = Bs + NCOEF * RP;    // [32]
  for (int i = threadIdx.x; i < NCOEF * r; i += blockDim.x) Bs[(i / r) * RP + i % r] = P.Bw[i];
  if (threadIdx.x < 32) dbias_s[threadIdx.x] = 0.f;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float db = 0.f, da = 0.f;
  const float alpha = lane < 4 ? P.alphas[0] : lane < 8 ? P.alphas[1] : P.alphas[2];
  for (int t = blockIdx.x * CW + warp; t < T; t += gridDim.x * CW) {
    const float cv = lane < NCOEF ? coef[(size_t)t * NCOEF + lane] : 0.f;
    const float dc = lane < NCOEF ? dcoef[(size_t)t * NCOEF + lane] : 0.f;
    const float z = lane < NCOEF ? zsave[(size_t)t * NCOEF + lane] : 0.f;
    const float inv = inv_save[t];
    float dlogit = 0.f;
    if (lane < 4) dlogit = dc * cv * (1.f - cv);
    else if (lane < 8) dlogit = dc * cv * (1.f - 0.5f * cv);                  // post = 2 sigmoid
    float dres_logit = 0.f;
    {
      const float zr = __shfl_sync(0xffffffffu, z, (lane & 15) + 8);
      const float dres = __shfl_sync(0xffffffffu, dc, (lane & 15) + 8);
      if (lane < 16) {
        const float logit = P.b_res[lane] + P.alphas[2] * zr;
        if (iters == 20) {                                  // the presets' iteration count: register-resident variant
          dres_logit = sinkhorn_fwd_bwd_unrolled<20>(logit, dres);
        } else {
          float Y[2 * MAX_SINKHORN], S[2 * MAX_SINKHORN];
          sinkhorn_fwd(logit, iters, Y, S, true);
          dres_logit = sinkhorn_bwd(dres, logit, iters, Y, S);
        }
      }
    }
    const float moved = __shfl_sync(0xffffffffu, dres_logit, (lane + 24) & 31);   // lane j gets lane j - 8
    if (lane >= 8 && lane < NCOEF) dlogit = moved;
    if (lane < NCOEF) { db += dlogit; da += dlogit * z; }
    const float dlin = lane < NCOEF ? dlogit * alpha * (1.f - z * z) : 0.f;
    if (lane < NCOEF) dlin_out[(size_t)t * NCOEF + lane] = dlin;
    // dL_i = sum_j B[j,i] dlin_j ;  dLraw_i = inv dL_i ;  dinv = sum_i dL_i Lraw_i
    const float* Lt = Lraw + (size_t)t * r;
    const int i0 = min(lane, r - 1), i1 = min(lane + 32, r - 1), i2 = min(lane + 64, r - 1);
    float dl0 = 0.f, dl1 = 0.f, dl2 = 0.f;
#pragma unroll
    for (int j = 0; j < NCOEF; ++j) {
      const float dj = __shfl_sync(0xffffffffu, dlin, j);
      dl0 += Bs[j * RP + i0] * dj;
      dl1 += Bs[j * RP + i1] * dj;
      dl2 += Bs[j * RP + i2] * dj;
    }
    float dinv = 0.f;
    if (lane < r) { dLraw[(size_t)t * r + lane] = inv * dl0; dinv += dl0 * Lt[lane]; }
    if (lane + 32 < r) { dLraw[(size_t)t * r + lane + 32] = inv * dl1; dinv += dl1 * Lt[lane + 32]; }
    if (lane + 64 < r) { dLraw[(size_t)t * r + lane + 64] = inv * dl2; dinv += dl2 * Lt[lane + 64]; }
    dinv = warp_sum(dinv);
    if (lane == 0) c1_out[t] = -dinv * inv * inv * inv / (NB * h);
  }
  if (lane < NCOEF) {
    atomicAdd(&dbias_s[lane], db);
    atomicAdd(&dbias_s[24 + (lane < 4 ? 0 : lane < 8 ? 1 : 2)], da);
  }
  __syncthreads();
  if (threadIdx.x < 27) atomicAdd(&dbias[threadIdx.x], dbias_s[threadIdx.x]);
}

// dB[j,i] += sum_t dlin[t,j] inv_t Lraw[t,i] over a slab of tokens per CTA.
constexpr int DB_TOK = 64;
__global__ void __launch_bounds__(256) mhc_dB_kernel(const float* __restrict__ dlin, const float* __restrict__ Lraw, const float* __restrict__ inv,
                                                     float* __restrict__ dBw, int T, int r) {
  extern __shared__ float sm[];
  float* dl_s = sm;                    // [DB_TOK][24]
  float* l_s = sm + DB_TOK * NCOEF;    // [DB_TOK][r]
  const int t0 = blockIdx.x * DB_TOK, nt = min(DB_TOK, T - t0);
  for (int i = threadIdx.x; i < nt * NCOEF; i += blockDim.x) dl_s[i] = dlin[(size_t)t0 * NCOEF + i];
  for (int i = threadIdx.x; i < nt * r; i += blockDim.x) l_s[i] = Lraw[(size_t)t0 * r + i] * inv[t0 + i / r];
  __syncthreads();
  for (int o = threadIdx.x; o < NCOEF * r; o += blockDim.x) {
    const int j = o / r, i = o % r;
    float acc = 0.f;
    for (int t = 0; t < nt; ++t) acc += dl_s[t * NCOEF + j] * l_s[t * r + i];
    atomicAdd(&dBw[o], acc);
  }
}

// ---- host wrappers -------------------------------------------------------------------------------------------------------
static MhcParams params_of(const at::Tensor& Bw, const at::Tensor& b_pre, const at::Tensor& b_post, const at::Tensor& b_res, const at::Tensor& alphas) {
  return MhcParams{Bw.data_ptr<float>(), b_pre.data_ptr<float>(), b_post.data_ptr<float>(), b_res.data_ptr<float>(), alphas.data_ptr<float>()};
}

std::vector<at::Tensor> mhc_coef_fwd(const at::Tensor& X, const at::Tensor& Lraw, const at::Tensor& Bw, const at::Tensor& b_pre,
                                     const at::Tensor& b_post, const at::Tensor& b_res, const at::Tensor& alphas, const at::Tensor& norm_w,
                                     int64_t iters, double norm_eps, bool out_bf16) {
  TORCH_CHECK(X.is_cuda() && X.scalar_type() == at::kFloat && X.is_contiguous() && X.dim() == 3 && X.size(1) == NB, "mhc_coef_fwd: X must be fp32 [T,4,h]");
  TORCH_CHECK(Lraw.scalar_type() == at::kFloat && Lraw.is_contiguous() && iters <= MAX_SINKHORN && Bw.size(0) == NCOEF, "mhc_coef_fwd: bad operands");
  const c10::cuda::CUDAGuard guard(X.device());
  const int T = X.size(0), h = X.size(2), r = Lraw.size(1);
  TORCH_CHECK(h % 4 == 0, "mhc: hidden size must be a multiple of 4");
  auto f32 = X.options();
  auto xout = at::empty({T, h}, f32.dtype(out_bf16 ? at::kBFloat16 : at::kFloat));
  auto coef = at::empty({T, NCOEF}, f32), z = at::empty({T, NCOEF}, f32), inv = at::empty({T}, f32), rstd = at::empty({T}, f32);
  auto stream = at::cuda::getCurrentCUDAStream();
  MhcParams P = params_of(Bw, b_pre, b_post, b_res, alphas);
  const int nq = (h / 4 + 31) / 32;
  if (r <= 96 && nq <= 8) {
    const size_t smem = NCOEF * (r + 1) * sizeof(float);
    const int grid = std::min((T + RW - 1) / RW, 4 * kNumSMs);
#define Q38_ROWS(OutT, NQ) mhc_coef_fwd_rows_kernel<OutT, NQ><<<grid, 32 * RW, smem, stream>>>(X.data_ptr<float>(), Lraw.data_ptr<float>(), P, norm_w.data_ptr<float>(), \
      (OutT*)xout.data_ptr(), coef.data_ptr<float>(), z.data_ptr<float>(), inv.data_ptr<float>(), rstd.data_ptr<float>(), T, h, r, (int)iters, (float)norm_eps)
#define Q38_ROWS_NQ(OutT) switch (nq) { case 1: Q38_ROWS(OutT, 1); break; case 2: Q38_ROWS(OutT, 2); break; case 3: Q38_ROWS(OutT, 3); break; case 4: Q38_ROWS(OutT, 4); break; \
      case 5: Q38_ROWS(OutT, 5); break; case 6: Q38_ROWS(OutT, 6); break; default: Q38_ROWS(OutT, 8); break; }
    if (out_bf16) Q38_ROWS_NQ(__nv_bfloat16) else Q38_ROWS_NQ(float)
#undef Q38_ROWS_NQ
#undef Q38_ROWS
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    count_launch();
    return {xout, coef, z, inv, rstd};
  }
  const size_t smem = (NCOEF * r + WARPS * h) * sizeof(float);
  const int grid = (T + WARPS - 1) / WARPS;
  if (out_bf16) {
    auto k = mhc_coef_fwd_kernel<__nv_bfloat16>;
    C10_CUDA_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    k<<<grid, 32 * WARPS, smem, stream>>>(X.data_ptr<float>(), Lraw.data_ptr<float>(), P, norm_w.data_ptr<float>(), (__nv_bfloat16*)xout.data_ptr(),
                                          coef.data_ptr<float>(), z.data_ptr<float>(), inv.data_ptr<float>(), rstd.data_ptr<float>(), T, h, r, (int)iters, (float)norm_eps);
  } else {
    auto k = mhc_coef_fwd_kernel<float>;
    C10_CUDA_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    k<<<grid, 32 * WARPS, smem, stream>>>(X.data_ptr<float>(), Lraw.data_ptr<float>(), P, norm_w.data_ptr<float>(), xout.data_ptr<float>(),
                                          coef.data_ptr<float>(), z.data_ptr<float>(), inv.data_ptr<float>(), rstd.data_ptr<float>(), T, h, r, (int)iters, (float)norm_eps);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {xout, coef, z, inv, rstd};
}

at::Tensor mhc_post_fwd(const at::Tensor& X, const at::Tensor& y, const at::Tensor& coef) {
  TORCH_CHECK(X.is_cuda() && X.scalar_type() == at::kFloat && X.is_contiguous() && y.is_contiguous() && coef.is_contiguous(), "mhc_post_fwd: bad inputs");
  const c10::cuda::CUDAGuard guard(X.device());
  const int T = X.size(0), h = X.size(2);
  auto out = at::empty_like(X);
  TORCH_CHECK(h % 4 == 0, "mhc_post_fwd: hidden size must be a multiple of 4");
  const size_t n = (size_t)T * (h / 4);
  auto stream = at::cuda::getCurrentCUDAStream();
  if (y.scalar_type() == at::kBFloat16)
    mhc_post_fwd_kernel<__nv_bfloat16><<<(n + 255) / 256, 256, 0, stream>>>(X.data_ptr<float>(), (const __nv_bfloat16*)y.data_ptr(), coef.data_ptr<float>(), out.data_ptr<float>(), T, h);
  else
    mhc_post_fwd_kernel<float><<<(n + 255) / 256, 256, 0, stream>>>(X.data_ptr<float>(), y.data_ptr<float>(), coef.data_ptr<float>(), out.data_ptr<float>(), T, h);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return out;
}

std::vector<at::Tensor> mhc_post_bwd(const at::Tensor& dXo, const at::Tensor& X, const at::Tensor& y, const at::Tensor& coef) {
  TORCH_CHECK(dXo.is_cuda() && dXo.scalar_type() == at::kFloat && dXo.is_contiguous() && X.is_contiguous() && y.is_contiguous(), "mhc_post_bwd: bad inputs");
  const c10::cuda::CUDAGuard guard(X.device());
  const int T = X.size(0), h = X.size(2);
  auto dy = at::empty_like(y);
  auto dcoef = at::empty({T, NCOEF}, X.options());
  auto stream = at::cuda::getCurrentCUDAStream();
  const int grid = (T + WARPS - 1) / WARPS;
  if (y.scalar_type() == at::kBFloat16)
    mhc_post_bwd_kernel<__nv_bfloat16><<<grid, 32 * WARPS, 0, stream>>>(dXo.data_ptr<float>(), X.data_ptr<float>(), (const __nv_bfloat16*)y.data_ptr(),
                                                                        coef.data_ptr<float>(), (__nv_bfloat16*)dy.data_ptr(), dcoef.data_ptr<float>(), T, h);
  else
    mhc_post_bwd_kernel<float><<<grid, 32 * WARPS, 0, stream>>>(dXo.data_ptr<float>(), X.data_ptr<float>(), y.data_ptr<float>(), coef.data_ptr<float>(),
                                                                dy.data_ptr<float>(), dcoef.data_ptr<float>(), T, h);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {dy, dcoef};
}

// Returns {dLraw [T,r], c1 [T], dxin [T,h], dBw [24,r], dbias [27], dnorm_w [h], bf16 copy of X [T,4h]}; dcoef is completed in place.
std::vector<at::Tensor> mhc_pre_bwd_a(const at::Tensor& dxout, const at::Tensor& X, const at::Tensor& Lraw, const at::Tensor& Bw,
                                      const at::Tensor& b_pre, const at::Tensor& b_post, const at::Tensor& b_res, const at::Tensor& alphas,
                                      const at::Tensor& norm_w, const at::Tensor& coef, const at::Tensor& z, const at::Tensor& inv,
                                      const at::Tensor& rstd, at::Tensor& dcoef, int64_t iters) {
  TORCH_CHECK(dxout.is_cuda() && dxout.is_contiguous() && X.is_contiguous() && dcoef.is_contiguous() && iters <= MAX_SINKHORN, "mhc_pre_bwd_a: bad inputs");
  const c10::cuda::CUDAGuard guard(X.device());
  const int T = X.size(0), h = X.size(2), r = Lraw.size(1);
  auto f32 = X.options();
  auto dLraw = at::empty({T, r}, f32), c1 = at::empty({T}, f32), dxin = at::empty({T, h}, f32);
  // one zero fill for the three small accumulators (offsets kept multiples of 4 floats)
  const int64_t n_bw = (int64_t)NCOEF * r, off_bias = (n_bw + 3) / 4 * 4, off_nw = off_bias + 28;
  auto small = at::zeros({off_nw + h}, f32);
  auto dBw = small.narrow(0, 0, n_bw).view({NCOEF, r}), dbias = small.narrow(0, off_bias, 27), dnw = small.narrow(0, off_nw, h);
  auto stream = at::cuda::getCurrentCUDAStream();
  MhcParams P = params_of(Bw, b_pre, b_post, b_res, alphas);
  const int nq = (h / 4 + 31) / 32;
  if (h % 4 == 0 && r <= 96 && nq <= 8) {
    auto dlin = at::empty({T, NCOEF}, f32);
    auto xbf = at::empty({T, NB * h}, f32.dtype(at::kBFloat16));
    const int grid_r = std::min((T + RW - 1) / RW, 3 * kNumSMs);
#define Q38_ROWS(GT, NQ) mhc_pre_bwd_rows_kernel<GT, NQ><<<grid_r, 32 * RW, h * sizeof(float), stream>>>((const GT*)dxout.data_ptr(), X.data_ptr<float>(), \
      norm_w.data_ptr<float>(), coef.data_ptr<float>(), rstd.data_ptr<float>(), dcoef.data_ptr<float>(), dxin.data_ptr<float>(), dnw.data_ptr<float>(), \
      (__nv_bfloat16*)xbf.data_ptr(), T, h)
#define Q38_ROWS_NQ(GT) switch (nq) { case 1: Q38_ROWS(GT, 1); break; case 2: Q38_ROWS(GT, 2); break; case 3: Q38_ROWS(GT, 3); break; case 4: Q38_ROWS(GT, 4); break; \
      case 5: Q38_ROWS(GT, 5); break; case 6: Q38_ROWS(GT, 6); break; default: Q38_ROWS(GT, 8); break; }
    if (dxout.scalar_type() == at::kBFloat16) Q38_ROWS_NQ(__nv_bfloat16) else Q38_ROWS_NQ(float)
#undef Q38_ROWS_NQ
#undef Q38_ROWS
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    count_launch();
    mhc_coef_bwd_kernel<<<std::min((T + CW - 1) / CW, 8 * kNumSMs), 32 * CW, (NCOEF * (r + 1) + 32) * sizeof(float), stream>>>(
        Lraw.data_ptr<float>(), P, coef.data_ptr<float>(), z.data_ptr<float>(), inv.data_ptr<float>(), dcoef.data_ptr<float>(), dLraw.data_ptr<float>(),
        c1.data_ptr<float>(), dlin.data_ptr<float>(), dbias.data_ptr<float>(), T, h, r, (int)iters);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    count_launch();
    mhc_dB_kernel<<<(T + DB_TOK - 1) / DB_TOK, 256, DB_TOK * (NCOEF + r) * sizeof(float), stream>>>(dlin.data_ptr<float>(), Lraw.data_ptr<float>(), inv.data_ptr<float>(),
                                                                                                  dBw.data_ptr<float>(), T, r);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    count_launch();
    return {dLraw, c1, dxin, dBw, dbias, dnw, xbf};
  }
  const size_t smem = (2 * NCOEF * r + h + 32 + WARPS * h + WARPS * NCOEF) * sizeof(float);
  const int grid = (T + WARPS - 1) / WARPS;
#define LAUNCH(GT) { auto k = mhc_pre_bwd_a_kernel<GT>; \
    C10_CUDA_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); \
    k<<<grid, 32 * WARPS, smem, stream>>>((const GT*)dxout.data_ptr(), X.data_ptr<float>(), Lraw.data_ptr<float>(), P, norm_w.data_ptr<float>(), \
      coef.data_ptr<float>(), z.data_ptr<float>(), inv.data_ptr<float>(), rstd.data_ptr<float>(), dcoef.data_ptr<float>(), dLraw.data_ptr<float>(), \
      c1.data_ptr<float>(), dxin.data_ptr<float>(), dBw.data_ptr<float>(), dbias.data_ptr<float>(), dnw.data_ptr<float>(), T, h, r, (int)iters); }
  if (dxout.scalar_type() == at::kBFloat16) LAUNCH(__nv_bfloat16) else LAUNCH(float)
#undef LAUNCH
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {dLraw, c1, dxin, dBw, dbias, dnw, X.reshape({T, NB * h}).to(at::kBFloat16)};
}

// G [T,4,h] bf16 or fp32 -> dX [T,4,h] fp32
at::Tensor mhc_pre_bwd_c(const at::Tensor& G, const at::Tensor& dXo, const at::Tensor& X, const at::Tensor& dxin, const at::Tensor& coef, const at::Tensor& c1) {
  TORCH_CHECK(G.is_cuda() && G.is_contiguous() && dXo.is_contiguous() && X.is_contiguous() && dxin.is_contiguous() && X.size(2) % 4 == 0 &&
                  (G.scalar_type() == at::kFloat || G.scalar_type() == at::kBFloat16) && G.numel() == X.numel() && dXo.scalar_type() == at::kFloat,
              "mhc_pre_bwd_c: bad inputs");
  const c10::cuda::CUDAGuard guard(X.device());
  const int T = X.size(0), h = X.size(2);
  auto dX = at::empty_like(X);
  const size_t n = (size_t)T * (h / 4);
  auto stream = at::cuda::getCurrentCUDAStream();
  if (G.scalar_type() == at::kFloat)
    mhc_pre_bwd_c_kernel<float><<<(n + 255) / 256, 256, 0, stream>>>(dX.data_ptr<float>(), G.data_ptr<float>(), dXo.data_ptr<float>(), X.data_ptr<float>(),
                                                                     dxin.data_ptr<float>(), coef.data_ptr<float>(), c1.data_ptr<float>(), T, h);
  else
    mhc_pre_bwd_c_kernel<__nv_bfloat16><<<(n + 255) / 256, 256, 0, stream>>>(dX.data_ptr<float>(), (const __nv_bfloat16*)G.data_ptr(), dXo.data_ptr<float>(),
                                                                             X.data_ptr<float>(), dxin.data_ptr<float>(), coef.data_ptr<float>(), c1.data_ptr<float>(), T, h);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return dX;
}

}  // namespace q38
