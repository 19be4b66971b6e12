// QSA indexer path: everything that is O(S^2) around block selection, as 64x64-tile kernels on the tensor cores.
//
//   qsa_main_block_stats  dense causal scores of the main attention (all heads), reduced on the fly to a per
//                         (head, query, key block) pair (max, sum exp): the raw material of the distillation target.
//   qsa_indexer_fwd       indexer scores I[t,s] = sum_j w_j(t) relu(q_j(t).k(s)) / 8, reduced to the block log-sum-exp
//                         bLSE[t,b] = log sum_{s in b, s<=t} exp I[t,s].  The [S,S] score matrix never exists in memory.
//   qsa_kl_combine        per token: target P[t,b] (head-averaged block mass), lp_blk[t,b] = bLSE - logsumexp_b bLSE,
//                         KL_t = sum_b P (log P - lp_blk) and the gradient seed (exp(lp_blk) - P).
//   qsa_select            per query block: top-k key blocks from the first query's lp_blk (own block forced, future excluded).
//   qsa_indexer_bwd_q / _k  recompute the score tiles and produce d(q_idx), d(w) / d(k_idx).
//
// Layouts: main q [B,nq,S,64], main k [B,nkv,S,64], indexer q [B,NI,S,64], indexer k [B,S,64] (bf16); w [B,S,NI] fp32.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"
#include "host.h"
#include "mma_tile.cuh"

namespace q38 {

constexpr int NI_MAX = 4;
constexpr float MASKED = -1e9f;

// Row-wise (max, sum exp(x - max)) of a fragment tile; entries with col > row + diag_shift are excluded when `diag`.
__device__ __forceinline__ void frag_row_max_sum(const float (&acc)[8][4], bool diag, int warp, int lane, float (&mx)[2], float (&sm)[2]) {
  const int r0 = 16 * warp + (lane >> 2), cq = 2 * (lane & 3);
#pragma unroll
  for (int hrow = 0; hrow < 2; ++hrow) {
    const int row = r0 + 8 * hrow;
    float m = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int col = 8 * nt + cq + e;
        if (!diag || col <= row) m = fmaxf(m, acc[nt][2 * hrow + e]);
      }
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
    float s = 0.f;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int col = 8 * nt + cq + e;
        if (!diag || col <= row) s += __expf(acc[nt][2 * hrow + e] - m);
      }
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    mx[hrow] = m; sm[hrow] = s;
  }
}

// ---- main attention block statistics -----------------------------------------------------------------------------------
// grid (nb, nq, B).  stats[b, h, t, j] = (max, sumexp) of scale * q_h(t).k(s) over s in block j, s <= t.
__global__ void __launch_bounds__(128) qsa_main_block_stats_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, float2* __restrict__ stats,
                                                                   int S, int nq, int nkv, float scale) {
  extern __shared__ __align__(16) uint8_t smem_bytes[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_bytes);
  bf16* Ks = Qs + TILE_ELEMS;                      // two buffers
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nb = S / 64, i = nb - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;     // late query blocks (longest loops) first
  const bf16* qsrc = q + (((long long)b * nq + h) * S + (long long)i * 64) * 64;
  const bf16* kbase = k + ((long long)b * nkv + h / (nq / nkv)) * S * 64;
  load_tile_async(Qs, qsrc, 64, tid);
  load_tile_async(Ks, kbase, 64, tid);
  cp_async_commit();
  for (int j = 0; j <= i; ++j) {
    const int buf = j & 1;
    if (j < i) { load_tile_async(Ks + (buf ^ 1) * TILE_ELEMS, kbase + (long long)(j + 1) * 4096, 64, tid); cp_async_commit(); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();
    float acc[8][4];
    zero_acc(acc);
    mma64<false, true>(Qs, Ks + buf * TILE_ELEMS, acc, warp, lane);
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) { acc[nt][0] *= scale; acc[nt][1] *= scale; acc[nt][2] *= scale; acc[nt][3] *= scale; }
    float mx[2], sm[2];
    frag_row_max_sum(acc, j == i, warp, lane, mx, sm);
    if ((lane & 3) == 0) {
      const int r0 = 16 * warp + (lane >> 2);
#pragma unroll
      for (int hrow = 0; hrow < 2; ++hrow) {
        const long long t = (long long)i * 64 + r0 + 8 * hrow;
        stats[(((long long)b * nq + h) * S + t) * nb + j] = make_float2(mx[hrow], sm[hrow]);
      }
    }
    __syncthreads();
  }
}

// ---- indexer forward ---------------------------------------------------------------------------------------------------
// grid (nb, B).  blse[b, t, j] for j <= block(t); entries j > block(t) are left untouched (the caller pre-fills them).
__global__ void __launch_bounds__(128) qsa_indexer_fwd_kernel(const bf16* __restrict__ qi, const bf16* __restrict__ ki, const float* __restrict__ wi,
                                                              float* __restrict__ blse, int S, int NI, float scale) {
  extern __shared__ __align__(16) uint8_t smem_bytes[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_bytes);          // NI tiles
  bf16* Ks = Qs + NI_MAX * TILE_ELEMS;                     // two buffers
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Query block i scores key blocks j <= i; late query blocks (most work) are issued first and the key loop of a query block is
  // shared by gridDim.z CTAs (j = z, z + gridDim.z, ...), each writing its own columns of blse.
  const int nb = S / 64, i = nb - 1 - blockIdx.x, b = blockIdx.y, jstep = gridDim.z;
  if ((int)blockIdx.z > i) return;
  for (int hh = 0; hh < NI; ++hh) load_tile_async(Qs + hh * TILE_ELEMS, qi + (((long long)b * NI + hh) * S + (long long)i * 64) * 64, 64, tid);
  const bf16* kbase = ki + (long long)b * S * 64;
  load_tile_async(Ks, kbase + (long long)blockIdx.z * 4096, 64, tid);
  cp_async_commit();
  const int r0 = 16 * warp + (lane >> 2);
  float wrow[2][NI_MAX];
#pragma unroll
  for (int hrow = 0; hrow < 2; ++hrow)
    for (int hh = 0; hh < NI; ++hh) wrow[hrow][hh] = wi[((long long)b * S + (long long)i * 64 + r0 + 8 * hrow) * NI + hh] * scale;
  int buf = 0;
  for (int j = blockIdx.z; j <= i; j += jstep, buf ^= 1) {
    if (j + jstep <= i) { load_tile_async(Ks + (buf ^ 1) * TILE_ELEMS, kbase + (long long)(j + jstep) * 4096, 64, tid); cp_async_commit(); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();
    float score[8][4];
    zero_acc(score);
    for (int hh = 0; hh < NI; ++hh) {
      float acc[8][4];
      zero_acc(acc);
      mma64<false, true>(Qs + hh * TILE_ELEMS, Ks + buf * TILE_ELEMS, acc, warp, lane);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        // the reference rounds q.k to bf16 before the relu (its matmul output dtype)
        score[nt][0] += wrow[0][hh] * fmaxf(bf16_round(acc[nt][0]), 0.f); score[nt][1] += wrow[0][hh] * fmaxf(bf16_round(acc[nt][1]), 0.f);
        score[nt][2] += wrow[1][hh] * fmaxf(bf16_round(acc[nt][2]), 0.f); score[nt][3] += wrow[1][hh] * fmaxf(bf16_round(acc[nt][3]), 0.f);
      }
    }
    float mx[2], sm[2];
    frag_row_max_sum(score, j == i, warp, lane, mx, sm);
    if ((lane & 3) == 0) {
#pragma unroll
      for (int hrow = 0; hrow < 2; ++hrow) {
        const long long t = (long long)i * 64 + r0 + 8 * hrow;
        blse[((long long)b * S + t) * nb + j] = mx[hrow] + __logf(sm[hrow]);
      }
    }
    __syncthreads();
  }
}

// ---- combine: target mass, lp_blk, KL --------------------------------------------------------------------------------
// One warp per token, nb <= 128 (lane-strided).  P, lp_blk, dblse: [B,S,nb] fp32; kl_tok [B*S].
__global__ void __launch_bounds__(256) qsa_kl_combine_kernel(const float2* __restrict__ stats, const float* __restrict__ blse, float* __restrict__ P,
                                                             float* __restrict__ lp_blk, float* __restrict__ kl_tok, float* __restrict__ dblse,
                                                             int B, int S, int nq, int want_target) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long tok = (long long)blockIdx.x * 8 + warp;
  if (tok >= (long long)B * S) return;
  const int b = tok / S, t = tok % S, nb = S / 64, own = t / 64;
  constexpr int PER = 4;                                      // nb <= 128
  float pm[PER] = {0.f, 0.f, 0.f, 0.f};
  if (want_target) {
    for (int h = 0; h < nq; ++h) {
      const float2* st = stats + (((long long)b * nq + h) * S + t) * nb;
      float2 v[PER];
      float m = -INFINITY;
#pragma unroll
      for (int x = 0; x < PER; ++x) { const int j = lane + 32 * x; v[x] = j <= own ? st[j] : make_float2(-INFINITY, 0.f); m = fmaxf(m, v[x].x); }
      m = warp_max(m);
      float tot = 0.f;
#pragma unroll
      for (int x = 0; x < PER; ++x) { v[x].y = v[x].y * __expf(v[x].x - m); tot += v[x].y; }
      tot = warp_sum(tot);
#pragma unroll
      for (int x = 0; x < PER; ++x) pm[x] += v[x].y / tot;
    }
  }
  const float* bl = blse + tok * nb;
  float lv[PER], m = -INFINITY;
#pragma unroll
  for (int x = 0; x < PER; ++x) { const int j = lane + 32 * x; lv[x] = j <= own ? bl[j] : -INFINITY; m = fmaxf(m, lv[x]); }
  m = warp_max(m);
  float tot = 0.f;
#pragma unroll
  for (int x = 0; x < PER; ++x) tot += (lv[x] > -INFINITY) ? __expf(lv[x] - m) : 0.f;
  tot = warp_sum(tot);
  const float lse = m + __logf(tot);
  float kl = 0.f;
#pragma unroll
  for (int x = 0; x < PER; ++x) {
    const int j = lane + 32 * x;
    if (j < nb) {
      const bool causal = j <= own;
      // non-causal blocks: every score is the finite mask value, so their log-probability is hugely negative, not -inf
      const float lp = causal ? lv[x] - lse : MASKED;
      lp_blk[tok * nb + j] = lp;
      if (want_target) {
        const float p = causal ? pm[x] / nq : 0.f;
        P[tok * nb + j] = p;
        if (p > 0.f) kl += p * (__logf(fmaxf(p, 1e-12f)) - lp);
        dblse[tok * nb + j] = causal ? (__expf(lp) - p) : 0.f;
      }
    }
  }
  if (want_target) {
    kl = warp_sum(kl);
    if (lane == 0) kl_tok[tok] = kl;
  }
}

// ---- block selection -----------------------------------------------------------------------------------------------------
// One warp per (batch, query block).  count[b, j] = min(j + 1, k); index[b, j, :k] sorted by decreasing score.
__global__ void __launch_bounds__(256) qsa_select_kernel(const float* __restrict__ lp_blk, long long row_stride, int B, int nb, int K,
                                                         int* __restrict__ count, int* __restrict__ index) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int id = blockIdx.x * 8 + warp;
  if (id >= B * nb) return;
  const int b = id / nb, j = id % nb;
  const float* row = lp_blk + ((long long)b * nb + j) * row_stride;        // first query of block j
  constexpr int PER = 4;
  float v[PER];
#pragma unroll
  for (int x = 0; x < PER; ++x) {
    const int c = lane + 32 * x;
    v[x] = c >= nb ? -3.f : (c > j ? -1.f : (c == j ? 2.f : __expf(row[c])));
  }
  const int k = K < nb ? K : nb;
  for (int r = 0; r < k; ++r) {
    float best = v[0]; int bc = lane;
#pragma unroll
    for (int x = 1; x < PER; ++x) if (v[x] > best) { best = v[x]; bc = lane + 32 * x; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oc = __shfl_xor_sync(0xffffffffu, bc, o);
      if (ob > best || (ob == best && oc < bc)) { best = ob; bc = oc; }
    }
    if (lane == 0) index[((long long)b * nb + j) * k + r] = bc;
    if ((bc & 31) == lane) v[bc >> 5] = -4.f;
  }
  if (lane == 0) count[b * nb + j] = (j + 1 < k) ? j + 1 : k;
}

// ---- indexer backward ------------------------------------------------------------------------------------------------------
// dI[t,s] = dblse[t, blk(s)] * exp(I[t,s] - blse[t, blk(s)]) for s <= t;   I = sum_h w_h relu(S_h) scale
// Score tile of (query block i, key block j): all heads contribute to `score`; relu(S_own) is kept for head `own`.
__device__ __forceinline__ void indexer_score_tile(const bf16* __restrict__ Qs, const bf16* __restrict__ Kt, const float (&wrow)[2][NI_MAX], int NI, int own,
                                                   float (&score)[8][4], float (&sown)[8][4], int warp, int lane) {
  zero_acc(score);
  for (int hh = 0; hh < NI; ++hh) {
    float acc[8][4];
    zero_acc(acc);
    mma64<false, true>(Qs + hh * TILE_ELEMS, Kt, acc, warp, lane);
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float r = fmaxf(bf16_round(acc[nt][e]), 0.f);
        score[nt][e] += (e < 2 ? wrow[0][hh] : wrow[1][hh]) * r;
        if (hh == own) sown[nt][e] = r;
      }
  }
}

__device__ __forceinline__ void indexer_dI_tile(const float (&score)[8][4], const float* __restrict__ blse, const float* __restrict__ dblse, float gscale,
                                                long long row_base, int nb, int j, bool diag, float (&dI)[8][4], int warp, int lane) {
  const int r0 = 16 * warp + (lane >> 2), cq = 2 * (lane & 3);
#pragma unroll
  for (int hrow = 0; hrow < 2; ++hrow) {
    const int row = r0 + 8 * hrow;
    const float bl = blse[(row_base + row) * nb + j], g = dblse[(row_base + row) * nb + j] * gscale;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int col = 8 * nt + cq + e;
        dI[nt][2 * hrow + e] = (!diag || col <= row) ? g * __expf(score[nt][2 * hrow + e] - bl) : 0.f;
      }
  }
}

// Query pass, grid (nb, NI, B): d q_own(t) = sum_s dI w_own scale [S_own > 0] k(s);  d w_own(t) = sum_s dI relu(S_own) scale.
__global__ void __launch_bounds__(128) qsa_indexer_bwd_q_kernel(const bf16* __restrict__ qi, const bf16* __restrict__ ki, const float* __restrict__ wi,
                                                                const float* __restrict__ blse, const float* __restrict__ dblse, float gscale,
                                                                bf16* __restrict__ dqi, float* __restrict__ dwi, int S, int NI, float scale) {
  extern __shared__ __align__(16) uint8_t smem_bytes[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_bytes);
  bf16* Ks = Qs + NI_MAX * TILE_ELEMS;                     // two buffers
  bf16* Ts = Ks + 2 * TILE_ELEMS;                          // dS_own tile (bf16) as A operand
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nb = S / 64, i = nb - 1 - blockIdx.x, own = blockIdx.y, b = blockIdx.z;   // late query blocks (longest loops) first
  for (int hh = 0; hh < NI; ++hh) load_tile_async(Qs + hh * TILE_ELEMS, qi + (((long long)b * NI + hh) * S + (long long)i * 64) * 64, 64, tid);
  const bf16* kbase = ki + (long long)b * S * 64;
  load_tile_async(Ks, kbase, 64, tid);
  cp_async_commit();
  const int r0 = 16 * warp + (lane >> 2);
  float wrow[2][NI_MAX];
#pragma unroll
  for (int hrow = 0; hrow < 2; ++hrow)
#pragma unroll
    for (int hh = 0; hh < NI_MAX; ++hh)
      wrow[hrow][hh] = hh < NI ? wi[((long long)b * S + (long long)i * 64 + r0 + 8 * hrow) * NI + hh] * scale : 0.f;
  const float wown[2] = {wi[((long long)b * S + (long long)i * 64 + r0) * NI + own] * scale, wi[((long long)b * S + (long long)i * 64 + r0 + 8) * NI + own] * scale};
  float dw[2] = {0.f, 0.f};
  float dq[8][4];
  zero_acc(dq);
  for (int j = 0; j <= i; ++j) {
    const int buf = j & 1;
    if (j < i) { load_tile_async(Ks + (buf ^ 1) * TILE_ELEMS, kbase + (long long)(j + 1) * 4096, 64, tid); cp_async_commit(); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();
    const bf16* Kt = Ks + buf * TILE_ELEMS;
    float score[8][4], sown[8][4], dI[8][4];
    indexer_score_tile(Qs, Kt, wrow, NI, own, score, sown, warp, lane);
    indexer_dI_tile(score, blse, dblse, gscale, (long long)b * S + (long long)i * 64, nb, j, j == i, dI, warp, lane);
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        dw[e >> 1] += dI[nt][e] * sown[nt][e] * scale;
        dI[nt][e] = sown[nt][e] > 0.f ? dI[nt][e] * wown[e >> 1] : 0.f;        // dS_own
      }
    acc_to_smem(dI, Ts, warp, lane);
    __syncthreads();
    mma64<false, false>(Ts, Kt, dq, warp, lane);           // dS_own K
    __syncthreads();
  }
  acc_to_global(dq, dqi + (((long long)b * NI + own) * S + (long long)i * 64) * 64, 64, warp, lane);
#pragma unroll
  for (int hrow = 0; hrow < 2; ++hrow) {
    float v = dw[hrow];
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    if ((lane & 3) == 0) dwi[((long long)b * S + (long long)i * 64 + r0 + 8 * hrow) * NI + own] = v;
  }
}

// Key pass, grid (nb, B): d k(s) = sum_{t >= s} sum_h dS_h[t,s] q_h(t), looping over query blocks i >= j.
__global__ void __launch_bounds__(128) qsa_indexer_bwd_k_kernel(const bf16* __restrict__ qi, const bf16* __restrict__ ki, const float* __restrict__ wi,
                                                                const float* __restrict__ blse, const float* __restrict__ dblse, float gscale,
                                                                float* __restrict__ dki, int S, int NI, float scale) {
  extern __shared__ __align__(16) uint8_t smem_bytes[];
  bf16* Ks = reinterpret_cast<bf16*>(smem_bytes);
  bf16* Qs = Ks + TILE_ELEMS;                              // NI tiles of the current query block
  bf16* Ts = Qs + NI_MAX * TILE_ELEMS;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Key block j is scored by every query block i >= j: the loop is shared by gridDim.z CTAs (i = j + z, j + z + gridDim.z, ...)
  // whose partial gradients are added in fp32.
  const int j = blockIdx.x, b = blockIdx.y, nb = S / 64;
  if (j + (int)blockIdx.z >= nb) return;
  load_tile_async(Ks, ki + ((long long)b * S + (long long)j * 64) * 64, 64, tid);
  cp_async_commit();
  const int r0 = 16 * warp + (lane >> 2);
  float dk[8][4];
  zero_acc(dk);
  for (int i = j + blockIdx.z; i < nb; i += gridDim.z) {
    __syncthreads();
    for (int hh = 0; hh < NI; ++hh) load_tile_async(Qs + hh * TILE_ELEMS, qi + (((long long)b * NI + hh) * S + (long long)i * 64) * 64, 64, tid);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    float wrow[2][NI_MAX];
#pragma unroll
    for (int hrow = 0; hrow < 2; ++hrow)
#pragma unroll
      for (int hh = 0; hh < NI_MAX; ++hh)
        wrow[hrow][hh] = hh < NI ? wi[((long long)b * S + (long long)i * 64 + r0 + 8 * hrow) * NI + hh] * scale : 0.f;
    float score[8][4], sown[8][4], dI[8][4];
    indexer_score_tile(Qs, Ks, wrow, NI, -1, score, sown, warp, lane);
    indexer_dI_tile(score, blse, dblse, gscale, (long long)b * S + (long long)i * 64, nb, j, j == i, dI, warp, lane);
    for (int hh = 0; hh < NI; ++hh) {
      float acc[8][4];
      zero_acc(acc);
      mma64<false, true>(Qs + hh * TILE_ELEMS, Ks, acc, warp, lane);          // recompute S_h
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[nt][e] = bf16_round(acc[nt][e]) > 0.f ? dI[nt][e] * (e < 2 ? wrow[0][hh] : wrow[1][hh]) : 0.f;
      __syncthreads();
      acc_to_smem(acc, Ts, warp, lane);
      __syncthreads();
      mma64<true, false>(Ts, Qs + hh * TILE_ELEMS, dk, warp, lane);           // dS_h^T Q_h
    }
  }
  float* dst = dki + ((long long)b * S + (long long)j * 64) * 64;
  const int cq = 2 * (lane & 3);
#pragma unroll
  for (int nt = 0; nt < 8; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) atomicAdd(dst + (r0 + 8 * (e >> 1)) * 64 + 8 * nt + cq + (e & 1), dk[nt][e]);
}

// ---- host ----------------------------------------------------------------------------------------------------------------------
static void check4(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.is_contiguous() && t.size(-1) == 64, name, ": contiguous bf16 [...,64] required");
}

// q [B,nq,S,64], k [B,nkv,S,64] -> stats [B,nq,S,nb,2] fp32
at::Tensor qsa_main_block_stats(const at::Tensor& q, const at::Tensor& k, double scale) {
  check4(q, "qsa_main_block_stats q"); check4(k, "qsa_main_block_stats k");
  const c10::cuda::CUDAGuard guard(q.device());
  const int B = q.size(0), nq = q.size(1), S = q.size(2), nkv = k.size(1), nb = S / 64;
  TORCH_CHECK(S % 64 == 0 && nq % nkv == 0, "qsa: sequence must be a multiple of 64");
  auto stats = at::empty({B, nq, S, nb, 2}, q.options().dtype(at::kFloat));
  const int smem = 3 * TILE_ELEMS * 2;
  static bool cfg = false;
  if (!cfg) { C10_CUDA_CHECK(cudaFuncSetAttribute(qsa_main_block_stats_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); cfg = true; }
  qsa_main_block_stats_kernel<<<dim3(nb, nq, B), 128, smem, at::cuda::getCurrentCUDAStream()>>>((const bf16*)q.data_ptr(), (const bf16*)k.data_ptr(),
      reinterpret_cast<float2*>(stats.data_ptr<float>()), S, nq, nkv, (float)scale);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return stats;
}

// qi [B,NI,S,64], ki [B,S,64], wi [B,S,NI] fp32 -> blse [B,S,nb] fp32 (non-causal entries = -1e9)
at::Tensor qsa_indexer_fwd(const at::Tensor& qi, const at::Tensor& ki, const at::Tensor& wi, double scale) {
  check4(qi, "qsa_indexer_fwd q"); check4(ki, "qsa_indexer_fwd k");
  const c10::cuda::CUDAGuard guard(qi.device());
  const int B = qi.size(0), NI = qi.size(1), S = qi.size(2), nb = S / 64;
  TORCH_CHECK(NI <= NI_MAX && S % 64 == 0 && wi.scalar_type() == at::kFloat && wi.is_contiguous(), "qsa_indexer_fwd: at most 4 indexer heads");
  auto blse = at::full({B, S, nb}, (double)MASKED, qi.options().dtype(at::kFloat));
  const int smem = (NI_MAX + 2) * TILE_ELEMS * 2;
  static bool cfg = false;
  if (!cfg) { C10_CUDA_CHECK(cudaFuncSetAttribute(qsa_indexer_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); cfg = true; }
  qsa_indexer_fwd_kernel<<<dim3(nb, B, std::min(nb, 4)), 128, smem, at::cuda::getCurrentCUDAStream()>>>((const bf16*)qi.data_ptr(), (const bf16*)ki.data_ptr(), wi.data_ptr<float>(),
      blse.data_ptr<float>(), S, NI, (float)scale);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch(2);
  return blse;
}

// Returns {P [B,S,nb], lp_blk [B,S,nb], kl_tok [B,S], dblse [B,S,nb]}; stats may be undefined when no target is wanted.
std::vector<at::Tensor> qsa_kl_combine(const c10::optional<at::Tensor>& stats, const at::Tensor& blse, int64_t nq) {
  const c10::cuda::CUDAGuard guard(blse.device());
  const int B = blse.size(0), S = blse.size(1), nb = blse.size(2);
  TORCH_CHECK(nb <= 128, "qsa_kl_combine: at most 128 blocks (sequence <= 8192)");
  const bool want = stats.has_value();
  auto opts = blse.options();
  auto P = at::empty({want ? B : 0, S, nb}, opts), lp = at::empty({B, S, nb}, opts), kl = at::empty({want ? B : 0, S}, opts), dbl = at::empty({want ? B : 0, S, nb}, opts);
  const long long tokens = (long long)B * S;
  qsa_kl_combine_kernel<<<(unsigned)((tokens + 7) / 8), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      want ? reinterpret_cast<const float2*>(stats->data_ptr<float>()) : nullptr, blse.data_ptr<float>(), want ? P.data_ptr<float>() : nullptr,
      lp.data_ptr<float>(), want ? kl.data_ptr<float>() : nullptr, want ? dbl.data_ptr<float>() : nullptr, B, S, (int)nq, want ? 1 : 0);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {P, lp, kl, dbl};
}

// lp_blk [B,Q,nb] with Q == S (all queries) or Q == nb (first queries only) -> {count [B,nb] int32, index [B,nb,k] int32}
std::vector<at::Tensor> qsa_select(const at::Tensor& lp_blk, int64_t budget) {
  TORCH_CHECK(lp_blk.is_cuda() && lp_blk.scalar_type() == at::kFloat && lp_blk.is_contiguous() && lp_blk.dim() == 3, "qsa_select: fp32 [B,Q,nb] required");
  const c10::cuda::CUDAGuard guard(lp_blk.device());
  const int B = lp_blk.size(0), Q = lp_blk.size(1), nb = lp_blk.size(2);
  TORCH_CHECK(nb <= 128 && (Q == nb || Q == nb * 64), "qsa_select: unexpected query count");
  const int k = std::min<int>((int)budget, nb);
  auto i32 = lp_blk.options().dtype(at::kInt);
  auto count = at::empty({B, nb}, i32), index = at::empty({B, nb, k}, i32);
  const long long row_stride = (Q == nb) ? nb : (long long)64 * nb;
  qsa_select_kernel<<<(B * nb + 7) / 8, 256, 0, at::cuda::getCurrentCUDAStream()>>>(lp_blk.data_ptr<float>(), row_stride, B, nb, (int)budget, count.data_ptr<int>(), index.data_ptr<int>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {count, index};
}

// Returns {dqi [B,NI,S,64] bf16, dki [B,S,64] bf16, dwi [B,S,NI] fp32}; gscale multiplies dblse (upstream grad / token count).
std::vector<at::Tensor> qsa_indexer_bwd(const at::Tensor& qi, const at::Tensor& ki, const at::Tensor& wi, const at::Tensor& blse, const at::Tensor& dblse,
                                        double gscale, double scale) {
  const c10::cuda::CUDAGuard guard(qi.device());
  const int B = qi.size(0), NI = qi.size(1), S = qi.size(2), nb = S / 64;
  auto dqi = at::empty_like(qi);
  auto dki32 = at::zeros(ki.sizes(), ki.options().dtype(at::kFloat));
  auto dwi = at::empty_like(wi);
  const int smem = (NI_MAX + 3) * TILE_ELEMS * 2;
  static bool cfg = false;
  if (!cfg) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(qsa_indexer_bwd_q_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    C10_CUDA_CHECK(cudaFuncSetAttribute(qsa_indexer_bwd_k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    cfg = true;
  }
  auto stream = at::cuda::getCurrentCUDAStream();
  qsa_indexer_bwd_q_kernel<<<dim3(nb, NI, B), 128, smem, stream>>>((const bf16*)qi.data_ptr(), (const bf16*)ki.data_ptr(), wi.data_ptr<float>(), blse.data_ptr<float>(),
      dblse.data_ptr<float>(), (float)gscale, (bf16*)dqi.data_ptr(), dwi.data_ptr<float>(), S, NI, (float)scale);
  qsa_indexer_bwd_k_kernel<<<dim3(nb, B, std::min(nb, 8)), 128, smem, stream>>>((const bf16*)qi.data_ptr(), (const bf16*)ki.data_ptr(), wi.data_ptr<float>(),
      blse.data_ptr<float>(), dblse.data_ptr<float>(), (float)gscale, dki32.data_ptr<float>(), S, NI, (float)scale);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch(2);
  return {dqi, dki32.to(at::kBFloat16), dwi};
}

}  // namespace q38
