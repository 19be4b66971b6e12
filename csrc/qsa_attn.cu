// Block-sparse (and dense causal) GQA attention for QSA, forward and backward, on 64x64 tiles.
//
// Query block i attends to the key blocks listed in index[b, i, :count[b, i]] (all <= i, own block included); inside the
// own block the mask is causal.  `dense` ignores the lists and uses every block j <= i (the warm-up phase).
//
//   qsa_attn_fwd     grid (nb, nq, B): online-softmax over the selected key blocks; writes o token-major [B,S,nq,64]
//                    and the row log-sum-exp.
//   qsa_attn_bwd_q   grid (nb, nq, B): D = rowsum(dO o); dQ = sum_j (P (dP - D)) K scale.
//   qsa_attn_bwd_kv  grid (nb, nkv, B): for key block j, loops over the query heads of the group and over the query
//                    blocks i >= j that selected j (a [B,nb,nb] selection matrix built on the device): dV += P^T dO,
//                    dK += dS^T Q scale.  No atomics: one CTA owns a (key block, kv head).
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"
#include "host.h"
#include "mma_tile.cuh"

namespace q38 {

// sel[b, i, j] = 1 iff query block i attends key block j
__global__ void qsa_selection_matrix_kernel(const int* __restrict__ count, const int* __restrict__ index, int kmax, int nb, int dense,
                                            unsigned char* __restrict__ sel) {
  const int b = blockIdx.y, i = blockIdx.x;
  unsigned char* row = sel + ((long long)b * nb + i) * nb;
  for (int j = threadIdx.x; j < nb; j += blockDim.x) row[j] = dense ? (j <= i) : 0;
  __syncthreads();
  if (!dense) {
    const int c = count[b * nb + i];
    for (int s = threadIdx.x; s < c; s += blockDim.x) {
      const int j = index[((long long)b * nb + i) * kmax + s];
      if (j >= 0 && j <= i) row[j] = 1;
    }
  }
}

// exp-weights of one score tile given the running row maxima; returns P in `acc` and row sums in rs[2]
__device__ __forceinline__ void scores_to_probs(float (&acc)[8][4], const float (&m)[2], bool diag, int warp, int lane, float (&rs)[2]) {
  const int r0 = 16 * warp + (lane >> 2), cq = 2 * (lane & 3);
  rs[0] = rs[1] = 0.f;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int row = r0 + 8 * (e >> 1), col = 8 * nt + cq + (e & 1);
      const float p = (diag && col > row) ? 0.f : __expf(acc[nt][e] - m[e >> 1]);
      acc[nt][e] = p;
      rs[e >> 1] += p;
    }
#pragma unroll
  for (int x = 0; x < 2; ++x) { rs[x] += __shfl_xor_sync(0xffffffffu, rs[x], 1); rs[x] += __shfl_xor_sync(0xffffffffu, rs[x], 2); }
}

__global__ void __launch_bounds__(128) qsa_attn_fwd_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                                                           const unsigned char* __restrict__ sel, bf16* __restrict__ o, float* __restrict__ lse,
                                                           int S, int nq, int nkv, float scale) {
  extern __shared__ __align__(16) uint8_t smem_bytes[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_bytes);
  bf16* Ks = Qs + TILE_ELEMS;
  bf16* Vs = Ks + TILE_ELEMS;
  bf16* Ps = Vs + TILE_ELEMS;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int i = blockIdx.x, h = blockIdx.y, b = blockIdx.z, nb = S / 64, kvh = h / (nq / nkv);
  const bf16* kbase = k + ((long long)b * nkv + kvh) * S * 64;
  const bf16* vbase = v + ((long long)b * nkv + kvh) * S * 64;
  const unsigned char* srow = sel + ((long long)b * nb + i) * nb;
  load_tile_async(Qs, q + (((long long)b * nq + h) * S + (long long)i * 64) * 64, 64, tid);
  cp_async_commit();
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float out[8][4];
  zero_acc(out);
  for (int j = 0; j <= i; ++j) {
    if (!srow[j]) continue;
    __syncthreads();                                       // previous tile's readers are done with Ks, Vs, Ps
    load_tile_async(Ks, kbase + (long long)j * 4096, 64, tid);
    load_tile_async(Vs, vbase + (long long)j * 4096, 64, tid);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    float acc[8][4];
    zero_acc(acc);
    mma64<false, true>(Qs, Ks, acc, warp, lane);
    const bool diag = j == i;
    {
      const int r0 = 16 * warp + (lane >> 2), cq = 2 * (lane & 3);
      float tm[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          acc[nt][e] *= scale;
          const int row = r0 + 8 * (e >> 1), col = 8 * nt + cq + (e & 1);
          if (!diag || col <= row) tm[e >> 1] = fmaxf(tm[e >> 1], acc[nt][e]);
        }
      float mn[2], corr[2], rs[2];
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        tm[x] = fmaxf(tm[x], __shfl_xor_sync(0xffffffffu, tm[x], 1));
        tm[x] = fmaxf(tm[x], __shfl_xor_sync(0xffffffffu, tm[x], 2));
        mn[x] = fmaxf(m[x], tm[x]);
        corr[x] = __expf(m[x] - mn[x]);
      }
      scores_to_probs(acc, mn, diag, warp, lane, rs);
#pragma unroll
      for (int x = 0; x < 2; ++x) { l[x] = l[x] * corr[x] + rs[x]; m[x] = mn[x]; }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) { out[nt][0] *= corr[0]; out[nt][1] *= corr[0]; out[nt][2] *= corr[1]; out[nt][3] *= corr[1]; }
    }
    acc_to_smem(acc, Ps, warp, lane);
    __syncthreads();
    mma64<false, false>(Ps, Vs, out, warp, lane);
  }
  const int r0 = 16 * warp + (lane >> 2);
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) { out[nt][0] /= l[0]; out[nt][1] /= l[0]; out[nt][2] /= l[1]; out[nt][3] /= l[1]; }
  acc_to_global(out, o + (((long long)b * S + (long long)i * 64) * nq + h) * 64, (long long)nq * 64, warp, lane);
  if ((lane & 3) == 0) {
#pragma unroll
    for (int x = 0; x < 2; ++x) lse[((long long)b * nq + h) * S + (long long)i * 64 + r0 + 8 * x] = m[x] + __logf(l[x]);
  }
}

// dO, o: token-major [B,S,nq,64].  Writes dq [B,nq,S,64] and D [B,nq,S].
__global__ void __launch_bounds__(128) qsa_attn_bwd_q_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                                                             const bf16* __restrict__ o, const bf16* __restrict__ dout, const float* __restrict__ lse,
                                                             const unsigned char* __restrict__ sel, bf16* __restrict__ dq, float* __restrict__ Dout,
                                                             int S, int nq, int nkv, float scale) {
  extern __shared__ __align__(16) uint8_t smem_bytes[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_bytes);
  bf16* dOs = Qs + TILE_ELEMS;
  bf16* Ks = dOs + TILE_ELEMS;
  bf16* Vs = Ks + TILE_ELEMS;
  bf16* Ts = Vs + TILE_ELEMS;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int i = blockIdx.x, h = blockIdx.y, b = blockIdx.z, nb = S / 64, kvh = h / (nq / nkv);
  const bf16* kbase = k + ((long long)b * nkv + kvh) * S * 64;
  const bf16* vbase = v + ((long long)b * nkv + kvh) * S * 64;
  const unsigned char* srow = sel + ((long long)b * nb + i) * nb;
  const long long tok_off = (((long long)b * S + (long long)i * 64) * nq + h) * 64, ld_tok = (long long)nq * 64;
  load_tile_async(Qs, q + (((long long)b * nq + h) * S + (long long)i * 64) * 64, 64, tid);
  load_tile_async(dOs, dout + tok_off, ld_tok, tid);
  load_tile_async(Ts, o + tok_off, ld_tok, tid);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
  const int r0 = 16 * warp + (lane >> 2);
  float D[2], L[2];
  {
    float a[8][4], c[8][4];
    frag_from_smem(dOs, a, warp, lane);
    frag_from_smem(Ts, c, warp, lane);
    D[0] = D[1] = 0.f;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) { D[0] += a[nt][0] * c[nt][0] + a[nt][1] * c[nt][1]; D[1] += a[nt][2] * c[nt][2] + a[nt][3] * c[nt][3]; }
#pragma unroll
    for (int x = 0; x < 2; ++x) {
      D[x] += __shfl_xor_sync(0xffffffffu, D[x], 1);
      D[x] += __shfl_xor_sync(0xffffffffu, D[x], 2);
      const long long idx = ((long long)b * nq + h) * S + (long long)i * 64 + r0 + 8 * x;
      L[x] = lse[idx];
      if ((lane & 3) == 0) Dout[idx] = D[x];
    }
  }
  float dQ[8][4];
  zero_acc(dQ);
  for (int j = 0; j <= i; ++j) {
    if (!srow[j]) continue;
    __syncthreads();
    load_tile_async(Ks, kbase + (long long)j * 4096, 64, tid);
    load_tile_async(Vs, vbase + (long long)j * 4096, 64, tid);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    float s[8][4], dp[8][4];
    zero_acc(s);
    mma64<false, true>(Qs, Ks, s, warp, lane);
    zero_acc(dp);
    mma64<false, true>(dOs, Vs, dp, warp, lane);
    const bool diag = j == i;
    const int cq = 2 * (lane & 3);
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = r0 + 8 * (e >> 1), col = 8 * nt + cq + (e & 1);
        const float p = (diag && col > row) ? 0.f : __expf(s[nt][e] * scale - L[e >> 1]);
        s[nt][e] = p * (dp[nt][e] - D[e >> 1]) * scale;            // dS (already times the score scale)
      }
    acc_to_smem(s, Ts, warp, lane);
    __syncthreads();
    mma64<false, false>(Ts, Ks, dQ, warp, lane);
  }
  acc_to_global(dQ, dq + (((long long)b * nq + h) * S + (long long)i * 64) * 64, 64, warp, lane);
}

__global__ void __launch_bounds__(128) qsa_attn_bwd_kv_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                                                              const bf16* __restrict__ dout, const float* __restrict__ lse, const float* __restrict__ Din,
                                                              const unsigned char* __restrict__ sel, float* __restrict__ dk, float* __restrict__ dv,
                                                              int S, int nq, int nkv, float scale) {
  extern __shared__ __align__(16) uint8_t smem_bytes[];
  bf16* Ks = reinterpret_cast<bf16*>(smem_bytes);
  bf16* Vs = Ks + TILE_ELEMS;
  bf16* Qs = Vs + TILE_ELEMS;
  bf16* dOs = Qs + TILE_ELEMS;
  bf16* Ps = dOs + TILE_ELEMS;
  bf16* dSs = Ps + TILE_ELEMS;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // One CTA per (key block, query head, batch): the key blocks near the start of the sequence are selected by almost every
  // later query block, so the work of a key block is spread over the heads of its group; partial dK / dV are added in fp32.
  const int j = blockIdx.x, h = blockIdx.y, b = blockIdx.z, nb = S / 64, rep = nq / nkv, kvh = h / rep;
  load_tile_async(Ks, k + (((long long)b * nkv + kvh) * S + (long long)j * 64) * 64, 64, tid);
  load_tile_async(Vs, v + (((long long)b * nkv + kvh) * S + (long long)j * 64) * 64, 64, tid);
  cp_async_commit();
  const int r0 = 16 * warp + (lane >> 2), cq = 2 * (lane & 3);
  const long long ld_tok = (long long)nq * 64;
  float dK[8][4], dV[8][4];
  zero_acc(dK);
  zero_acc(dV);
  for (int i = j; i < nb; ++i) {
    if (!sel[((long long)b * nb + i) * nb + j]) continue;
    {
      __syncthreads();
      load_tile_async(Qs, q + (((long long)b * nq + h) * S + (long long)i * 64) * 64, 64, tid);
      load_tile_async(dOs, dout + (((long long)b * S + (long long)i * 64) * nq + h) * 64, ld_tok, tid);
      cp_async_commit();
      cp_async_wait<0>();
      __syncthreads();
      float s[8][4], dp[8][4];
      zero_acc(s);
      mma64<false, true>(Qs, Ks, s, warp, lane);
      zero_acc(dp);
      mma64<false, true>(dOs, Vs, dp, warp, lane);
      float L[2], D[2];
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        const long long idx = ((long long)b * nq + h) * S + (long long)i * 64 + r0 + 8 * x;
        L[x] = lse[idx]; D[x] = Din[idx];
      }
      const bool diag = j == i;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int row = r0 + 8 * (e >> 1), col = 8 * nt + cq + (e & 1);
          const float p = (diag && col > row) ? 0.f : __expf(s[nt][e] * scale - L[e >> 1]);
          s[nt][e] = p;
          dp[nt][e] = p * (dp[nt][e] - D[e >> 1]) * scale;
        }
      acc_to_smem(s, Ps, warp, lane);
      acc_to_smem(dp, dSs, warp, lane);
      __syncthreads();
      mma64<true, false>(Ps, dOs, dV, warp, lane);         // P^T dO
      mma64<true, false>(dSs, Qs, dK, warp, lane);         // dS^T Q
    }
  }
  cp_async_wait<0>();
  float* dkp = dk + (((long long)b * nkv + kvh) * S + (long long)j * 64) * 64;
  float* dvp = dv + (((long long)b * nkv + kvh) * S + (long long)j * 64) * 64;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int row = r0 + 8 * (e >> 1), col = 8 * nt + cq + (e & 1);
      atomicAdd(dkp + row * 64 + col, dK[nt][e]);
      atomicAdd(dvp + row * 64 + col, dV[nt][e]);
    }
}

// ---- host ----------------------------------------------------------------------------------------------------------------------
static void check_heads(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.is_contiguous() && t.dim() == 4 && t.size(3) == 64, name, ": contiguous bf16 [B,H,S,64] required");
}

static at::Tensor selection_matrix(const c10::optional<at::Tensor>& count, const c10::optional<at::Tensor>& index, int B, int nb, const at::TensorOptions& opts,
                                   cudaStream_t stream) {
  auto sel = at::empty({B, nb, nb}, opts.dtype(at::kByte));
  const bool dense = !count.has_value();
  if (!dense) TORCH_CHECK(count->scalar_type() == at::kInt && index->scalar_type() == at::kInt && count->is_contiguous() && index->is_contiguous(), "qsa: int32 block lists required");
  qsa_selection_matrix_kernel<<<dim3(nb, B), 64, 0, stream>>>(dense ? nullptr : count->data_ptr<int>(), dense ? nullptr : index->data_ptr<int>(),
                                                              dense ? 0 : (int)index->size(2), nb, dense ? 1 : 0, sel.data_ptr<unsigned char>());
  count_launch();
  return sel;
}

// Returns {o [B,S,nq,64] bf16, lse [B,nq,S] fp32, sel [B,nb,nb] uint8}
std::vector<at::Tensor> qsa_attn_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const c10::optional<at::Tensor>& count,
                                     const c10::optional<at::Tensor>& index, double scale) {
  check_heads(q, "qsa_attn_fwd q"); check_heads(k, "qsa_attn_fwd k"); check_heads(v, "qsa_attn_fwd v");
  const c10::cuda::CUDAGuard guard(q.device());
  const int B = q.size(0), nq = q.size(1), S = q.size(2), nkv = k.size(1), nb = S / 64;
  TORCH_CHECK(S % 64 == 0 && nq % nkv == 0, "qsa_attn_fwd: bad shapes");
  auto stream = at::cuda::getCurrentCUDAStream();
  auto sel = selection_matrix(count, index, B, nb, q.options(), stream);
  auto o = at::empty({B, S, nq, 64}, q.options());
  auto lse = at::empty({B, nq, S}, q.options().dtype(at::kFloat));
  const int smem = 4 * TILE_ELEMS * 2;
  static bool cfg = false;
  if (!cfg) { C10_CUDA_CHECK(cudaFuncSetAttribute(qsa_attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); cfg = true; }
  qsa_attn_fwd_kernel<<<dim3(nb, nq, B), 128, smem, stream>>>((const bf16*)q.data_ptr(), (const bf16*)k.data_ptr(), (const bf16*)v.data_ptr(),
      sel.data_ptr<unsigned char>(), (bf16*)o.data_ptr(), lse.data_ptr<float>(), S, nq, nkv, (float)scale);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {o, lse, sel};
}

// Returns {dq [B,nq,S,64], dk, dv [B,nkv,S,64]}
std::vector<at::Tensor> qsa_attn_bwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& o, const at::Tensor& dout,
                                     const at::Tensor& lse, const at::Tensor& sel, double scale) {
  check_heads(q, "qsa_attn_bwd q");
  TORCH_CHECK(dout.is_contiguous() && dout.scalar_type() == at::kBFloat16 && o.is_contiguous(), "qsa_attn_bwd: contiguous bf16 dO/o [B,S,nq,64] required");
  const c10::cuda::CUDAGuard guard(q.device());
  const int B = q.size(0), nq = q.size(1), S = q.size(2), nkv = k.size(1), nb = S / 64;
  auto dq = at::empty_like(q);
  auto dk32 = at::zeros(k.sizes(), k.options().dtype(at::kFloat)), dv32 = at::zeros(v.sizes(), v.options().dtype(at::kFloat));
  auto D = at::empty({B, nq, S}, q.options().dtype(at::kFloat));
  auto stream = at::cuda::getCurrentCUDAStream();
  const int smem_q = 5 * TILE_ELEMS * 2, smem_kv = 6 * TILE_ELEMS * 2;
  static bool cfg = false;
  if (!cfg) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(qsa_attn_bwd_q_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_q));
    C10_CUDA_CHECK(cudaFuncSetAttribute(qsa_attn_bwd_kv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_kv));
    cfg = true;
  }
  qsa_attn_bwd_q_kernel<<<dim3(nb, nq, B), 128, smem_q, stream>>>((const bf16*)q.data_ptr(), (const bf16*)k.data_ptr(), (const bf16*)v.data_ptr(),
      (const bf16*)o.data_ptr(), (const bf16*)dout.data_ptr(), lse.data_ptr<float>(), sel.data_ptr<unsigned char>(), (bf16*)dq.data_ptr(), D.data_ptr<float>(),
      S, nq, nkv, (float)scale);
  qsa_attn_bwd_kv_kernel<<<dim3(nb, nq, B), 128, smem_kv, stream>>>((const bf16*)q.data_ptr(), (const bf16*)k.data_ptr(), (const bf16*)v.data_ptr(),
      (const bf16*)dout.data_ptr(), lse.data_ptr<float>(), D.data_ptr<float>(), sel.data_ptr<unsigned char>(), dk32.data_ptr<float>(), dv32.data_ptr<float>(),
      S, nq, nkv, (float)scale);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch(2);
  return {dq, dk32.to(at::kBFloat16), dv32.to(at::kBFloat16)};
}

}  // namespace q38
