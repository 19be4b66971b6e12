// 64x64x64 bf16 tile products on the warp-level tensor-core path (mma.sync m16n8k16, fp32 accumulation) for kernels
// whose chains of small dependent products are latency bound: the delta-rule scan, the QSA indexer and the block-sparse
// attention.  Four warps cooperate on one 64x64 output; warp w owns rows 16w..16w+15 and keeps them in registers.
#pragma once
#include "common.cuh"

namespace q38 {

constexpr int C64 = 64, LDS = 72;                 // 64x64 bf16 tiles padded to 72 columns (bank-conflict-free fragment loads)
constexpr int TILE_ELEMS = C64 * LDS;
using bf16 = __nv_bfloat16;

__device__ __forceinline__ uint32_t pack2(bf16 a, bf16 b) {
  return (uint32_t)__bfloat16_as_ushort(a) | ((uint32_t)__bfloat16_as_ushort(b) << 16);
}

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Four 8x8 b16 matrices from shared memory; lane l supplies the (16-byte aligned) address of row l % 8 of matrix l / 8.
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const bf16* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const bf16* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

// acc[64x64] += A * B with four warps; warp w owns rows 16w..16w+15.
//   A(i,k) = TA ? As[k*LDS + i] : As[i*LDS + k]          B(k,n) = TB ? Bs[n*LDS + k] : Bs[k*LDS + n]
// Accumulator element acc[nt][e]: row = 16w + lane/4 + 8*(e>>1), col = 8nt + 2*(lane%4) + (e&1).
// Fragments come from ldmatrix (.trans when the tile is stored with the contraction index as its row): one instruction per
// A fragment and one per pair of B fragments.  Rows are 144 bytes apart, so the eight row addresses of a matrix hit distinct banks.
template <bool TA, bool TB>
__device__ __forceinline__ void mma64(const bf16* __restrict__ As, const bf16* __restrict__ Bs, float (&acc)[8][4], int warp, int lane) {
  const int l8 = lane & 7, m = lane >> 3;          // row inside a matrix, matrix index
  // A: matrices (i 0-7, k 0-7), (i 8-15, k 0-7), (i 0-7, k 8-15), (i 8-15, k 8-15)
  const bf16* a_ptr = TA ? As + (l8 + 8 * (m >> 1)) * LDS + 16 * warp + 8 * (m & 1)
                         : As + (16 * warp + l8 + 8 * (m & 1)) * LDS + 8 * (m >> 1);
  // B, for a pair of n-tiles: (k 0-7, n 0-7), (k 8-15, n 0-7), (k 0-7, n 8-15), (k 8-15, n 8-15)
  const bf16* b_ptr = TB ? Bs + (l8 + 8 * (m >> 1)) * LDS + 8 * (m & 1)
                         : Bs + (l8 + 8 * (m & 1)) * LDS + 8 * (m >> 1);
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    uint32_t a[4];
    if (TA) ldmatrix_x4_trans(a, a_ptr + 16 * ks * LDS);
    else ldmatrix_x4(a, a_ptr + 16 * ks);
#pragma unroll
    for (int np = 0; np < 4; ++np) {
      uint32_t b[4];
      if (TB) ldmatrix_x4(b, b_ptr + 16 * np * LDS + 16 * ks);
      else ldmatrix_x4_trans(b, b_ptr + 16 * ks * LDS + 16 * np);
      mma16816(acc[2 * np], a, b[0], b[1]);
      mma16816(acc[2 * np + 1], a, b[2], b[3]);
    }
  }
}

__device__ __forceinline__ void zero_acc(float (&acc)[8][4]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
}

// Accumulator fragment -> padded bf16 tile in shared memory (row-major).
__device__ __forceinline__ void acc_to_smem(const float (&acc)[8][4], bf16* __restrict__ dst, int warp, int lane) {
  const int r = 16 * warp + (lane >> 2), cq = 2 * (lane & 3);
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    *reinterpret_cast<__nv_bfloat162*>(dst + r * LDS + 8 * nt + cq) = __floats2bfloat162_rn(acc[nt][0], acc[nt][1]);
    *reinterpret_cast<__nv_bfloat162*>(dst + (r + 8) * LDS + 8 * nt + cq) = __floats2bfloat162_rn(acc[nt][2], acc[nt][3]);
  }
}

// Accumulator fragment -> dense [64,64] bf16 tile in global memory with row stride `ld` elements.
__device__ __forceinline__ void acc_to_global(const float (&acc)[8][4], bf16* __restrict__ dst, long long ld, int warp, int lane, float scale = 1.f) {
  const int r = 16 * warp + (lane >> 2), cq = 2 * (lane & 3);
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    *reinterpret_cast<__nv_bfloat162*>(dst + (long long)r * ld + 8 * nt + cq) = __floats2bfloat162_rn(acc[nt][0] * scale, acc[nt][1] * scale);
    *reinterpret_cast<__nv_bfloat162*>(dst + (long long)(r + 8) * ld + 8 * nt + cq) = __floats2bfloat162_rn(acc[nt][2] * scale, acc[nt][3] * scale);
  }
}

// cp.async of a dense [64,64] bf16 tile (row stride `ld` elements, 16-byte aligned rows) into a padded shared tile.
__device__ __forceinline__ void load_tile_async(bf16* __restrict__ dst, const bf16* __restrict__ src, long long ld, int tid) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int chunk = tid + 128 * i;                 // 512 chunks of 16 bytes
    const int row = chunk >> 3, col = (chunk & 7) * 8;
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst + row * LDS + col));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src + (long long)row * ld + col) : "memory");
  }
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }


// Fragment of a dense [64,64] bf16 tile in global memory.
__device__ __forceinline__ void frag_from_global(const bf16* __restrict__ src, float (&dst)[8][4], int warp, int lane) {
  const int r = 16 * warp + (lane >> 2), cq = 2 * (lane & 3);
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(src + r * 64 + 8 * nt + cq);
    const __nv_bfloat162 b2 = *reinterpret_cast<const __nv_bfloat162*>(src + (r + 8) * 64 + 8 * nt + cq);
    dst[nt][0] = __low2float(a); dst[nt][1] = __high2float(a); dst[nt][2] = __low2float(b2); dst[nt][3] = __high2float(b2);
  }
}
__device__ __forceinline__ void frag_from_smem(const bf16* __restrict__ src, float (&dst)[8][4], int warp, int lane) {
  const int r = 16 * warp + (lane >> 2), cq = 2 * (lane & 3);
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(src + r * LDS + 8 * nt + cq);
    const __nv_bfloat162 b2 = *reinterpret_cast<const __nv_bfloat162*>(src + (r + 8) * LDS + 8 * nt + cq);
    dst[nt][0] = __low2float(a); dst[nt][1] = __high2float(a); dst[nt][2] = __low2float(b2); dst[nt][3] = __high2float(b2);
  }
}

// ---- half-width variants for CTAs of eight warps -----------------------------------------------------------------------
// Warp w owns rows 16 (w & 3) .. +15 and columns 32 (w >> 2) .. +31 of the 64x64 output: twice the warps of mma64 work on
// one tile, each with half the accumulator registers, which doubles the latency hiding of chains of dependent products.
// Accumulator element acc[nt][e]: row = 16 (w & 3) + lane/4 + 8*(e>>1), col = 32 (w >> 2) + 8nt + 2*(lane%4) + (e&1).
template <bool TA, bool TB>
__device__ __forceinline__ void mma64h(const bf16* __restrict__ As, const bf16* __restrict__ Bs, float (&acc)[4][4], int warp, int lane) {
  const int l8 = lane & 7, m = lane >> 3, wr = warp & 3, n0 = 32 * (warp >> 2);
  const bf16* a_ptr = TA ? As + (l8 + 8 * (m >> 1)) * LDS + 16 * wr + 8 * (m & 1)
                         : As + (16 * wr + l8 + 8 * (m & 1)) * LDS + 8 * (m >> 1);
  const bf16* b_ptr = TB ? Bs + (n0 + l8 + 8 * (m >> 1)) * LDS + 8 * (m & 1)
                         : Bs + (l8 + 8 * (m & 1)) * LDS + n0 + 8 * (m >> 1);
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    uint32_t a[4];
    if (TA) ldmatrix_x4_trans(a, a_ptr + 16 * ks * LDS);
    else ldmatrix_x4(a, a_ptr + 16 * ks);
#pragma unroll
    for (int np = 0; np < 2; ++np) {
      uint32_t b[4];
      if (TB) ldmatrix_x4(b, b_ptr + 16 * np * LDS + 16 * ks);
      else ldmatrix_x4_trans(b, b_ptr + 16 * ks * LDS + 16 * np);
      mma16816(acc[2 * np], a, b[0], b[1]);
      mma16816(acc[2 * np + 1], a, b[2], b[3]);
    }
  }
}

__device__ __forceinline__ void zero_acc(float (&acc)[4][4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
}

__device__ __forceinline__ void acc_to_smem_h(const float (&acc)[4][4], bf16* __restrict__ dst, int warp, int lane) {
  const int r = 16 * (warp & 3) + (lane >> 2), c0 = 32 * (warp >> 2) + 2 * (lane & 3);
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) {
    *reinterpret_cast<__nv_bfloat162*>(dst + r * LDS + 8 * nt + c0) = __floats2bfloat162_rn(acc[nt][0], acc[nt][1]);
    *reinterpret_cast<__nv_bfloat162*>(dst + (r + 8) * LDS + 8 * nt + c0) = __floats2bfloat162_rn(acc[nt][2], acc[nt][3]);
  }
}

__device__ __forceinline__ void acc_to_global_h(const float (&acc)[4][4], bf16* __restrict__ dst, long long ld, int warp, int lane, float scale = 1.f) {
  const int r = 16 * (warp & 3) + (lane >> 2), c0 = 32 * (warp >> 2) + 2 * (lane & 3);
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) {
    *reinterpret_cast<__nv_bfloat162*>(dst + (long long)r * ld + 8 * nt + c0) = __floats2bfloat162_rn(acc[nt][0] * scale, acc[nt][1] * scale);
    *reinterpret_cast<__nv_bfloat162*>(dst + (long long)(r + 8) * ld + 8 * nt + c0) = __floats2bfloat162_rn(acc[nt][2] * scale, acc[nt][3] * scale);
  }
}

// load_tile_async for a CTA of 256 threads.
__device__ __forceinline__ void load_tile_async_256(bf16* __restrict__ dst, const bf16* __restrict__ src, long long ld, int tid) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int chunk = tid + 256 * i;                 // 512 chunks of 16 bytes
    const int row = chunk >> 3, col = (chunk & 7) * 8;
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst + row * LDS + col));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src + (long long)row * ld + col) : "memory");
  }
}

}  // namespace q38
