// C entry point for callers that must not allocate device memory.
//
// This function has no counterpart in the reference implementation; it exists for embedders of this library.
//
// Who needs it: code that runs where cudaMalloc / cudaFree (and therefore any torch allocation) is off limits, for
// example a serving loop whose memory is fully pre-planned and handed out from one arena, a host callback or a
// latency-critical thread that may not take the allocator's locks or trigger its implicit device synchronisation,
// or a component that runs after the process has given its whole memory budget to other users.  Such callers already
// own their input and output buffers; the only thing the regular `moe_sort` operator would still allocate is its scratch
// (the per-block expert histograms of the counting sort).  Here that scratch lives inside the library image itself.
//
//   q38_moe_sort_static  sorts the P = T*k (token, slot) pairs of an MoE routing decision by expert, exactly like the
//                        `q38::moe_sort` operator (stable: ties keep pair order), and writes the 128-row tile schedule
//                        of the grouped GEMMs.
//
// Scratch: a file-scope `static __device__` array of Q38_SORT_STATIC_MAX_BLOCKS * 64 ints (256 KiB).  Every GPU that
// loads the library holds this array until the process exits.  It bounds the problem size: P may not exceed
// Q38_SORT_STATIC_MAX_PAIRS; larger calls are rejected with Q38_NOALLOC_TOO_LARGE and nothing is launched.
//
// Set-up: the first call on a device resolves the array's device address (cudaGetSymbolAddress with that device
// current).  Make that first call outside of any CUDA stream capture.
//
// Sharing: all calls on a device use the same array and it keeps whatever the previous call left in it.  The sort
// overwrites every word it later reads, so nothing has to be cleared between calls, but two calls whose kernels may
// overlap on the GPU (different streams without an ordering between them) race on it: serialise them.
//
// The function calls no cudaMalloc, cudaFree or allocating library routine.  Kernels are enqueued on `stream` and the
// function returns without synchronising.
#pragma once
#include <cuda_runtime.h>

#define Q38_SORT_STATIC_MAX_BLOCKS 1024
#define Q38_SORT_STATIC_MAX_PAIRS (Q38_SORT_STATIC_MAX_BLOCKS * 1024)

enum {
  Q38_NOALLOC_OK = 0,
  Q38_NOALLOC_TOO_LARGE = 1,      // P > Q38_SORT_STATIC_MAX_PAIRS or experts > 64
  Q38_NOALLOC_BAD_ARGUMENT = 2,   // null pointer, non-positive size, or a schedule buffer that is too small
  Q38_NOALLOC_CUDA_ERROR = 3,     // a CUDA runtime call failed (set-up or launch); see cudaGetLastError
};

#ifdef __cplusplus
extern "C" {
#endif

// expert_of_pair [P] int32 (device): expert chosen for pair p = token * k + slot.  Precondition: 0 <= id < experts for every
// pair.  A pair that violates it (for instance a -1 "dropped token" marker) is skipped, not sorted: it is counted in no
// expert's range, its inv_perm entry is set to -1, and as many entries at the end of perm as there are such pairs are left
// unwritten.  No out-of-range memory is touched.
// perm [P], inv_perm [P], offsets [experts + 1], sched [1 + 3 * max_tiles] int32 (device), caller-owned.
// max_tiles must be at least ceil(P / 128) + experts.
int q38_moe_sort_static(const int* expert_of_pair, int P, int experts, int* perm, int* inv_perm, int* offsets, int* sched,
                        int max_tiles, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
