// Expert parallelism: the 64 experts are split over the ranks; routed token rows travel to the GPU that owns their
// expert and the expert outputs travel back.  Both directions are peer-memory stores issued from inside the kernels that
// produce the rows, so no separate all-to-all runs:
//
//   ep_plan        from the per-rank, per-expert row counts (exchanged through peer stores): where each of my rows lands
//                  on its owner (rows of one expert are contiguous on the owner, ordered by source rank), the owner's
//                  128-row tile schedule and its per-expert offsets.
//   ep_dispatch    fused permute + send: sorted row i (of expert e) is read from the local activations (gathered by token
//                  or taken from a sorted buffer) and stored straight into the owner's receive buffer, together with its
//                  return address (source rank, sorted position).
//   (grouped GEMMs of csrc/moe.cu run on the received rows; the epilogue of the last GEMM of each direction stores every
//    output row directly into the source rank's buffer at its return address: the combine transfer is fused into the GEMM.)
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"
#include "host.h"

namespace q38 {

constexpr int EP_MAX_PEERS = 16;
struct EpPeers { void* p[EP_MAX_PEERS]; };

// counts_all [W, E] (row s = counts of source rank s).  One CTA of 64 threads.
// send_base [E]: first row on the owner for my rows of expert e.   recv_offsets [E_loc + 1]: owner-side expert offsets.
// sched: [0] = tiles, then (local expert, row0, rows) per tile.     status[0] = total rows received, status[1] = overflow flag.
__global__ void __launch_bounds__(64) ep_plan_kernel(const int* __restrict__ counts_all, int rank, int world, int E, int E_loc, int capacity,
                                                     int* __restrict__ send_base, int* __restrict__ recv_offsets, int* __restrict__ sched,
                                                     int max_tiles, int tile_rows, int* __restrict__ status, int* __restrict__ err) {
  __shared__ int tot[64], base[65];
  const int e = threadIdx.x;
  if (e < E) {
    int t = 0;
    for (int s = 0; s < world; ++s) t += counts_all[s * E + e];
    tot[e] = t;
  }
  __syncthreads();
  if (e == 0) {
    // per owner: exclusive scan over its local experts
    for (int o = 0; o < world; ++o) {
      int acc = 0;
      for (int l = 0; l < E_loc; ++l) { base[o * E_loc + l] = acc; acc += tot[o * E_loc + l]; }
      if (o == rank) { status[0] = acc; status[1] = acc > capacity ? 1 : 0; if (acc > capacity) report_error(err, ERR_BOUNDS); }
    }
  }
  __syncthreads();
  if (e < E) {
    int before = 0;
    for (int s = 0; s < rank; ++s) before += counts_all[s * E + e];
    send_base[e] = base[e] + before;
  }
  if (e < E_loc) {
    const int ge = rank * E_loc + e;
    recv_offsets[e] = base[ge];
    if (e == E_loc - 1) recv_offsets[E_loc] = base[ge] + tot[ge];
  }
  if (e == 0) {
    int tile = 0;
    for (int l = 0; l < E_loc; ++l) {
      const int ge = rank * E_loc + l, n = tot[ge];
      for (int i = 0; i * tile_rows < n && tile < max_tiles; ++i, ++tile) {
        sched[1 + 3 * tile] = l; sched[2 + 3 * tile] = base[ge] + i * tile_rows; sched[3 + 3 * tile] = min(tile_rows, n - i * tile_rows);
      }
    }
    sched[0] = tile;
    for (int t2 = tile; t2 < max_tiles; ++t2) { sched[1 + 3 * t2] = 0; sched[2 + 3 * t2] = 0; sched[3 + 3 * t2] = 0; }
  }
}

// One warp per sorted row.  src: [T, h] gathered by token (gather = 1) or [P, h] sorted rows (gather = 0).
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ perm, const int* __restrict__ expert_of_pair,
                                                          const int* __restrict__ offsets, const int* __restrict__ send_base, int P, int K, int h, int E_loc,
                                                          int capacity, int gather, int rank, EpPeers recv_rows, EpPeers ret_rank, EpPeers ret_row) {
  const int i = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (i >= P) return;
  const int pair = perm[i], e = expert_of_pair[pair];
  const int owner = e / E_loc, dest = send_base[e] + (i - offsets[e]);
  if (dest >= capacity) return;                                   // overflow is reported by ep_plan; never write out of bounds
  const uint4* s = reinterpret_cast<const uint4*>(src + (size_t)(gather ? pair / K : i) * h);
  uint4* d = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(recv_rows.p[owner]) + (size_t)dest * h);
  for (int c = lane; c < h / 8; c += 32) d[c] = s[c];
  if (lane == 0) {
    reinterpret_cast<int*>(ret_rank.p[owner])[dest] = rank;
    reinterpret_cast<int*>(ret_row.p[owner])[dest] = i;
  }
}

// Every rank publishes its per-expert counts (offsets[e+1] - offsets[e]) into row `rank` of every peer's counts_all.
__global__ void ep_publish_counts_kernel(const int* __restrict__ offsets, int E, int rank, int world, EpPeers counts_all) {
  const int e = threadIdx.x;
  if (e >= E) return;
  const int c = offsets[e + 1] - offsets[e];
  for (int p = 0; p < world; ++p) reinterpret_cast<int*>(counts_all.p[p])[rank * E + e] = c;
}

static EpPeers ep_ptrs(const std::vector<int64_t>& v) {
  TORCH_CHECK((int)v.size() <= EP_MAX_PEERS, "at most 16 peers");
  EpPeers p{};
  for (size_t i = 0; i < v.size(); ++i) p.p[i] = reinterpret_cast<void*>(v[i]);
  return p;
}

void ep_publish_counts(const at::Tensor& offsets, int64_t rank, std::vector<int64_t> peer_counts) {
  const c10::cuda::CUDAGuard guard(offsets.device());
  const int E = offsets.numel() - 1;
  ep_publish_counts_kernel<<<1, 64, 0, at::cuda::getCurrentCUDAStream()>>>(offsets.data_ptr<int>(), E, (int)rank, (int)peer_counts.size(), ep_ptrs(peer_counts));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

// Returns {send_base [E], recv_offsets [E_loc+1], sched [1+3*max_tiles], status [2]}
std::vector<at::Tensor> ep_plan(const at::Tensor& counts_all, int64_t rank, int64_t world, int64_t capacity, at::Tensor& err) {
  const c10::cuda::CUDAGuard guard(counts_all.device());
  const int E = counts_all.numel() / world, E_loc = E / world;
  TORCH_CHECK(E <= 64 && E % world == 0, "ep_plan: experts must divide evenly over the ranks (at most 64)");
  auto i32 = counts_all.options().dtype(at::kInt);
  const int max_tiles = (int)(capacity + 127) / 128 + E_loc;
  auto send_base = at::empty({E}, i32), recv_offsets = at::empty({E_loc + 1}, i32), sched = at::empty({1 + 3 * max_tiles}, i32), status = at::zeros({2}, i32);
  ep_plan_kernel<<<1, 64, 0, at::cuda::getCurrentCUDAStream()>>>(counts_all.data_ptr<int>(), (int)rank, (int)world, E, E_loc, (int)capacity, send_base.data_ptr<int>(),
                                                                 recv_offsets.data_ptr<int>(), sched.data_ptr<int>(), max_tiles, 128, status.data_ptr<int>(), err.data_ptr<int>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {send_base, recv_offsets, sched, status};
}

void ep_dispatch(const at::Tensor& src, const at::Tensor& perm, const at::Tensor& expert_of_pair, const at::Tensor& offsets, const at::Tensor& send_base,
                 int64_t K, int64_t E_loc, int64_t capacity, bool gather, int64_t rank, std::vector<int64_t> recv_rows, std::vector<int64_t> ret_rank,
                 std::vector<int64_t> ret_row) {
  TORCH_CHECK(src.is_cuda() && src.scalar_type() == at::kBFloat16 && src.is_contiguous() && src.size(1) % 8 == 0, "ep_dispatch: contiguous bf16 rows required");
  const c10::cuda::CUDAGuard guard(src.device());
  const int P = perm.numel(), h = src.size(1);
  if (P) ep_dispatch_kernel<<<(P + 7) / 8, 256, 0, at::cuda::getCurrentCUDAStream()>>>((const __nv_bfloat16*)src.data_ptr(), perm.data_ptr<int>(), expert_of_pair.data_ptr<int>(),
      offsets.data_ptr<int>(), send_base.data_ptr<int>(), P, (int)K, h, (int)E_loc, (int)capacity, gather ? 1 : 0, (int)rank, ep_ptrs(recv_rows), ep_ptrs(ret_rank), ep_ptrs(ret_row));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

}  // namespace q38
