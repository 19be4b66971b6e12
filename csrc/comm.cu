// Peer-memory collectives for the data-parallel gradient path: every rank maps the other ranks' gradient / parameter
// arenas (cudaMalloc + CUDA IPC handles over NVLink) and the kernels below read and write them directly.
//
//   p2p_barrier          flag barrier across GPUs: rank r stores `epoch` into slot r of every peer's flag array (after a
//                        system-scope fence) and waits until all slots of its own array reached `epoch`.
//   p2p_reduce_scatter   rank r replaces segment r of its gradient arena by scale * sum_p grads_p[segment r]; the cast /
//                        mean scaling is fused into the reduction and the summation order is the same on every rank.
//   p2p_all_gather       rank r stores its updated fp32 parameters and bf16 shadow of segment r into every peer's arenas.
//   p2p_publish_scalar   writes one double into slot r of every peer's scalar array (global gradient norm).
//
//   *_nvls               the same two transfers through the NVSwitch: `multimem.ld_reduce` sums the segment over all GPUs
//                        inside the switch (each rank receives one copy instead of world - 1), `multimem.st` writes the
//                        updated parameters to every GPU with one store.  They need a multicast mapping of the arenas.
//   p2p_push_segments /  push variant of the reduce-scatter: every rank stores its contribution to segment r into a
//   p2p_reduce_staged    staging slot on rank r (posted writes), then rank r sums the slots locally in rank order.
//
// Every wait is bounded by a clock budget; on expiry the kernel records ERR_PEER_WAIT and returns, the context stays
// usable and the host raises.  Loads from peers are plain or multimem (no TMA, no cluster multicast).
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"
#include "host.h"

namespace q38 {

constexpr int MAX_PEERS = 16;

struct PeerPtrs { void* p[MAX_PEERS]; };

__device__ __forceinline__ long long ld_volatile_ll(const long long* p) {
  long long v;
  asm volatile("ld.volatile.global.s64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// Layout of a rank's flag array (int64 words): [0, MAX_PEERS) arrival slots written by the peers, [MAX_PEERS] the
// device-side epoch counter, [MAX_PEERS + 1] the abort word.
constexpr int FLAG_EPOCH = MAX_PEERS, FLAG_ABORT = MAX_PEERS + 1;

// One CTA of 32 threads.  wait_cycles bounds the spin (about a second at 2 GHz by default).
// epoch < 0: take the next value of the device-side counter own_flags[FLAG_EPOCH] (all ranks execute the same sequence
// of barriers, so the counters stay in lockstep; this form can be captured in a CUDA graph and replayed).
// A rank whose wait runs out records ERR_PEER_WAIT and raises the abort word of every peer; a rank that finds its abort
// word raised (on entry or while it waits) records the same error.  Kernels that write parameters, optimizer state or
// peer memory return without writing once the error word is set, so a late or missing rank cannot make the others step
// on unreduced gradients or tear a checkpoint that is being written.
__global__ void p2p_barrier_kernel(long long* __restrict__ own_flags, PeerPtrs peers, int rank, int world, long long epoch,
                                   long long wait_cycles, int* __restrict__ err) {
  const int t = threadIdx.x;
  __shared__ long long next;
  __shared__ int failed;
  if (t == 0) failed = 0;
  if (epoch < 0) {
    if (t == 0) { next = own_flags[FLAG_EPOCH] + 1; own_flags[FLAG_EPOCH] = next; }
    __syncthreads();
    epoch = next;
  }
  __syncthreads();
  __threadfence_system();                                  // everything this GPU wrote before the barrier is visible first
  if (t < world) {
    long long* dst = reinterpret_cast<long long*>(peers.p[t]) + rank;
    asm volatile("st.volatile.global.s64 [%0], %1;" ::"l"(dst), "l"(epoch) : "memory");
  }
  if (t < world) {
    const long long start = clock64();
    bool ok = false;
    while (clock64() - start < wait_cycles) {
      if (ld_volatile_ll(own_flags + FLAG_ABORT) != 0) break;
      if (ld_volatile_ll(own_flags + t) >= epoch) { ok = true; break; }
      __nanosleep(200);
    }
    if (!ok) { report_error(err, ERR_PEER_WAIT); failed = 1; }
  }
  __syncthreads();
  if (failed && t < world) {
    long long* dst = reinterpret_cast<long long*>(peers.p[t]) + FLAG_ABORT;
    asm volatile("st.volatile.global.s64 [%0], %1;" ::"l"(dst), "l"(1LL) : "memory");
  }
  __threadfence_system();
}

__device__ __forceinline__ bool aborted(const int* err) {
  if (err == nullptr) return false;
  int v;
  asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(err) : "memory");
  return v != 0;
}

// own[i] = scale * sum_p grads_p[i] for i in [start, start + count); 16-byte loads; count and start multiples of 4.
__global__ void __launch_bounds__(256) p2p_reduce_scatter_kernel(PeerPtrs grads, int rank, int world, long long start, long long count, float scale,
                                                                 const int* __restrict__ err) {
  if (aborted(err)) return;
  const float4* src[MAX_PEERS];
#pragma unroll
  for (int p = 0; p < MAX_PEERS; ++p) src[p] = p < world ? reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[p]) + start) : nullptr;
  float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(grads.p[rank]) + start);
  const long long n4 = count / 4;
  // two 16-byte elements per thread and step: twice the loads in flight per thread on a path whose latency is a NVLink round trip
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += 2 * stride) {
    const long long j = i + stride;
    const bool second = j < n4;
    float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
#pragma unroll
    for (int p = 0; p < MAX_PEERS; ++p) {
      if (p < world) {
        const float4 v = src[p][i];
        a0.x += v.x; a0.y += v.y; a0.z += v.z; a0.w += v.w;
        if (second) { const float4 w = src[p][j]; a1.x += w.x; a1.y += w.y; a1.z += w.z; a1.w += w.w; }
      }
    }
    dst[i] = make_float4(a0.x * scale, a0.y * scale, a0.z * scale, a0.w * scale);
    if (second) dst[j] = make_float4(a1.x * scale, a1.y * scale, a1.z * scale, a1.w * scale);
  }
}

// Push segment [start, start + count) of the local fp32 parameters (and bf16 shadow) into every peer's arenas.
__global__ void __launch_bounds__(256) p2p_all_gather_kernel(const float* __restrict__ params, const __nv_bfloat16* __restrict__ shadow, PeerPtrs peer_params,
                                                             PeerPtrs peer_shadow, int rank, int world, long long start, long long count,
                                                             const int* __restrict__ err) {
  if (aborted(err)) return;
  const long long n4 = count / 4;
  const float4* src = reinterpret_cast<const float4*>(params + start);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 v = src[i];
    uint2 packed;
    {
      __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
      packed.x = *reinterpret_cast<uint32_t*>(&lo); packed.y = *reinterpret_cast<uint32_t*>(&hi);
    }
#pragma unroll
    for (int p = 0; p < MAX_PEERS; ++p) {
      if (p < world && p != rank) {
        reinterpret_cast<float4*>(reinterpret_cast<float*>(peer_params.p[p]) + start)[i] = v;
        if (shadow != nullptr) reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(peer_shadow.p[p]) + start)[i] = packed;
      }
    }
  }
}

// ---- NVLS: reductions and broadcasts performed by the NVSwitch on a multicast address ------------------------------------------
__device__ __forceinline__ float4 multimem_ld_reduce_add(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st(float* mc, const float4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// own[i] = scale * (sum over all GPUs of grads[i]) for i in [start, start + count), the sum taken by the switch.
__global__ void __launch_bounds__(256) nvls_reduce_scatter_kernel(const float* __restrict__ mc_grads, float* __restrict__ own, long long start, long long count,
                                                                  float scale, const int* __restrict__ err) {
  if (aborted(err)) return;
  const long long n4 = count / 4, stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += 2 * stride) {
    const long long j = i + stride;
    float4 v = multimem_ld_reduce_add(mc_grads + start + 4 * i);
    float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
    if (j < n4) w = multimem_ld_reduce_add(mc_grads + start + 4 * j);
    v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale;
    reinterpret_cast<float4*>(own + start)[i] = v;
    if (j < n4) { w.x *= scale; w.y *= scale; w.z *= scale; w.w *= scale; reinterpret_cast<float4*>(own + start)[j] = w; }
  }
}

// Every GPU's params[i] = this rank's params[i] for i in [start, start + count): one multicast store per 16 bytes.
__global__ void __launch_bounds__(256) nvls_all_gather_kernel(const float* __restrict__ params, float* __restrict__ mc_params, long long start, long long count,
                                                              const int* __restrict__ err) {
  if (aborted(err)) return;
  const long long n4 = count / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x)
    multimem_st(mc_params + start + 4 * i, reinterpret_cast<const float4*>(params + start)[i]);
}

// ---- push variant of the reduce-scatter --------------------------------------------------------------------------------------------
struct SegmentTable { long long start[MAX_PEERS]; long long count[MAX_PEERS]; long long slot_stride; };

// For every peer p != rank: staging_p[rank * slot_stride + i] = grads[start_p + i], i < count_p.  blockIdx.y walks the peers.
__global__ void __launch_bounds__(256) p2p_push_segments_kernel(const float* __restrict__ grads, PeerPtrs staging, SegmentTable seg, int rank, int world,
                                                                const int* __restrict__ err) {
  if (aborted(err)) return;
  const int p = blockIdx.y;
  if (p >= world || p == rank) return;
  const float4* src = reinterpret_cast<const float4*>(grads + seg.start[p]);
  float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(staging.p[p]) + (long long)rank * seg.slot_stride);
  const long long n4 = seg.count[p] / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) dst[i] = src[i];
}

// own[start + i] = scale * (sum over ranks q in rank order of (q == rank ? own[start + i] : staging[q * slot_stride + i]))
__global__ void __launch_bounds__(256) p2p_reduce_staged_kernel(float* __restrict__ own, const float* __restrict__ staging, long long slot_stride, int rank, int world,
                                                                long long start, long long count, float scale, const int* __restrict__ err) {
  if (aborted(err)) return;
  const long long n4 = count / 4;
  float4* dst = reinterpret_cast<float4*>(own + start);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int q = 0; q < world; ++q) {
      const float4 v = q == rank ? dst[i] : reinterpret_cast<const float4*>(staging + (long long)q * slot_stride)[i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    dst[i] = make_float4(acc.x * scale, acc.y * scale, acc.z * scale, acc.w * scale);
  }
}

// shadow[i] = bf16(params[i]) for every i outside [skip_start, skip_start + skip_count): after the all-gather has delivered the
// peers' fp32 segments, each rank derives their bf16 copies locally instead of receiving them over NVLink.
__global__ void __launch_bounds__(256) cast_shadow_except_kernel(const float* __restrict__ params, __nv_bfloat16* __restrict__ shadow, long long n4,
                                                                 long long skip_lo4, long long skip_hi4, const int* __restrict__ err) {
  if (aborted(err)) return;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    if (i >= skip_lo4 && i < skip_hi4) continue;
    const float4 v = reinterpret_cast<const float4*>(params)[i];
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 packed;
    packed.x = *reinterpret_cast<const uint32_t*>(&lo); packed.y = *reinterpret_cast<const uint32_t*>(&hi);
    reinterpret_cast<uint2*>(shadow)[i] = packed;
  }
}

__global__ void p2p_publish_scalar_kernel(const double* __restrict__ value, PeerPtrs slots, int rank, int world) {
  const int t = threadIdx.x;
  if (t < world) reinterpret_cast<double*>(slots.p[t])[rank] = *value;
}

// ---- host: allocation and IPC ------------------------------------------------------------------------------------------------
at::Tensor p2p_alloc(int64_t nbytes, int64_t device) {
  const c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
  void* ptr = nullptr;
  C10_CUDA_CHECK(cudaMalloc(&ptr, (size_t)nbytes));
  C10_CUDA_CHECK(cudaMemset(ptr, 0, (size_t)nbytes));
  return at::from_blob(ptr, {nbytes}, [](void* p) { cudaFree(p); }, at::TensorOptions().dtype(at::kByte).device(at::kCUDA, (c10::DeviceIndex)device));
}

at::Tensor p2p_get_handle(const at::Tensor& t) {
  cudaIpcMemHandle_t h;
  C10_CUDA_CHECK(cudaIpcGetMemHandle(&h, t.data_ptr()));
  auto out = at::empty({(int64_t)sizeof(h)}, at::TensorOptions().dtype(at::kByte));
  std::memcpy(out.data_ptr(), &h, sizeof(h));
  return out;
}

int64_t p2p_open_handle(const at::Tensor& handle, int64_t device) {
  const c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
  TORCH_CHECK(handle.numel() == (int64_t)sizeof(cudaIpcMemHandle_t), "p2p_open_handle: bad handle size");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle.data_ptr(), sizeof(h));
  void* ptr = nullptr;
  C10_CUDA_CHECK(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return reinterpret_cast<int64_t>(ptr);
}

void p2p_close_handle(int64_t ptr, int64_t device) {
  const c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
  cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr));
}

static PeerPtrs to_ptrs(const std::vector<int64_t>& v) {
  TORCH_CHECK((int)v.size() <= MAX_PEERS, "at most 16 peers");
  PeerPtrs p{};
  for (size_t i = 0; i < v.size(); ++i) p.p[i] = reinterpret_cast<void*>(v[i]);
  return p;
}

void p2p_barrier(at::Tensor& own_flags, std::vector<int64_t> peer_flags, int64_t rank, int64_t epoch, double wait_seconds, at::Tensor& err) {
  const c10::cuda::CUDAGuard guard(own_flags.device());
  const long long cycles = (long long)(wait_seconds * 1.9e9);
  p2p_barrier_kernel<<<1, 32, 0, at::cuda::getCurrentCUDAStream()>>>(reinterpret_cast<long long*>(own_flags.data_ptr()), to_ptrs(peer_flags), (int)rank,
                                                                     (int)peer_flags.size(), (long long)epoch, cycles, err.data_ptr<int>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

void p2p_reduce_scatter(std::vector<int64_t> grads, int64_t rank, int64_t start, int64_t count, double scale, int64_t device,
                        const c10::optional<at::Tensor>& err) {
  const c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
  TORCH_CHECK(start % 4 == 0 && count % 4 == 0, "p2p_reduce_scatter: segment must be 16-byte aligned");
  if (count == 0) return;
  const int grid = (int)std::min<int64_t>((count / 4 + 255) / 256, kNumSMs * 8);
  p2p_reduce_scatter_kernel<<<grid, 256, 0, at::cuda::getCurrentCUDAStream()>>>(to_ptrs(grads), (int)rank, (int)grads.size(), start, count, (float)scale,
                                                                                err.has_value() ? err->data_ptr<int>() : nullptr);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

void p2p_all_gather(const at::Tensor& params, const c10::optional<at::Tensor>& shadow, std::vector<int64_t> peer_params, std::vector<int64_t> peer_shadow,
                    int64_t rank, int64_t start, int64_t count, const c10::optional<at::Tensor>& err) {
  const c10::cuda::CUDAGuard guard(params.device());
  TORCH_CHECK(start % 4 == 0 && count % 4 == 0, "p2p_all_gather: segment must be 16-byte aligned");
  if (count == 0) return;
  const int grid = (int)std::min<int64_t>((count / 4 + 255) / 256, kNumSMs * 8);
  p2p_all_gather_kernel<<<grid, 256, 0, at::cuda::getCurrentCUDAStream()>>>(params.data_ptr<float>(),
      shadow.has_value() ? (const __nv_bfloat16*)shadow->data_ptr() : nullptr, to_ptrs(peer_params), to_ptrs(peer_shadow), (int)rank,
      (int)peer_params.size(), start, count, err.has_value() ? err->data_ptr<int>() : nullptr);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

static int stream_grid(long long count) { return (int)std::min<int64_t>((count / 4 + 255) / 256, kNumSMs * 8); }
static const int* err_or_null(const c10::optional<at::Tensor>& err) { return err.has_value() ? err->data_ptr<int>() : nullptr; }

void nvls_reduce_scatter(int64_t mc_grads, at::Tensor& grads, int64_t start, int64_t count, double scale, const c10::optional<at::Tensor>& err) {
  TORCH_CHECK(mc_grads != 0 && (mc_grads & 15) == 0, "nvls_reduce_scatter: a 16-byte aligned multicast address is required");
  TORCH_CHECK(grads.is_cuda() && grads.scalar_type() == at::kFloat && grads.is_contiguous() && start % 4 == 0 && count % 4 == 0 && start + count <= grads.numel(),
              "nvls_reduce_scatter: flat fp32 arena and a 16-byte aligned segment inside it required");
  if (count == 0) return;
  const c10::cuda::CUDAGuard guard(grads.device());
  nvls_reduce_scatter_kernel<<<stream_grid(count), 256, 0, at::cuda::getCurrentCUDAStream()>>>(reinterpret_cast<const float*>(mc_grads), grads.data_ptr<float>(), start,
                                                                                                 count, (float)scale, err_or_null(err));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

void nvls_all_gather(const at::Tensor& params, int64_t mc_params, int64_t start, int64_t count, const c10::optional<at::Tensor>& err) {
  TORCH_CHECK(mc_params != 0 && (mc_params & 15) == 0, "nvls_all_gather: a 16-byte aligned multicast address is required");
  TORCH_CHECK(params.is_cuda() && params.scalar_type() == at::kFloat && params.is_contiguous() && start % 4 == 0 && count % 4 == 0 && start + count <= params.numel(),
              "nvls_all_gather: flat fp32 arena and a 16-byte aligned segment inside it required");
  if (count == 0) return;
  const c10::cuda::CUDAGuard guard(params.device());
  nvls_all_gather_kernel<<<stream_grid(count), 256, 0, at::cuda::getCurrentCUDAStream()>>>(params.data_ptr<float>(), reinterpret_cast<float*>(mc_params), start, count,
                                                                                             err_or_null(err));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

void p2p_push_segments(const at::Tensor& grads, std::vector<int64_t> peer_staging, std::vector<int64_t> starts, std::vector<int64_t> counts, int64_t slot_stride,
                       int64_t rank, const c10::optional<at::Tensor>& err) {
  const int world = (int)peer_staging.size();
  TORCH_CHECK(world <= MAX_PEERS && (int)starts.size() == world && (int)counts.size() == world && slot_stride % 4 == 0, "p2p_push_segments: bad segment table");
  SegmentTable seg{};
  long long longest = 0;
  for (int p = 0; p < world; ++p) {
    TORCH_CHECK(starts[p] % 4 == 0 && counts[p] % 4 == 0 && counts[p] <= slot_stride, "p2p_push_segments: segments must be 16-byte aligned and fit a staging slot");
    seg.start[p] = starts[p]; seg.count[p] = counts[p];
    longest = std::max<long long>(longest, counts[p]);
  }
  seg.slot_stride = slot_stride;
  if (longest == 0) return;
  const c10::cuda::CUDAGuard guard(grads.device());
  const int gx = std::max(1, std::min<int>((int)((longest / 4 + 255) / 256), kNumSMs * 8 / std::max(1, world - 1)));
  p2p_push_segments_kernel<<<dim3(gx, world), 256, 0, at::cuda::getCurrentCUDAStream()>>>(grads.data_ptr<float>(), to_ptrs(peer_staging), seg, (int)rank, world,
                                                                                            err_or_null(err));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

void p2p_reduce_staged(at::Tensor& grads, const at::Tensor& staging, int64_t slot_stride, int64_t rank, int64_t world, int64_t start, int64_t count, double scale,
                       const c10::optional<at::Tensor>& err) {
  TORCH_CHECK(grads.scalar_type() == at::kFloat && staging.scalar_type() == at::kFloat && staging.numel() >= world * slot_stride && start % 4 == 0 && count % 4 == 0 &&
              count <= slot_stride, "p2p_reduce_staged: fp32 arena, staging of world slots and an aligned segment required");
  if (count == 0) return;
  const c10::cuda::CUDAGuard guard(grads.device());
  p2p_reduce_staged_kernel<<<stream_grid(count), 256, 0, at::cuda::getCurrentCUDAStream()>>>(grads.data_ptr<float>(), staging.data_ptr<float>(), slot_stride, (int)rank,
                                                                                               (int)world, start, count, (float)scale, err_or_null(err));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

void cast_shadow_except(const at::Tensor& params, at::Tensor& shadow, int64_t skip_start, int64_t skip_count, const c10::optional<at::Tensor>& err) {
  TORCH_CHECK(params.is_cuda() && params.scalar_type() == at::kFloat && shadow.scalar_type() == at::kBFloat16 && params.numel() == shadow.numel() &&
              params.is_contiguous() && shadow.is_contiguous(), "cast_shadow_except: flat fp32 parameters and a bf16 shadow of the same length required");
  TORCH_CHECK(params.numel() % 4 == 0 && skip_start % 4 == 0 && skip_count % 4 == 0, "cast_shadow_except: lengths must be multiples of 4");
  const c10::cuda::CUDAGuard guard(params.device());
  const long long n4 = params.numel() / 4;
  if (!n4) return;
  const int grid = (int)std::min<int64_t>((n4 + 255) / 256, kNumSMs * 8);
  cast_shadow_except_kernel<<<grid, 256, 0, at::cuda::getCurrentCUDAStream()>>>(params.data_ptr<float>(), (__nv_bfloat16*)shadow.data_ptr(), n4, skip_start / 4,
                                                                                (skip_start + skip_count) / 4, err.has_value() ? err->data_ptr<int>() : nullptr);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

void p2p_publish_scalar(const at::Tensor& value, std::vector<int64_t> peer_slots, int64_t rank) {
  const c10::cuda::CUDAGuard guard(value.device());
  TORCH_CHECK(value.scalar_type() == at::kDouble && value.numel() == 1, "p2p_publish_scalar: one double required");
  p2p_publish_scalar_kernel<<<1, 32, 0, at::cuda::getCurrentCUDAStream()>>>(value.data_ptr<double>(), to_ptrs(peer_slots), (int)rank, (int)peer_slots.size());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

}  // namespace q38
