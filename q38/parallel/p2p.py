"""Peer-memory transport of the gradient engine: CUDA-IPC mapped arenas + the kernels of `csrc/comm.cu`.

Every rank allocates its gradient arena, parameter arena, bf16 shadow, a flag array and a scalar array with `cudaMalloc`
(through the extension, so CUDA IPC handles can be taken), publishes the handles through `torch.distributed` and opens
the handles of all peers.  From then on a step's communication is three kernels on the compute stream and three
flag barriers; NCCL is only used for the bootstrap and for the few-byte metric averages.

    barrier                       all ranks finished backward
    reduce_scatter_mean           rank r: grads_r[seg r] = mean_p grads_p[seg r]          (peer loads, scale fused)
    allreduce_sum_scalar          squared gradient norm: publish to peers, barrier, sum in rank order
    (owner-computes optimizer step on segment r)
    all_gather_params + barrier   rank r stores its fp32 params[seg r] into every peer    (peer stores)

Waits inside the barrier kernel are bounded (`wait_seconds`); a missing peer surfaces as a `RuntimeError` from
`q38.ops.check_errors()` instead of a hang.  The rank whose wait ran out also raises an abort word in every peer's flag
array, and every kernel of the step that writes parameters, optimizer state or peer memory returns without writing once
the error word is set: a late rank cannot push parameters into a rank that has given up, and nobody steps on gradients
that were never reduced.
"""
import torch
import torch.distributed as dist

from .. import ops


class PeerTransport:
    def __init__(self, device, rank, world, wait_seconds=20.0):
        self.device, self.rank, self.world = torch.device(device), rank, world
        self.ops = ops.load()
        import os
        self.wait_seconds = float(os.environ.get("Q38_PEER_WAIT_SECONDS", wait_seconds))
        self.local = {}          # name -> uint8 tensor owning the allocation
        self.peers = {}          # name -> list of device pointers (own pointer at index rank)
        self.epoch = 0
        self.arena = None
        self._named = 0
        self.flags = self._alloc_raw("flags", 8 * 32).view(torch.int64)          # 16 peer slots + the device-side epoch counter
        self.scalars = self._alloc_raw("scalars", 8 * max(world, 16)).view(torch.float64)

    def _alloc_raw(self, name, nbytes):
        nbytes = (nbytes + 255) // 256 * 256
        buf = self.ops.p2p_alloc(nbytes, self.device.index)
        self.local[name] = buf
        return buf

    def allocate(self, numel, dtype):
        """Zero-filled flat tensor in peer-mappable memory (called by `ParamArena` for params, grads and shadow)."""
        name = ("params", "grads", "shadow")[self._named] if self._named < 3 else f"buf{self._named}"
        self._named += 1
        size = torch.empty((), dtype=dtype).element_size()
        return self._alloc_raw(name, numel * size)[:numel * size].view(dtype)

    def allocate_named(self, name, numel, dtype):
        size = torch.empty((), dtype=dtype).element_size()
        return self._alloc_raw(name, numel * size)[:numel * size].view(dtype)

    def bind(self, arena):
        """Exchange IPC handles of every local buffer and map the peers' buffers."""
        self.arena = arena
        self.exchange()

    def exchange(self):
        """Publish the handles of buffers allocated since the last exchange and map the peers' counterparts (collective)."""
        names = sorted(n for n in self.local if n not in self.peers)
        if not names:
            return
        mine = {n: bytes(self.ops.p2p_get_handle(self.local[n]).numpy().tobytes()) for n in names}
        gathered = [None] * self.world
        dist.all_gather_object(gathered, mine)
        for n in names:
            ptrs = []
            for r in range(self.world):
                if r == self.rank:
                    ptrs.append(self.local[n].data_ptr())
                else:
                    handle = torch.frombuffer(bytearray(gathered[r][n]), dtype=torch.uint8)
                    ptrs.append(int(self.ops.p2p_open_handle(handle, self.device.index)))
            self.peers[n] = ptrs
        dist.barrier()

    def barrier(self):
        """Cross-GPU barrier on the current stream.  The epoch lives in device memory, so the same launch can be captured in a
        CUDA graph and replayed; every rank must issue the same sequence of barriers."""
        self.ops.p2p_barrier(self.flags, self.peers["flags"], self.rank, -1, self.wait_seconds, ops.error_flag(self.device))

    def reduce_scatter_mean(self):
        self.barrier()
        s, e = self.arena.segments[self.rank]
        self.ops.p2p_reduce_scatter(self.peers["grads"], self.rank, s, e - s, 1.0 / self.world, self.device.index, ops.error_flag(self.device))

    def allreduce_sum_scalar(self, value):
        """`value`: 0-dim float64 device tensor.  Returns the sum over ranks, added in rank order on every rank."""
        self.ops.p2p_publish_scalar(value.reshape(1), self.peers["scalars"], self.rank)
        self.barrier()
        return self.scalars[:self.world].sum()

    def all_gather_params(self):
        s, e = self.arena.segments[self.rank]
        # fp32 only: the receivers derive the bf16 shadow themselves, a third fewer bytes over NVLink
        self.ops.p2p_all_gather(self.arena.params, None, self.peers["params"], [], self.rank, s, e - s, ops.error_flag(self.device))
        self.barrier()

    def reset_abort(self):
        """Clear the abort word after the host has handled a failed barrier (all ranks, between steps)."""
        self.flags[17] = 0

    def close(self):
        if not self.peers:
            return
        torch.cuda.synchronize(self.device)
        if dist.is_initialized():
            dist.barrier()
        for name, ptrs in self.peers.items():
            for r, ptr in enumerate(ptrs):
                if r != self.rank:
                    self.ops.p2p_close_handle(ptr, self.device.index)
        self.peers = {}
