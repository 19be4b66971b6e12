"""Peer-memory transport of the gradient engine: peer-mapped arenas + the kernels of `csrc/comm.cu`.

Every rank allocates its gradient arena, parameter arena, bf16 shadow, a flag array and a scalar array in memory that
the other GPUs can address.  Two allocation back ends:

  ``symm``  `torch.distributed._symmetric_memory` (driver virtual-memory API): besides the peers' addresses it yields a
            multicast address of each buffer when the NVSwitch supports it, which is what the NVLS kernels
            (`multimem.ld_reduce`, `multimem.st`) need.  Default when it comes up.
  ``ipc``   `cudaMalloc` + CUDA IPC handles published through `torch.distributed`.  No multicast; always available.
            Selected with ``Q38_PEER_ALLOC=ipc`` and used by the failure tests (a rank must not disappear while its
            memory is bound to a multicast object).

Reduce-scatter algorithms (``Q38_RS_ALGO`` = auto | nvls | pull | push; auto = nvls when a multicast address exists
and there are at least four ranks, else pull):
  ``pull``  one shot: rank r loads segment r from every peer and sums                 (world - 1 segments in over NVLink)
  ``push``  two shots: every rank stores its part of segment r into a slot on rank r, rank r sums its slots locally
  ``nvls``  the switch sums: rank r issues `multimem.ld_reduce` over segment r        (one segment in over NVLink)
The all-gather stores fp32 parameters into every peer (``pull``/``push``) or once to the multicast address (``nvls``).
From then on a step's communication is three kernels on the compute stream and three flag barriers; NCCL is only used
for the bootstrap and for the few-byte metric averages.

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

CANARY_BYTES, CANARY_BYTE = 256, 0xA5


class PeerTransport:
    def __init__(self, device, rank, world, wait_seconds=20.0):
        import os
        self.device, self.rank, self.world = torch.device(device), rank, world
        self.ops = ops.load()
        self.wait_seconds = float(os.environ.get("Q38_PEER_WAIT_SECONDS", wait_seconds))
        self.local = {}          # name -> uint8 tensor owning the allocation (payload + canary)
        self._payload = {}       # name -> payload bytes (the canary follows)
        self.peers = {}          # name -> list of device pointers (own pointer at index rank)
        self.multicast = {}      # name -> multicast address of the buffer (0 when there is none)
        self.epoch = 0
        self.arena = None
        self._named = 0
        self._handles = []
        self.alloc_backend = self._pick_alloc_backend(os.environ.get("Q38_PEER_ALLOC", "auto"))
        self.flags = self._alloc_raw("flags", 8 * 32).view(torch.int64)          # 16 peer slots, the epoch counter, the abort word
        self.scalars = self._alloc_raw("scalars", 8 * max(world, 16)).view(torch.float64)
        self.rs_algo = os.environ.get("Q38_RS_ALGO", "auto")
        self.staging = None

    def _pick_alloc_backend(self, wanted):
        if wanted == "ipc":
            return "ipc"
        works, why = 1, ""
        try:
            import torch.distributed._symmetric_memory as symm_mem
            probe = symm_mem.empty(256, dtype=torch.uint8, device=self.device)
            symm_mem.rendezvous(probe, dist.group.WORLD)
        except Exception as exc:
            works, why = 0, f"{type(exc).__name__}: {exc}"
        flag = torch.tensor([works], device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)              # every rank must take the same branch
        if int(flag.item()):
            return "symm"
        if wanted == "symm":
            raise RuntimeError(f"Q38_PEER_ALLOC=symm: symmetric memory did not come up on every rank ({why or 'another rank failed'})")
        if self.rank == 0:
            print(f"[q38.p2p] symmetric memory is unavailable ({why or 'another rank failed'}); using CUDA IPC allocations", flush=True)
        return "ipc"

    def _alloc_raw(self, name, nbytes):
        """A buffer of at least `nbytes` in peer-mappable memory, followed by a 256-byte canary: peers write into these buffers
        by raw address (reduce-scatter staging, parameter all-gather), so an overrun would land in whatever the allocator put
        next; `check_canaries` finds it instead."""
        nbytes = (nbytes + 255) // 256 * 256
        total = nbytes + CANARY_BYTES
        if self.alloc_backend == "symm":
            import torch.distributed._symmetric_memory as symm_mem
            buf = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
            buf.zero_()
        else:
            buf = self.ops.p2p_alloc(total, self.device.index)
        buf[nbytes:].fill_(CANARY_BYTE)
        self.local[name] = buf
        self._payload[name] = nbytes
        return buf[:nbytes]

    def check_canaries(self):
        """Raise if the guard bytes after any peer-mapped buffer of this rank were overwritten (by this rank or by a peer)."""
        for name, buf in self.local.items():
            tail = buf[self._payload[name]:]
            if not bool((tail == CANARY_BYTE).all()):
                bad = int((tail != CANARY_BYTE).nonzero()[0])
                raise RuntimeError(f"peer buffer '{name}' of rank {self.rank} was overrun: guard byte {bad} after its {self._payload[name]} bytes changed")

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
        """Exchange the addresses of every local buffer and map the peers' buffers."""
        self.arena = arena
        self.exchange()
        if self.rs_algo == "auto":
            # with two ranks a peer load moves one segment, exactly what the switch reduction would deliver; the switch pays
            # off from four ranks on, where it replaces world - 1 incoming copies by one
            have_mc = bool(self.multicast.get("grads") and self.multicast.get("params"))
            self.rs_algo = "nvls" if (have_mc and self.world >= 4) else "pull"
        if self.rs_algo == "nvls" and not (self.multicast.get("grads") and self.multicast.get("params")):
            raise RuntimeError("Q38_RS_ALGO=nvls needs multicast addresses of the arenas (symmetric-memory allocations on an NVSwitch system)")
        if self.rs_algo == "push":
            longest = max(e - s for s, e in arena.segments)
            self.slot_stride = (longest + 63) // 64 * 64
            self.staging = self.allocate_named("rs_staging", self.world * self.slot_stride, torch.float32)
            self.exchange()

    def exchange(self):
        """Publish the buffers allocated since the last exchange and map the peers' counterparts (collective)."""
        names = sorted(n for n in self.local if n not in self.peers)
        if not names:
            return
        if self.alloc_backend == "symm":
            import torch.distributed._symmetric_memory as symm_mem
            torch.cuda.synchronize(self.device)
            for n in names:
                handle = symm_mem.rendezvous(self.local[n], dist.group.WORLD)
                self._handles.append(handle)
                self.peers[n] = [int(p) for p in handle.buffer_ptrs]
                self.multicast[n] = int(getattr(handle, "multicast_ptr", 0) or 0)
            dist.barrier()
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
            self.multicast[n] = 0
        dist.barrier()

    def barrier(self):
        """Cross-GPU barrier on the current stream.  The epoch lives in device memory, so the same launch can be captured in a
        CUDA graph and replayed; every rank must issue the same sequence of barriers."""
        self.ops.p2p_barrier(self.flags, self.peers["flags"], self.rank, -1, self.wait_seconds, ops.error_flag(self.device))

    def reduce_scatter_mean(self):
        self.barrier()
        s, e = self.arena.segments[self.rank]
        err = ops.error_flag(self.device)
        if self.rs_algo == "nvls":
            self.ops.nvls_reduce_scatter(self.multicast["grads"], self.arena.grads, s, e - s, 1.0 / self.world, err)
        elif self.rs_algo == "push":
            starts = [a for a, _ in self.arena.segments]
            counts = [b - a for a, b in self.arena.segments]
            self.ops.p2p_push_segments(self.arena.grads, self.peers["rs_staging"], starts, counts, self.slot_stride, self.rank, err)
            self.barrier()
            self.ops.p2p_reduce_staged(self.arena.grads, self.staging, self.slot_stride, self.rank, self.world, s, e - s, 1.0 / self.world, err)
        else:
            self.ops.p2p_reduce_scatter(self.peers["grads"], self.rank, s, e - s, 1.0 / self.world, self.device.index, err)

    def allreduce_sum_scalar(self, value):
        """`value`: 0-dim float64 device tensor.  Returns the sum over ranks, added in rank order on every rank."""
        self.ops.p2p_publish_scalar(value.reshape(1), self.peers["scalars"], self.rank)
        self.barrier()
        return self.scalars[:self.world].sum()

    def all_gather_params(self):
        s, e = self.arena.segments[self.rank]
        # fp32 only: the receivers derive the bf16 shadow themselves, a third fewer bytes over NVLink
        if self.rs_algo == "nvls":
            self.ops.nvls_all_gather(self.arena.params, self.multicast["params"], s, e - s, ops.error_flag(self.device))
        else:
            self.ops.p2p_all_gather(self.arena.params, None, self.peers["params"], [], self.rank, s, e - s, ops.error_flag(self.device))
        self.barrier()

    def reset_abort(self):
        """Clear the abort word after the host has handled a failed barrier (all ranks, between steps)."""
        self.flags[17] = 0

    def close(self):
        if not self.peers:
            return
        torch.cuda.synchronize(self.device)
        self.check_canaries()
        if dist.is_initialized():
            dist.barrier()
        if self.alloc_backend == "ipc":
            for name, ptrs in self.peers.items():
                for r, ptr in enumerate(ptrs):
                    if r != self.rank:
                        self.ops.p2p_close_handle(ptr, self.device.index)
        self.peers, self.multicast, self._handles = {}, {}, []
