"""Data-parallel gradient engine with owner-computes optimizer.

One optimizer step on `world` ranks:

1. every rank accumulates its micro-batch gradients into its flat gradient arena (`ParamArena`);
2. **reduce-scatter**: rank r obtains the mean over ranks of segment r of the gradient arena;
3. the global gradient norm is the root of the all-reduced sum of the per-segment squared norms; the
   clip coefficient ``min(1, clip / (norm + 1e-6))`` is folded into the update;
4. **owner computes**: rank r runs AdamW / Muon on the parameters of segment r only;
5. **all-gather**: rank r publishes its updated fp32 parameters (and bf16 shadow) to every rank.

Replicas are bit-identical after every step because each parameter is updated by exactly one rank from
one reduced gradient and then copied.  The result equals DDP with replicated optimizers up to the
summation order of the gradient mean (reference: DDP wiring at q38/train.py:472-479, update order
clip -> AdamW -> Muon at q38/train.py:558-559).

Transports
  ``p2p``         hand-written sm_100a kernels reading/writing peer GPUs' arenas over NVLink
                  (`q38.parallel.p2p`), launched on the compute stream after the last micro-step.  Only fp32 parameters
                  cross NVLink in the all-gather; every rank derives the bf16 shadow of the received segments locally.
  ``collective``  `torch.distributed` reduce / broadcast per segment (NCCL on GPUs, gloo on CPU).  This is the
                  baseline transport and the one the CPU multi-process tests exercise.
"""
import torch
import torch.distributed as dist

from ..optim.hybrid import HybridOptimizer
from .arena import ParamArena


class GradEngine:
    def __init__(self, model, device, rank=0, world=1, mode="auto", lr=1e-3, weight_decay=0.1, muon=True, expert_parallel=False):
        self.model, self.device, self.rank, self.world = model, torch.device(device), rank, world
        self.expert_parallel = bool(expert_parallel) and world > 1
        if self.expert_parallel and not muon:
            raise ValueError("expert parallelism keeps the experts in the Muon group; run it with --muon 1")
        if mode == "auto":
            mode = "p2p" if (world > 1 and self.device.type == "cuda") else "collective"
        self.mode = mode
        self.transport = None
        allocate = None
        if self.expert_parallel and mode != "p2p":
            raise ValueError("expert parallelism needs the peer-memory transport (--grad_sync p2p on GPUs)")
        if world > 1 and mode == "p2p":
            from .p2p import PeerTransport
            self.transport = PeerTransport(self.device, rank, world)
            allocate = self.transport.allocate
        if world > 1:
            # rank 0's initial weights win, as with DDP's construction-time broadcast
            for p in model.parameters():
                dist.broadcast(p.data, 0)
        local_filter = (lambda name: ".mlp.experts." in name) if self.expert_parallel else None
        self.arena = ParamArena(model, self.device, world, muon=muon, allocate=allocate, local_filter=local_filter)
        self.optimizer = HybridOptimizer(model, lr=lr, weight_decay=weight_decay, muon=muon, arena=self.arena, rank=rank)
        if self.transport is not None:
            self.transport.bind(self.arena)
        self._last = True
        # CUDA events around the phases of `finish_step` (a handful per step; Q38_ENGINE_TIMING=0 turns them off)
        import os
        self._timing = [] if (os.environ.get("Q38_ENGINE_TIMING", "1") != "0" and self.device.type == "cuda") else None

    # ------------------------------------------------------------------ step protocol
    def set_lr(self, lr):
        for group in self.optimizer.param_groups:
            group["lr"] = lr

    def begin_micro_step(self, last):
        self._last = last

    def zero_grad(self):
        self.arena.zero_grad()

    def _reduce_scatter(self):
        if self.world == 1:
            return
        if self.transport is not None:
            self.transport.reduce_scatter_mean()
            return
        for owner, (s, e) in enumerate(self.arena.segments):
            if e > s:
                dist.reduce(self.arena.grads[s:e], dst=owner, op=dist.ReduceOp.SUM)
        s, e = self.arena.segments[self.rank]
        self.arena.grads[s:e].div_(self.world)

    def _fused_updates(self):
        """True when the update kernels write the bf16 shadow of what they update (GPU, fused optimizer kernels)."""
        import os
        return self.device.type == "cuda" and not os.environ.get("Q38_MUON_BASELINE")

    def _all_gather(self):
        fused = self._fused_updates()
        if self.world == 1:
            if not fused:
                self.arena.refresh_shadow()
            return
        s, e = self.arena.segments[self.rank]
        if self.transport is not None:
            if not fused:
                self.arena.refresh_shadow(self.rank)
            self.transport.all_gather_params()
            self._cast_received(s, e)
            return
        for owner, (s0, e0) in enumerate(self.arena.segments):
            if e0 > s0:
                dist.broadcast(self.arena.params[s0:e0], src=owner)
        if fused:
            self._cast_received(s, e)
        else:
            self.arena.refresh_shadow()

    def _cast_received(self, s, e):
        """bf16 shadow of every segment except this rank's own (already written by the update kernels)."""
        from .. import ops
        local = self.arena.local_range
        end = local[0] if local[1] > local[0] else self.arena.numel
        ops.load().cast_shadow_except(self.arena.params[:end], self.arena.shadow[:end], s, e - s, ops.error_flag(self.device))

    def _local_grad_slices(self):
        """This rank's slices of the expert-parallel gradient tensors."""
        out = []
        for unit in self.arena.local_units():
            n = unit.param.shape[0] // self.world
            out.append(unit.param.grad[self.rank * n:(self.rank + 1) * n])
        return out

    def grad_norm(self):
        s, e = self.arena.segments[self.rank]
        sq = self.arena.grads[s:e].double().pow(2).sum() if self.device.type == "cpu" else self._sumsq(s, e)
        for g in self._local_grad_slices():
            g.mul_(1.0 / self.world)                      # tokens of all ranks are already summed in: scale to the data-parallel mean
            sq = sq + g.double().pow(2).sum()
        if self.world > 1:
            if self.transport is not None:
                sq = self.transport.allreduce_sum_scalar(sq)
            else:
                sq = sq.clone()
                dist.all_reduce(sq)
        return sq.sqrt().float()

    def _sumsq(self, s, e):
        from .. import ops
        return ops.sum_squares(self.arena.grads[s:e])

    def finish_step(self, clip):
        """Reduce, clip, update owned parameters, publish them, clear gradients.  Returns the pre-clip gradient norm.
        With Q38_ENGINE_TIMING=1 on a GPU the phases are bracketed by CUDA events and `phase_times()` reports their means."""
        mark = self._mark
        mark("start")
        self._reduce_scatter()
        mark("reduce_scatter")
        norm = self.grad_norm()
        scale = None
        if clip and clip > 0:
            scale = (clip / (norm + 1e-6)).clamp(max=1.0)
        mark("grad_norm")
        self.optimizer.step(grad_scale=scale)
        mark("optimizer")
        self._all_gather()
        mark("all_gather")
        self.zero_grad()
        mark("zero_grad")
        return norm

    def _mark(self, name):
        if self._timing is None:
            return
        event = torch.cuda.Event(enable_timing=True)
        event.record()
        self._timing.append((name, event))

    def phase_times(self):
        """Median milliseconds per phase of `finish_step` over the steps recorded so far; the median ignores the first
        steps, whose device timeline contains host-side lazy initialisation and graph capture."""
        if not self._timing:
            return {}
        torch.cuda.synchronize(self.device)
        samples = {}
        for (_, e0), (name, e1) in zip(self._timing, self._timing[1:]):
            if name != "start":
                samples.setdefault(name, []).append(e0.elapsed_time(e1))
        self._timing = self._timing[-64:]
        return {k: round(sorted(v)[len(v) // 2], 3) for k, v in samples.items()}

    def comm_report(self, link_gbs=770.0):
        """Exposed communication of a step and how close it runs to the NVLink roofline.

        Nothing of `finish_step` overlaps with compute, so the exposed communication time is the sum of the reduce-scatter
        and all-gather phases (barriers included).  Both phases end when the busiest link direction of any rank is through,
        so the byte counts are maxima over ranks: the reduce-scatter brings the largest segment in from every peer (with the
        in-switch reduction the same bytes leave the peers); the all-gather brings every other segment into each rank and
        sends the largest segment out, once through the switch's multicast or once per peer with plain stores.
        `link_gbs` is the measured peer-copy bandwidth per direction."""
        times = self.phase_times()
        if self.world == 1 or not times:
            return {"exposed_comm_ms": 0.0, "comm_roofline_fraction": None}
        sizes = [e - s for s, e in self.arena.segments]
        multicast = "nvls" in self.describe_transport()
        rs_bytes = (self.world - 1) * max(sizes) * 4
        ag_bytes = max((sum(sizes) - min(sizes)) * 4, max(sizes) * 4 * (1 if multicast else self.world - 1))
        rs, ag = times.get("reduce_scatter", 0.0), times.get("all_gather", 0.0)
        frac = lambda nbytes, ms: round(nbytes / (link_gbs * 1e9 * ms * 1e-3), 3) if ms > 0 else None
        return {"exposed_comm_ms": round(rs + ag, 3), "nvlink_bytes_reduce_scatter": rs_bytes, "nvlink_bytes_all_gather": ag_bytes,
                "largest_segment_over_mean": round(max(sizes) * self.world / max(1, sum(sizes)), 3),
                "reduce_scatter_roofline_fraction": frac(rs_bytes, rs), "all_gather_roofline_fraction": frac(ag_bytes, ag),
                "comm_roofline_fraction": frac(rs_bytes + ag_bytes, rs + ag) if rs + ag > 0 else None,
                "link_gbs_per_direction_measured": link_gbs}

    def average_metrics(self, values):
        """Mean over ranks of the loss terms; the last entry (gradient norm) is already global."""
        if self.world > 1:
            head = values[:-1].clone()
            dist.all_reduce(head)
            values = torch.cat([head / self.world, values[-1:]])
        return values

    # ------------------------------------------------------------------ checkpoints
    def checkpoint_state(self):
        """(model state_dict, optimizer state_dict) with the layout of a replicated run.

        Optimizer moments are only maintained by the owner of each parameter; before rank 0 serialises them
        every owner publishes its segments (a collective, so all ranks must call this)."""
        if self.world > 1:
            for flat in (self.arena.exp_avg, self.arena.exp_avg_sq, self.arena.muon_buf):
                for owner, (s, e) in enumerate(self.arena.segments):
                    if e > s:
                        dist.broadcast(flat[s:e], src=owner)
            for unit in self.arena.local_units():             # assemble the full expert tensors from the ranks' slices
                n = unit.param.shape[0] // self.world
                for flat in (self.arena.params, self.arena.muon_buf):
                    full = self.arena.view(flat, unit)
                    for owner in range(self.world):
                        dist.broadcast(full[owner * n:(owner + 1) * n], src=owner)
            if self.arena.local_units():
                self.arena.refresh_shadow()
        return self.model.state_dict(), self.optimizer.state_dict()

    def gather_experts(self):
        """Expert parallelism: make every rank's copy of the expert tensors complete (each rank trains only its slice), so that
        code that runs the replicated expert path (evaluation under `no_grad`, export) sees the whole model.  Collective."""
        units = self.arena.local_units()
        if self.world == 1 or not units:
            return
        for unit in units:
            n = unit.param.shape[0] // self.world
            full = self.arena.view(self.arena.params, unit)
            for owner in range(self.world):
                dist.broadcast(full[owner * n:(owner + 1) * n], src=owner)
        self.arena.refresh_shadow()

    def load_checkpoint(self, model_state, opt_state):
        self.model.load_state_dict(model_state)
        self.optimizer.load_state_dict(opt_state)
        self.arena.refresh_shadow()

    def check_canaries(self):
        """Guard bytes after every peer-mapped buffer of this rank are intact (no-op without the peer-memory transport)."""
        if self.transport is not None:
            self.transport.check_canaries()

    def describe_transport(self):
        """'collective', or 'p2p' with the reduce-scatter algorithm and the allocation back end of the peer arenas."""
        if self.transport is None:
            return self.mode
        return f"{self.mode}:{self.transport.rs_algo}:{self.transport.alloc_backend}"

    def describe(self):
        info = self.arena.describe()
        return f"{self.mode} world={self.world} arena={info['numel'] / 1e6:.1f}M elements owner_numel={info['owner_numel']}"

    def close(self):
        if self.transport is not None:
            self.transport.close()
            self.transport = None
