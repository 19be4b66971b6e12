"""Flat parameter / gradient / optimizer-state storage with an ownership map.

All parameters of the model are re-pointed into one flat fp32 buffer, their gradients into a second
one and the optimizer moments into three more (AdamW ``exp_avg`` / ``exp_avg_sq``, Muon ``buf``), all with
the same element offsets.  A bf16 *shadow* of the parameters with the same offsets feeds the tensor-core
GEMMs, so no per-use fp32 -> bf16 cast of a weight ever runs.

Every parameter tensor is owned by exactly one data-parallel rank.  The buffers are laid out owner by
owner, and inside an owner by optimizer group (Muon matrices, AdamW with decay, AdamW without decay), so

* the reduce-scatter of gradients is "rank r sums segment r of every rank's gradient buffer",
* AdamW runs as a flat elementwise kernel over (at most) two contiguous ranges per owner,
* the parameter all-gather is "rank r publishes segment r".

Ownership balances one estimate of the time a tensor costs its owner after the last micro-step, with a
longest-processing-time greedy: the Newton-Schulz FLOPs of a Muon matrix at the rate those small products
reach, plus, for every tensor, the bytes its owner moves for it in the gradient reduce-scatter, the elementwise
update and the parameter all-gather.  Balancing the Newton-Schulz work alone left the two n-gram tables (AdamW,
a quarter of the q38_c2 parameters) on two ranks whose segments were twice the mean, and the reduce-scatter and
the all-gather end when the largest segment is through.
Muon needs whole matrices, which is why the unit of ownership is a parameter tensor and not a byte range.
With ``world == 1`` there is a single segment and the layout degenerates to one flat buffer.
"""
from dataclasses import dataclass

import torch

from ..optim.hybrid import split_parameters

UNIT_ALIGN = 64          # elements; keeps every tensor 256-byte aligned in fp32 and 128-byte aligned in bf16
SEGMENT_ALIGN = 1024
GROUPS = ("muon", "decay", "no_decay")


@dataclass
class Unit:
    name: str
    param: torch.nn.Parameter
    group: str
    index: int          # registration order
    owner: int = 0
    offset: int = 0
    local: bool = False   # expert-parallel tensor: every rank owns its own slice, never reduced or gathered

    @property
    def numel(self):
        return self.param.numel()


def newton_schulz_flops(shape, steps=5):
    """FLOPs of the NS chain for a stack of matrices ``[..., rows, cols]``."""
    rows, cols = shape[-2], shape[-1]
    m, n = min(rows, cols), max(rows, cols)
    stack = 1
    for d in shape[:-2]:
        stack *= d
    return stack * steps * (4 * m * m * n + 2 * m ** 3)


NS_FLOPS_PER_SECOND = 180e12      # measured rate of the batched Newton-Schulz chain on the expert matrices
LINK_BYTES_PER_SECOND = 770e9      # measured peer-copy bandwidth per direction
HBM_BYTES_PER_SECOND = 6.5e12


def owner_seconds(unit, world):
    """Estimated time a tensor costs its owner between the last backward and the next forward."""
    comm = 2 * (world - 1) * 4 / LINK_BYTES_PER_SECOND          # fp32 in from every peer, fp32 out to every peer
    update = 16 / HBM_BYTES_PER_SECOND                          # parameter, gradient and moments
    seconds = unit.numel * (comm + update)
    if unit.group == "muon":
        seconds += newton_schulz_flops(tuple(unit.param.shape)) / NS_FLOPS_PER_SECOND
    return seconds


def assign_owners(units, world):
    """Longest-processing-time greedy over `owner_seconds`; deterministic, so every rank derives the same map."""
    load = [0.0] * world
    for unit in sorted(units, key=lambda u: (-owner_seconds(u, world), u.index)):
        owner = min(range(world), key=lambda r: (load[r], r))
        unit.owner = owner
        load[owner] += owner_seconds(unit, world)
    return load


def _align(x, a):
    return (x + a - 1) // a * a


class ParamArena:
    def __init__(self, model, device, world=1, muon=True, allocate=None, local_filter=None):
        """`allocate(numel, dtype)` returns a zero-filled flat tensor (peer-mapped memory for the p2p engine).
        `local_filter(name)` marks expert-parallel tensors: they live after all owner segments (`local_range`) and take no part
        in the gradient reduce-scatter or the parameter all-gather."""
        self.device, self.world = torch.device(device), world
        allocate = allocate or (lambda numel, dtype: torch.zeros(numel, dtype=dtype, device=self.device))
        matrices, decay, no_decay = split_parameters(model, muon)
        order = {name: i for i, (name, _) in enumerate(model.named_parameters())}
        self.units = [Unit(n, p, g, order[n]) for g, items in zip(GROUPS, (matrices, decay, no_decay)) for n, p in items]
        for unit in self.units:
            unit.local = bool(local_filter and local_filter(unit.name))
        self.load = assign_owners([u for u in self.units if not u.local], world)
        self.units.sort(key=lambda u: (u.local, u.owner, GROUPS.index(u.group), u.index))
        # layout
        self.segments = []                       # per owner: (start, end)
        self.group_ranges = {}                   # (owner, group) -> (start, end)
        cursor = 0
        for owner in range(world):
            start = cursor
            for group in GROUPS:
                g0 = cursor
                for unit in (u for u in self.units if u.owner == owner and u.group == group and not u.local):
                    unit.offset = cursor
                    cursor = _align(cursor + unit.numel, UNIT_ALIGN)
                self.group_ranges[(owner, group)] = (g0, cursor)
            cursor = _align(cursor, SEGMENT_ALIGN)
            self.segments.append((start, cursor))
        local_start = cursor
        for unit in (u for u in self.units if u.local):
            unit.offset = cursor
            cursor = _align(cursor + unit.numel, UNIT_ALIGN)
        cursor = _align(cursor, SEGMENT_ALIGN)
        self.local_range = (local_start, cursor)
        self.numel = cursor
        self.params = allocate(self.numel, torch.float32)
        self.grads = allocate(self.numel, torch.float32)
        self.exp_avg = torch.zeros(self.numel, dtype=torch.float32, device=self.device)
        self.exp_avg_sq = torch.zeros(self.numel, dtype=torch.float32, device=self.device)
        self.muon_buf = torch.zeros(self.numel, dtype=torch.float32, device=self.device)
        self.shadow = allocate(self.numel, torch.bfloat16) if self.device.type == "cuda" else None
        with torch.no_grad():
            for unit in self.units:
                p = unit.param
                view = self.view(self.params, unit)
                view.copy_(p.data)
                p.data = view
                p.grad = self.view(self.grads, unit)
                if self.shadow is not None:
                    p._q38_bf16 = self.view(self.shadow, unit)
        self.by_name = {u.name: u for u in self.units}
        self.refresh_shadow()

    def view(self, flat, unit):
        return flat[unit.offset:unit.offset + unit.numel].view(unit.param.shape)

    def owned(self, rank, group=None):
        return [u for u in self.units if not u.local and u.owner == rank and (group is None or u.group == group)]

    def local_units(self):
        return [u for u in self.units if u.local]

    def refresh_shadow(self, rank=None):
        """Re-derive the bf16 shadow from the fp32 parameters (all of it, or one owner's segment)."""
        if self.shadow is None:
            return
        s, e = (0, self.numel) if rank is None else self.segments[rank]
        self.shadow[s:e].copy_(self.params[s:e])
        if rank is not None and self.local_range[1] > self.local_range[0]:
            ls, le = self.local_range
            self.shadow[ls:le].copy_(self.params[ls:le])

    def zero_grad(self):
        self.grads.zero_()

    def describe(self):
        per_owner = [sum(u.numel for u in self.units if u.owner == r) for r in range(self.world)]
        return dict(numel=self.numel, world=self.world, owner_numel=per_owner, owner_cost=self.load)
