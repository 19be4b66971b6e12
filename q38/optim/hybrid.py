"""Muon + AdamW hybrid optimizer with the parameter split of the reference (q38/muon.py:122-166).

* Muon: every parameter with ``ndim >= 2`` that is not an embedding / hash table / router /
  shared-expert gate / GDN ``in_proj_a`` / ``in_proj_b``; inside mHC blocks only ``A.weight`` and ``B.weight``.
* AdamW with weight decay: the remaining ``ndim >= 2`` parameters outside the hash tables and mHC.
* AdamW without decay: hash tables, mHC scalars, norm weights, ``A_log``, ``dt_bias``, biases.

`state_dict()` is ``{"adam": ..., "muon": ...}`` with index-based torch optimizer state dicts, the layout
stored under ``"opt"`` in ``ckpt.pt``.

Two operating modes.  Stand-alone (``arena=None``): a `torch.optim.AdamW` and a `Muon` over the model's
parameters, every parameter updated locally.  Arena-backed (``arena=ParamArena``, used by the trainer): the
moments are views into the arena's flat state buffers, AdamW runs as one flat elementwise pass per
contiguous (owner, group) range and only the units owned by ``rank`` are updated; `state_dict()` still has
the stand-alone layout because the torch optimizer objects hold those views as their state.
"""
import math
import os

import torch

from .muon import Muon

NOT_MUON = ("embed_tokens", "lm_head", "emb2", "emb3", ".mlp.gate.weight", "shared_expert_gate", "in_proj_a", "in_proj_b")
NO_DECAY_MATRICES = ("emb2", "emb3", ".mhc.")
ADAM_BETAS, ADAM_EPS = (0.9, 0.95), 1e-8


def split_parameters(model, muon=True):
    """Returns ``(muon, adam_decay, adam_no_decay)`` lists of ``(name, parameter)`` in registration order."""
    matrices, decay, no_decay = [], [], []
    for name, p in model.named_parameters():
        is_matrix = p.ndim >= 2 and not any(key in name for key in NOT_MUON)
        if ".mhc." in name:
            is_matrix = name.endswith((".A.weight", ".B.weight"))
        if muon and is_matrix:
            matrices.append((name, p))
        elif p.ndim >= 2 and not any(key in name for key in NO_DECAY_MATRICES):
            decay.append((name, p))
        else:
            no_decay.append((name, p))
    return matrices, decay, no_decay


def adamw_flat_(p, g, m, v, step, lr, wd, grad_scale=None, betas=ADAM_BETAS, eps=ADAM_EPS, hyper=None, shadow=None, err=None):
    """In-place AdamW on flat fp32 tensors with torch.optim.AdamW's arithmetic (decoupled decay first).  On a GPU `shadow`
    (bf16, same length) receives the rounded parameters and `err` is the device error word: when it is set the kernel
    returns without writing."""
    if p.is_cuda:
        from ..ops import adamw_flat
        return adamw_flat(p, g, m, v, step, lr, wd, betas[0], betas[1], eps, grad_scale, shadow=shadow, hyper=hyper, err=err)
    if grad_scale is not None:
        g = g * grad_scale
    b1, b2 = betas
    p.mul_(1 - lr * wd)
    m.lerp_(g, 1 - b1)
    v.mul_(b2).addcmul_(g, g, value=1 - b2)
    bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    p.addcdiv_(m, denom, value=-lr / bc1)


class HybridOptimizer:
    def __init__(self, model, lr, weight_decay, muon=True, fused_adam=None, arena=None, rank=0):
        matrices, decay, no_decay = split_parameters(model, muon)
        self.names = dict(muon=[n for n, _ in matrices], decay=[n for n, _ in decay], no_decay=[n for n, _ in no_decay])
        self.arena, self.rank, self.steps_done = arena, rank, 0
        self._graph, self._warmed, self._hyper = None, False, None
        self._fused_muon = None
        on_gpu = next(model.parameters()).is_cuda
        fused = (on_gpu if fused_adam is None else fused_adam) and arena is None
        self.adam = torch.optim.AdamW(
            [{"params": [p for _, p in decay], "weight_decay": weight_decay},
             {"params": [p for _, p in no_decay], "weight_decay": 0.0}],
            lr=lr, betas=ADAM_BETAS, eps=ADAM_EPS, fused=fused)
        self.muon = Muon([p for _, p in matrices], lr=lr, weight_decay=weight_decay) if matrices else None
        self._link_groups()
        if arena is not None:
            self._bind_states()

    def _link_groups(self):
        self.param_groups = self.adam.param_groups + (self.muon.param_groups if self.muon else [])

    def _bind_states(self):
        a = self.arena
        for unit in a.units:
            if unit.group == "muon":
                self.muon.state[unit.param]["buf"] = a.view(a.muon_buf, unit)
            else:
                self.adam.state[unit.param].update(step=torch.zeros((), dtype=torch.float32),
                                                   exp_avg=a.view(a.exp_avg, unit), exp_avg_sq=a.view(a.exp_avg_sq, unit))

    def state_bytes(self):
        """Bytes of persistent state after the first step (two AdamW moments, one Muon momentum buffer)."""
        size = lambda groups: sum(p.numel() * p.element_size() for g in groups for p in g["params"])
        return 2 * size(self.adam.param_groups) + (size(self.muon.param_groups) if self.muon else 0)

    # ------------------------------------------------------------------ update
    def step(self, grad_scale=None):
        if self.arena is None:
            if grad_scale is not None:
                for group in self.param_groups:
                    for p in group["params"]:
                        if p.grad is not None:
                            p.grad.mul_(grad_scale)
            self.adam.step()
            if self.muon:
                self.muon.step()
            return
        a = self.arena
        self.steps_done += 1
        if a.device.type == "cuda" and os.environ.get("Q38_OPTIMIZER_GRAPH", "1") != "0" and self._same_lr():
            return self._replayed_step(grad_scale)
        self._arena_step(grad_scale, None, None)

    def _same_lr(self):
        lrs = {g["lr"] for g in self.param_groups}
        return len(lrs) == 1

    def _arena_step(self, grad_scale, hyper, lr_tensor):
        """AdamW over this rank's flat ranges, then Muon over the matrices it owns.  With `hyper` / `lr_tensor` the learning
        rate and the bias corrections are read from device memory.  On a GPU both write the bf16 shadow of what they update
        and both leave everything untouched when the device error word is set."""
        a = self.arena
        on_gpu = a.device.type == "cuda"
        err = None
        if on_gpu:
            from .. import ops
            err = ops.error_flag(a.device)
        for group_name, group in zip(("decay", "no_decay"), self.adam.param_groups):
            s, e = a.group_ranges[(self.rank, group_name)]
            if e > s:
                adamw_flat_(a.params[s:e], a.grads[s:e], a.exp_avg[s:e], a.exp_avg_sq[s:e], self.steps_done,
                            group["lr"], group["weight_decay"], grad_scale, hyper=hyper,
                            shadow=a.shadow[s:e] if (on_gpu and a.shadow is not None) else None, err=err)
        if not self.muon:
            return
        if on_gpu and not os.environ.get("Q38_MUON_BASELINE"):
            group = self.muon.param_groups[0]
            self._muon_plan().step(group["lr"], group["momentum"], group["weight_decay"], grad_scale=grad_scale, hyper=hyper, err=err)
            return
        owned = [u.param for u in a.owned(self.rank, "muon")]
        slices = {}
        for unit in a.local_units():                     # expert-parallel tensors: this rank updates its own experts only
            owned.append(unit.param)
            n = unit.param.shape[0] // a.world
            slices[id(unit.param)] = slice(self.rank * n, (self.rank + 1) * n)
        self.muon.step(params=owned, grad_scale=grad_scale, slices=slices, lr_tensor=lr_tensor)

    def _muon_plan(self):
        """Device tables of the matrices this rank updates (built once; the arena layout never changes)."""
        if self._fused_muon is None:
            from ..ops.muon_gpu import FusedMuon
            a = self.arena
            entries = []
            for unit in a.owned(self.rank, "muon"):
                rows, cols = unit.param.shape[-2:]
                entries.append((unit.offset, unit.numel // (rows * cols), rows, cols))
            for unit in a.local_units():
                rows, cols = unit.param.shape[-2:]
                n = unit.param.shape[0] // a.world
                per = unit.numel // unit.param.shape[0]
                entries.append((unit.offset + self.rank * n * per, n * per // (rows * cols), rows, cols))
            group = self.muon.param_groups[0]
            self._fused_muon = FusedMuon(a.params, a.grads, a.muon_buf, a.shadow, entries, rms_scale=group["rms_scale"], ns_steps=group["ns_steps"])
        return self._fused_muon

    def _replayed_step(self, grad_scale):
        """The optimizer step as one CUDA graph.  Hundreds of small launches (Newton-Schulz chains per matrix shape) otherwise
        leave the GPU waiting for the host; learning rate, bias corrections and the clip factor live in device tensors that
        are refreshed before every replay.  The first step runs eagerly (lazy initialisation), the second is captured."""
        dev = self.arena.device
        if self._hyper is None:
            self._hyper = torch.zeros(4, dtype=torch.float32, device=dev)
            # A ring of pinned staging buffers: the host may run several steps ahead of the GPU, so a buffer is only
            # rewritten after the copy that last read it has completed.
            self._hyper_ring = [(torch.zeros(4, dtype=torch.float32).pin_memory(), torch.cuda.Event()) for _ in range(4)]
            self._scale = torch.ones((), dtype=torch.float32, device=dev)
        lr = self.param_groups[0]["lr"]
        b1, b2 = ADAM_BETAS
        t = self.steps_done
        host, copied = self._hyper_ring[t % len(self._hyper_ring)]
        copied.synchronize()
        host[0], host[1], host[2] = lr, 1.0 / (1.0 - b1 ** t), 1.0 / math.sqrt(1.0 - b2 ** t)
        self._hyper.copy_(host, non_blocking=True)
        copied.record()
        if grad_scale is None:
            self._scale.fill_(1.0)
        else:
            self._scale.copy_(grad_scale.reshape(()).float())
        if self._graph is None:
            if not self._warmed:
                self._warmed = True
                self._arena_step(self._scale, self._hyper, self._hyper[0])
                return
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    self._arena_step(self._scale, self._hyper, self._hyper[0])
                self._graph = graph
            except Exception as exc:                         # pragma: no cover - depends on the driver
                print(f"[q38.optim] optimizer graph capture failed ({type(exc).__name__}: {exc}); stepping eagerly", flush=True)
                os.environ["Q38_OPTIMIZER_GRAPH"] = "0"
                torch.cuda.synchronize(dev)
                self._arena_step(self._scale, self._hyper, self._hyper[0])
                return
        self._graph.replay()

    def zero_grad(self, set_to_none=True):
        if self.arena is not None:
            self.arena.zero_grad()
            return
        self.adam.zero_grad(set_to_none=set_to_none)
        if self.muon:
            self.muon.zero_grad(set_to_none=set_to_none)

    # ------------------------------------------------------------------ (de)serialisation
    def state_dict(self):
        if self.arena is not None and self.steps_done:
            for state in self.adam.state.values():
                state["step"] = torch.tensor(float(self.steps_done))
        return {"adam": self.adam.state_dict(), "muon": self.muon.state_dict() if self.muon else None}

    def load_state_dict(self, state):
        if self.arena is None:
            self.adam.load_state_dict(state["adam"])
            if self.muon:
                self.muon.load_state_dict(state["muon"])
            self._link_groups()
            return
        # Arena-backed: copy into the existing views so the flat buffers stay the single source of truth.
        for optimizer, saved in ((self.adam, state["adam"]), (self.muon, state.get("muon"))):
            if optimizer is None or saved is None:
                continue
            params = [p for g in optimizer.param_groups for p in g["params"]]
            for group, saved_group in zip(optimizer.param_groups, saved["param_groups"]):
                for key, value in saved_group.items():
                    if key != "params":
                        group[key] = value
            for index, entry in saved["state"].items():
                target = optimizer.state[params[int(index)]]
                for key, value in entry.items():
                    if key == "step":
                        self.steps_done = max(self.steps_done, int(float(value)))
                    elif key in target:
                        target[key].copy_(value)
        self._link_groups()
