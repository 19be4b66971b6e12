"""Pretrain the Q38 sparse MoE model on one GPU or on all GPUs of a node.

  python -m q38.train --preset q38_c2                                            # one GPU
  torchrun --standalone --nproc_per_node=8 -m q38.train --preset q38_c2          # data parallel, same global batch

A preset (``configs/<name>.json``) supplies the model shape and the training defaults; command-line
flags override it.  ``--tokens 0`` derives the token budget from ``--compute``; ``--warmup 0`` means 1 % of
the steps (at least ``warmup_min``).  ``--resume 1`` (default) continues from ``run_dir/ckpt.pt`` after
checking that model, data, budget and schedule are unchanged.  ``--max_steps N`` stops at absolute step
N without changing the learning-rate curve.  ``--micro_bs`` is sequences per GPU per micro-step,
``--grad_ckpt 1`` recomputes each layer in backward, ``--auto_micro_bs 1`` probes the largest micro batch
that fits.  QSA uses dense attention while ``step < warmup`` (``--dense_warmup 1``), block-sparse afterwards.

Outputs in ``run_dir``: ``ckpt.pt`` (fp32 weights, optimizer, RNG of every rank), ``run_config.json``,
``training_metrics.csv``, ``tb/``, ``micro_bs_probe.json``, ``final_eval.json``, ``summary.json``,
``flops.json`` and ``hf/`` (bf16 export with the model code).  Flags, file layouts and resume rules are
those of the reference trainer (q38/train.py:43-116, 482-541, 586-606).

Data parallelism keeps the reference semantics (replicated weights, gradients averaged over ranks once
per optimizer step, replicas identical after every step) but not its mechanism: gradients live in one
flat peer-mapped arena, are reduce-scattered by peer-memory kernels, every rank updates only the
parameters it owns and the updated parameters are all-gathered by peer stores (`q38.parallel`).
``--grad_sync collective`` selects the library path (NCCL or gloo all-reduce), which is also what CPU runs use.
"""
import argparse
import contextlib
import csv
import gc
import hashlib
import json
import math
import os
import time
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

from .data import DEFAULT_DATA, DEFAULT_TOKENIZER, DEFAULT_VAL_DATA, TOKEN_DTYPE, load_tokenizer, open_tokens, tokenizer_sha256
from .flops import count as count_flops, validate_resume_accounting
from .losses import LossModel, linear_cross_entropy
from .models import Q38ForCausalLM, source_info
from .presets import CKPT_ROOT, MODEL_DEFAULTS, ROOT, budget_tokens, load_preset, load_training_config, model_config
from .sampling import ShuffledBlockSampler, sequential_windows

TRAIN_DEFAULTS = dict(
    run_dir="", data=str(DEFAULT_DATA), val_data=str(DEFAULT_VAL_DATA), tokenizer=str(DEFAULT_TOKENIZER),
    seq=4096, tokens=0, compute=0.0, batch_tokens=524288, micro_bs=8, lr=3.6e-3, min_lr_ratio=0.1, warmup=0,
    wd=0.1, clip=1.0, seed=0, log_every=10, eval_every=500, eval_tokens=2_000_000, ckpt_every=200, resume=1,
    max_steps=0, tensorboard=1, warmup_ratio=0.01, warmup_min=10, data_sampling="random", data_seed=-1,
    eval_sampling="random", eval_offset=0, final_eval_tokens=0, final_eval_offset=0, require_ready_pool=0,
    auto_micro_bs=0, probe_mem_frac=0.92, mtp_coef=0.3, kl_coef=0.05, muon=1, dense_warmup=1, grad_ckpt=0)
# Options of this framework that the reference trainer does not have (never part of the resume contract).
ENGINE_DEFAULTS = dict(grad_sync="auto", fp8_ffn=0, expert_parallel=0, ep_capacity=4.0, export_hf=1, device="auto", cuda_graphs=1, overlap_wgrad=1)

# Everything that shapes the model, the data stream or the schedule must be unchanged on resume.
RESUME_KEYS = (
    "layers", "hidden", "heads", "kv_heads", "head_dim", "lin_k_heads", "lin_v_heads", "lin_head_dim", "experts", "topk",
    "moe_ffn", "shared_ffn", "layer_types", "aux_coef", "rope_theta", "partial_rotary", "seq", "tokens", "batch_tokens",
    "seed", "data", "val_data", "tokenizer", "eval_tokens", "lr", "min_lr_ratio", "warmup", "wd", "clip",
    "data_sampling", "data_seed", "eval_sampling", "eval_offset", "final_eval_tokens", "final_eval_offset",
    "n_branch", "mhc_iters", "qsa_blocks", "indexer_heads", "indexer_head_dim", "ngram_rows", "mtp", "mtp_coef",
    "kl_coef", "muon", "dense_warmup")
# Keys that older run_config.json files may lack, with the value such runs used.
LATE_KEYS = ("data_sampling", "data_seed", "eval_sampling", "eval_offset", "final_eval_tokens", "final_eval_offset")
NEW_RESUME_DEFAULTS = {k: TRAIN_DEFAULTS[k] for k in LATE_KEYS}
METRIC_COLUMNS = ["step", "tokens", "loss", "aux", "lr", "grad_norm", "tok_per_s", "elapsed_s", "val_loss",
                  "active_nonvocab", "total_nonvocab", "mtp_loss", "indexer_kl"]


def int_like(text):
    """Accept ``3e9``-style integers."""
    return int(float(text))


# ------------------------------------------------------------------------------------------ arguments
def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    source = ap.add_mutually_exclusive_group()
    source.add_argument("--preset", default="", help="configs/<preset>.json")
    source.add_argument("--config", default="", help="training JSON file or a directory containing config.json")
    ap.add_argument("--dry-run", "--dry_run", dest="dry_run", action="store_true",
                    help="validate data, model shape and compute budget on CPU; create nothing")
    for key, value in {**MODEL_DEFAULTS, **TRAIN_DEFAULTS, **ENGINE_DEFAULTS}.items():
        ap.add_argument(f"--{key}", type=int_like if key in ("tokens", "eval_tokens") else type(value), default=value)
    first, _ = ap.parse_known_args(argv)
    if first.preset or first.config:
        preset = load_preset(first.preset) if first.preset else load_training_config(first.config)[1]
        unknown_model = set(preset["model"]) - set(MODEL_DEFAULTS)
        allowed_train = (set(TRAIN_DEFAULTS) | set(MODEL_DEFAULTS) | set(ENGINE_DEFAULTS)) - {"compute"}
        unknown_train = set(preset["train"]) - allowed_train
        if unknown_model or unknown_train:
            ap.error(f"Unknown config fields: model={sorted(unknown_model)}, train={sorted(unknown_train)}")
        ap.set_defaults(compute=preset["compute"], run_dir=str(CKPT_ROOT / first.preset) if first.preset else "",
                        **{**preset["model"], **preset["train"]})
    a = ap.parse_args(argv)
    if a.config:
        a.config = str(load_training_config(a.config)[0])
    for key in ("run_dir", "data", "val_data", "tokenizer"):
        value = getattr(a, key)
        if value:
            path = Path(value).expanduser()
            setattr(a, key, str(path if path.is_absolute() else ROOT / path))
    checks = [
        (bool(a.run_dir), "--run_dir is required without --preset"),
        (all(getattr(a, n) > 0 for n in ("layers", "hidden", "seq", "batch_tokens", "micro_bs", "log_every", "eval_every")),
         "--layers, --hidden, --seq, --batch_tokens, --micro_bs, --log_every and --eval_every must be positive"),
        (a.grad_ckpt in (0, 1), "--grad_ckpt must be 0 or 1"),
        (a.auto_micro_bs in (0, 1) and 0 < a.probe_mem_frac <= 1, "--auto_micro_bs must be 0 or 1; --probe_mem_frac must be in (0,1]"),
        (min(a.tokens, a.max_steps, a.ckpt_every) >= 0, "token and step limits must be nonnegative"),
        (bool(a.tokens or a.compute), "give --tokens or --compute (or a --preset)"),
        (a.eval_tokens >= a.seq + 2, "--eval_tokens must be at least seq + 2"),
        (a.compute >= 0 and a.lr > 0 and 0 <= a.min_lr_ratio <= 1,
         "compute must be nonnegative; lr must be positive; min_lr_ratio must be in [0,1]"),
        (0 <= a.warmup_ratio < 1 and min(a.warmup, a.warmup_min, a.eval_offset, a.final_eval_tokens, a.final_eval_offset) >= 0,
         "Invalid warmup or validation partition"),
        (a.data_sampling in ("random", "shuffled_blocks") and a.eval_sampling in ("random", "sequential"),
         "Invalid training or evaluation sampling mode"),
        (a.data_seed >= -1, "data_seed must be -1 (use model seed) or nonnegative"),
        (a.grad_sync in ("auto", "p2p", "collective"), "--grad_sync must be auto, p2p or collective"),
        (a.fp8_ffn in (0, 1) and not (a.fp8_ffn and a.expert_parallel), "--fp8_ffn must be 0 or 1 and cannot be combined with --expert_parallel 1"),
        (not a.fp8_ffn or (a.hidden % 16 == 0 and a.moe_ffn % 16 == 0), "--fp8_ffn 1 needs hidden and moe_ffn to be multiples of 16"),
    ]
    for ok, message in checks:
        if not ok:
            ap.error(message)
    return a


def _data_identity(path):
    path = Path(path)
    stat = path.stat()
    identity = dict(path=str(path.resolve()), bytes=stat.st_size, mtime_ns=stat.st_mtime_ns)
    meta = path.parent / "meta.json"
    if meta.exists():
        identity["declared_sha256"] = json.loads(meta.read_text()).get(
            "train_sha256" if path.name == "train.bin" else "valid_sha256")
    return identity


def micro_bs_candidates(per_rank, limit):
    """Divisors of the per-rank sequence count not above `limit`, largest first."""
    return [m for m in range(min(per_rank, limit), 0, -1) if per_rank % m == 0]


def _check_ready_pool(a, data, tok_sha):
    pool = Path(a.data).parent
    meta = json.loads((pool / "meta.json").read_text())
    verified = json.loads((pool / "verification.json").read_text())
    if not (pool / "READY").is_file() or meta.get("state") != "ready" or verified.get("state") != "ready":
        raise ValueError("Training pool is not verified READY")
    if meta["tokenizer_sha256"] != tok_sha or len(data) != meta["train_tokens"]:
        raise ValueError("Training pool identity does not match its manifest")
    if verified["train_sha256"] != meta["train_sha256"]:
        raise ValueError("Pool verification and manifest disagree")


def prepare_inputs(a, world=1):
    """Read-only preflight (also the whole of ``--dry-run``): tokenizer, model config, budget, data, sampler."""
    if world < 1:
        raise ValueError("WORLD_SIZE must be positive")
    tok = load_tokenizer(a.tokenizer)
    if tok.eos_token_id is None:
        raise ValueError("Tokenizer must have an EOS ID")
    tok_sha = tokenizer_sha256(a.tokenizer)
    cfg = model_config(vars(a), len(tok), a.seq, tok.bos_token_id, tok.eos_token_id, tok.pad_token_id)
    fc = count_flops(cfg.to_dict(), a.seq)
    if not a.tokens:
        a.tokens = budget_tokens(fc["train_flops_per_token"], a.compute, a.batch_tokens)
    steps = a.tokens // a.batch_tokens
    if steps < 1:
        raise ValueError("Budget must cover at least one global batch")
    per_rank, rest = divmod(a.batch_tokens, a.seq * world)
    if rest or not per_rank:
        raise ValueError("batch_tokens must be divisible by seq*WORLD_SIZE")
    a.micro_bs = min(a.micro_bs, per_rank)
    if not a.auto_micro_bs and per_rank % a.micro_bs:
        raise ValueError("batch_tokens must be divisible by micro_bs*seq*WORLD_SIZE")
    if not a.warmup:
        a.warmup = min(steps, max(a.warmup_min, round(steps * a.warmup_ratio)))
    if a.warmup > steps:
        raise ValueError("Warmup exceeds the full training horizon")
    if a.data_seed == -1:
        a.data_seed = a.seed
    data = open_tokens(a.data, tok_sha)
    if a.val_data:
        train, validation = data, open_tokens(a.val_data, tok_sha)
    else:
        train, validation = data[:-a.eval_tokens], data[-a.eval_tokens:]
    if len(train) < a.seq + 2 or len(validation) < a.seq + 2:
        raise ValueError("Not enough training or validation tokens")
    if a.require_ready_pool:
        _check_ready_pool(a, data, tok_sha)
    sampler = ShuffledBlockSampler(len(train), a.seq, a.data_seed) if a.data_sampling == "shuffled_blocks" else None
    if sampler and steps * (a.batch_tokens // a.seq) > sampler.blocks:
        raise ValueError("Training budget exceeds unique sequence blocks; corpus repetition is disabled")

    def partition(offset, targets):
        if offset < 0 or offset + targets + 1 > len(validation):
            raise ValueError("Requested evaluation partition exceeds validation corpus")
        return validation[offset:offset + targets + 1]

    dev = partition(a.eval_offset, a.eval_tokens) if a.eval_sampling == "sequential" else validation[:a.eval_tokens]
    final = partition(a.final_eval_offset, a.final_eval_tokens) if a.final_eval_tokens else None
    if final is not None and not a.val_data:
        raise ValueError("Final evaluation requires an independent validation file")
    identity = dict(train=_data_identity(a.data), validation=_data_identity(a.val_data) if a.val_data else None)
    plan = dict(
        config=a.config, run_dir=a.run_dir, compute_budget=a.compute, train_tokens=steps * a.batch_tokens, steps=steps,
        warmup_steps=a.warmup, actual_train_flops=fc["train_flops_per_token"] * steps * a.batch_tokens,
        train_flops_per_token=fc["train_flops_per_token"], flops_accounting=fc["accounting_method"],
        megatron_reference_train_flops_per_token=fc["megatron_reference_train_flops_per_token"],
        total_params=fc["total_nonvocab_params"] + fc["embed_params"], active_nonvocab_params=fc["active_nonvocab_params"],
        seq=a.seq, batch_tokens=a.batch_tokens, micro_bs="auto" if a.auto_micro_bs else a.micro_bs, world=world,
        micro_bs_candidates=micro_bs_candidates(per_rank, a.micro_bs) if a.auto_micro_bs else [a.micro_bs],
        accumulation=None if a.auto_micro_bs else per_rank // a.micro_bs, lr=a.lr, data=a.data, val_data=a.val_data,
        tokenizer=a.tokenizer, tokenizer_sha256=tok_sha, data_identity=identity,
        sampling=sampler.metadata() if sampler else dict(mode="random", replacement=True, seed=a.data_seed),
        eval_sampling=a.eval_sampling, eval_offset=a.eval_offset, eval_targets=len(dev) - 1,
        final_eval_offset=a.final_eval_offset, final_eval_targets=len(final) - 1 if final is not None else 0,
        config_sha256=hashlib.sha256(Path(a.config).read_bytes()).hexdigest() if a.config else None)
    return tok, cfg, fc, train, dev, final, sampler, plan


# ------------------------------------------------------------------------------------------ batches / schedule / eval
def host_batch(rng, src, bs, seq, offsets=None, pinned=False):
    """Cut (x, y) int64 host tensors ``[bs, seq]`` from a token array at random or given offsets."""
    starts = rng.integers(0, len(src) - seq - 1, bs) if offsets is None else offsets
    window = np.stack([np.asarray(src[s:s + seq + 1], dtype=np.int64) for s in starts])
    x, y = torch.from_numpy(window[:, :-1].copy()), torch.from_numpy(window[:, 1:].copy())
    if pinned:
        x, y = x.pin_memory(), y.pin_memory()
    return x, y


def sample_batch(rng, src, bs, seq, dev, offsets=None):
    dev = torch.device(dev)
    x, y = host_batch(rng, src, bs, seq, offsets, pinned=dev.type == "cuda")
    return x.to(dev, non_blocking=True), y.to(dev, non_blocking=True)


def lr_schedule(a, steps):
    """Linear warm-up to ``lr`` over ``warmup`` steps, then cosine to ``min_lr_ratio * lr`` at the last step."""
    def lr_at(step):
        if step < a.warmup:
            return a.lr * (step + 1) / a.warmup
        progress = (step - a.warmup) / max(1, steps - a.warmup - 1)
        return a.lr * (a.min_lr_ratio + (1 - a.min_lr_ratio) * 0.5 * (1 + math.cos(math.pi * progress)))
    return lr_at


@torch.no_grad()
def evaluate(model, eval_data, seq, dev, sampling="random", distributed=False):
    """Mean CE of the main head.  ``sequential`` scores every target exactly once (short tail included);
    ``random`` draws ``len // seq`` windows with a fixed seed.  The model's train/eval mode is restored."""
    dev = torch.device(dev)
    was_training = model.training
    model.eval()
    rng = np.random.default_rng(1234)
    if sampling == "sequential":
        windows = sequential_windows(len(eval_data), seq)
    else:
        # every rank draws the whole list, so a distributed evaluation scores exactly the windows a single rank would
        windows = [(int(rng.integers(0, len(eval_data) - seq - 1, 1)[0]), seq) for _ in range(len(eval_data) // seq)]
    rank, world = (dist.get_rank(), dist.get_world_size()) if distributed else (0, 1)
    total, scored = 0.0, 0
    try:
        for start, size in windows[rank::world]:
            x = torch.from_numpy(np.asarray(eval_data[start:start + size], dtype=np.int64)[None].copy()).to(dev)
            y = torch.from_numpy(np.asarray(eval_data[start + 1:start + size + 1], dtype=np.int64)[None].copy()).to(dev)
            logits = model(input_ids=x, use_cache=False).logits
            flat, target = logits.view(-1, logits.size(-1)), y.view(-1)
            rows = max(256, (8192 * 32768) // logits.size(-1))
            for o in range(0, target.numel(), rows):
                total += torch.nn.functional.cross_entropy(flat[o:o + rows].float(), target[o:o + rows], reduction="sum").item()
            scored += y.numel()
        if distributed:
            both = torch.tensor([total, scored], dtype=torch.float64, device=dev)
            dist.all_reduce(both)
            total, scored = both.tolist()
        if not scored:
            raise ValueError("No validation targets were scored")
        return total / scored
    finally:
        model.train(was_training)


# ------------------------------------------------------------------------------------------ trainer
def pick_device(name="auto", local_rank=0):
    if name == "cpu" or (name == "auto" and not torch.cuda.is_available()):
        return torch.device("cpu")
    if local_rank >= torch.cuda.device_count():
        raise ValueError("DDP ranks exceed visible GPUs")
    return torch.device("cuda", local_rank)


def gdn_kernel():
    """Where the chunked gated delta rule runs on a GPU: this library's kernels (the reference returns the FLA modules here and
    raises when the slow PyTorch fallback would be used, q38/train.py:267-273; so does this)."""
    from . import ops
    if not torch.cuda.is_available():
        raise RuntimeError("chunk_gated_delta_rule would run on the PyTorch fallback: no CUDA device")
    ops.load()
    return ["q38.ops (csrc/gdn.cu: gdn_prep_fwd/bwd, gdn_scan_fwd/bwd)"]


def install_fast_paths(model):
    """The reference's name for switching a model to its training fast paths (q38/train.py:285-308).  Here the fast paths are
    the process-wide kernel backend behind the model file's hooks: it is installed when the model is on a GPU, and the same
    kind of summary is returned."""
    from .inference import compile_inference_norms
    parameter = next(model.parameters())
    experts = "reference (PyTorch)"
    if parameter.is_cuda:
        from . import ops
        ops.install()
        experts = "grouped tcgen05 kernels"
    gdn = sum(type(m).__name__ == "Qwen3_8MoeGatedDeltaNet" for m in model.modules())
    return dict(experts=experts, gated_deltanet=gdn, norms=compile_inference_norms(model))


def build_model(cfg, dev, grad_ckpt=False):
    """fp32 master weights on `dev`; on a GPU the sm_100a kernel backend is installed and activations run in bf16."""
    model = Q38ForCausalLM(cfg).to(dev, dtype=torch.float32)
    model.tie_embeddings()
    model.model.gradient_checkpointing = bool(grad_ckpt)
    if dev.type == "cuda":
        from . import ops
        ops.install()                          # raises if the CUDA extension is missing: no silent PyTorch fallback
        model.model.compute_dtype = torch.bfloat16
    return model


class Trainer:
    """Model + objective + optimizer + gradient engine.  `train_step` is the unit the benchmark times.

    `batches` given to `train_step` is a list of ``(x, y)`` host tensors, one per micro-step (pinned when
    training on a GPU); the step copies them to the device, runs forward/backward for each, synchronises
    gradients on the last one, clips, updates and returns a 5-element device tensor
    ``[ce, aux, mtp, kl, grad_norm]`` averaged over micro-steps and ranks.
    """

    def __init__(self, cfg, a, dev, rank=0, world=1, model=None):
        self.cfg, self.a, self.dev, self.rank, self.world = cfg, a, dev, rank, world
        self.model = model if model is not None else build_model(cfg, dev, getattr(a, "grad_ckpt", 0))
        self.loss_model = LossModel(self.model, cfg.num_experts, cfg.num_experts_per_tok)
        from .parallel import GradEngine
        self.engine = GradEngine(self.model, dev, rank, world, mode=getattr(a, "grad_sync", "auto"),
                                 lr=a.lr, weight_decay=a.wd, muon=bool(a.muon), expert_parallel=getattr(a, "expert_parallel", 0))
        self.opt = self.engine.optimizer
        if self.engine.expert_parallel:
            from .models import modeling
            from .parallel.ep import ExpertParallel
            layers = cfg.num_hidden_layers + (1 if cfg.mtp else 0)
            modeling.get_backend().ep = ExpertParallel(
                self.engine.transport, rank, world, cfg.hidden_size, cfg.moe_intermediate_size, cfg.num_experts, cfg.num_experts_per_tok,
                tokens=a.micro_bs * a.seq, layers=layers, capacity_factor=float(getattr(a, "ep_capacity", 4.0)))
        if dev.type == "cuda":
            from .models import modeling
            modeling.get_backend().fp8_ffn = bool(getattr(a, "fp8_ffn", 0))      # routed experts on block-scaled MXFP8 GEMMs
        self.model.train()
        # One CUDA graph per (micro-batch shape, accumulation count, attention phase) replays forward + backward of a
        # micro-step without any per-kernel host work; the optimizer step stays eager.
        self.use_graphs = bool(getattr(a, "cuda_graphs", 1)) and dev.type == "cuda"
        self._graphs = {}
        self.replayed_launches = 0            # kernels of this library executed through graph replays
        if dev.type == "cuda":
            from .ops.backend import DEFERRED_GRADS, WGRAD_STREAM
            WGRAD_STREAM.enabled = bool(getattr(a, "overlap_wgrad", 1))   # weight gradients on a second stream during backward
            # small-parameter gradients are added into the arena by one multi-tensor launch per backward, flushed where the
            # weight-gradient stream is joined (up to +1 % on q38_c2; Q38_DEFER_SMALL_GRADS=0 returns them to autograd one by one)
            DEFERRED_GRADS.enabled = os.environ.get("Q38_DEFER_SMALL_GRADS", "1") != "0"

    def close(self):
        """Release peer mappings and detach the expert-parallel context from the kernel backend."""
        from .models import modeling
        backend = modeling.get_backend()
        if self.dev.type == "cuda":
            from .ops.backend import DEFERRED_GRADS, WGRAD_STREAM
            WGRAD_STREAM.join()
            WGRAD_STREAM.enabled = False
            DEFERRED_GRADS.flush()
            DEFERRED_GRADS.enabled = False
        if backend is not None and getattr(backend, "ep", None) is not None:
            backend.ep = None
        if backend is not None:
            backend.fp8_ffn = False
            if self.dev.type == "cuda":
                from .ops import fp8
                fp8.drop_weights()
        self._graphs = {}
        self.engine.close()

    def coefficients(self):
        return self.a.aux_coef, self.a.mtp_coef, self.a.kl_coef

    def micro_loss(self, x, y, accum):
        ce, aux, mtp, kl = self.loss_model(x, y)
        aux_c, mtp_c, kl_c = self.coefficients()
        return (ce + aux_c * aux + mtp_c * mtp + kl_c * kl) / accum, torch.stack(
            [ce.detach().float(), aux.detach().float(), mtp.detach().float(), kl.detach().float()])

    def _join_weight_gradients(self):
        """Weight-gradient GEMMs run on a second stream during backward (see q38.ops.backend._SideStream); wait for them."""
        if self.dev.type == "cuda":
            from .ops.backend import DEFERRED_GRADS, WGRAD_STREAM
            WGRAD_STREAM.join()
            DEFERRED_GRADS.flush()

    def _reset_generator_after_failed_capture(self):
        """A capture that ends with an error leaves the device's random-number generator marked as capturing, and the next
        `torch.randn` on the device raises.  A small capture that succeeds clears the mark."""
        try:
            probe = torch.zeros(8, device=self.dev)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                probe += 1
            torch.cuda.synchronize(self.dev)
            torch.randn(1, device=self.dev)
        except Exception as exc:                             # pragma: no cover - depends on the driver
            print(f"[q38.train] could not reset the generator after the failed capture ({type(exc).__name__})", flush=True)

    def _captured_micro_step(self, x, y, accum, dense):
        """Forward + backward of one micro-step through a CUDA graph (captured on first use of this configuration).
        Returns the 4 loss terms, or None when capture is unavailable and the caller should run eagerly."""
        key = (tuple(x.shape), accum, bool(dense))
        entry = self._graphs.get(key)
        if entry is None:
            try:
                sx = torch.zeros(x.shape, dtype=x.dtype, device=self.dev)
                sy = torch.zeros(y.shape, dtype=y.dtype, device=self.dev)
                sx.copy_(x)
                sy.copy_(y)
                saved = self.engine.arena.grads.clone()
                side = torch.cuda.Stream(self.dev)
                side.wait_stream(torch.cuda.current_stream(self.dev))
                with torch.cuda.stream(side):
                    for _ in range(2):                       # warm-up: lazy initialisation must not happen inside the capture
                        loss, _ = self.micro_loss(sx, sy, accum)
                        loss.backward()
                        self._join_weight_gradients()
                        # drop the warm-up graph now: while it lives, the parameters' gradient accumulators stay bound to this
                        # warm-up stream and the captured backward would run them there, outside the capturing stream
                        del loss, _
                torch.cuda.current_stream(self.dev).wait_stream(side)
                from . import ops
                graph = torch.cuda.CUDAGraph()
                before = ops.launch_count()
                with torch.cuda.graph(graph):
                    loss, parts = self.micro_loss(sx, sy, accum)
                    loss.backward()
                    self._join_weight_gradients()            # the weight-gradient branch rejoins the captured stream
                self.engine.arena.grads.copy_(saved)         # warm-up and capture passes must not leak into the gradients
                entry = (graph, sx, sy, parts, ops.launch_count() - before)
            except Exception as exc:                         # pragma: no cover - depends on the driver
                print(f"[q38.train] CUDA graph capture failed ({type(exc).__name__}: {exc}); running eagerly", flush=True)
                if os.environ.get("Q38_TRACE_CAPTURE"):
                    import traceback
                    traceback.print_exc()
                self.use_graphs = False
                torch.cuda.synchronize(self.dev)
                self._reset_generator_after_failed_capture()
                return None
            self._graphs[key] = entry
        graph, sx, sy, parts, launches = entry
        sx.copy_(x, non_blocking=True)
        sy.copy_(y, non_blocking=True)
        graph.replay()
        self.replayed_launches += launches
        return parts

    def train_step(self, batches, lr=None, dense=False):
        accum = len(batches)
        self.model.model.qsa_dense = bool(dense)
        if lr is not None:
            self.engine.set_lr(lr)
        totals = torch.zeros(4, dtype=torch.float32, device=self.dev)
        if self.dev.type == "cuda" and getattr(self.a, "fp8_ffn", 0):
            from .ops import fp8
            from .ops.backend import _bf16_weight
            fp8.refresh_weights(self.model, _bf16_weight)          # MXFP8 copies of the expert weights, once per optimizer step
        for i, (x, y) in enumerate(batches):
            self.engine.begin_micro_step(last=i == accum - 1)
            parts = self._captured_micro_step(x, y, accum, dense) if self.use_graphs else None
            if parts is None:
                xd, yd = x.to(self.dev, non_blocking=True), y.to(self.dev, non_blocking=True)
                loss, parts = self.micro_loss(xd, yd, accum)
                loss.backward()
                self._join_weight_gradients()
            totals += parts / accum
        grad_norm = self.engine.finish_step(self.a.clip)
        return self.engine.average_metrics(torch.cat([totals, grad_norm.detach().reshape(1).float()]))

    def read_step(self, result):
        """Host values ``[ce, aux, mtp, kl, grad_norm]`` of a step.  The device error word rides along in the same transfer:
        when a kernel reported a problem during the step (a peer that missed a barrier, a bounded wait that ran out) this
        raises `RuntimeError`; the update kernels have then left parameters and optimizer state untouched."""
        if self.dev.type != "cuda":
            return result.tolist()
        from . import ops
        flag = ops.error_flag(self.dev)
        values = torch.cat([result.float(), flag.float()]).tolist()
        code = int(values[-1])
        if code:
            flag.zero_()
            raise RuntimeError(f"q38 kernel error {code}: {ops.ERROR_NAMES.get(code, 'unknown')}; the step was not applied")
        return values[:-1]


def probe_micro_bs(trainer, train_data, a, log0):
    """Largest micro batch (a divisor of the per-rank sequences, at most ``--micro_bs``) whose
    forward+backward peak plus optimizer state fits into ``probe_mem_frac`` of the GPU memory.

    Runs on the bare loss model (no gradient synchronisation, so a rank that runs out of memory cannot
    stall a collective), never steps the optimizer and restores the RNG state; ranks agree on the
    result through an all-reduce(MIN)."""
    dev, world = trainer.dev, trainer.world
    candidates = micro_bs_candidates(a.batch_tokens // (a.seq * world), a.micro_bs)
    if len(candidates) == 1 or dev.type != "cuda":
        return candidates[0], []
    total = torch.cuda.get_device_properties(dev).total_memory
    reserve = trainer.opt.state_bytes()
    saved = torch.get_rng_state(), torch.cuda.get_rng_state(dev)
    rng = np.random.default_rng(0)
    chosen, trials = 0, []
    for m in candidates:
        peak = None
        try:
            torch.cuda.reset_peak_memory_stats(dev)
            for _ in range(2):                     # the second pass accumulates into existing gradients, as training does
                x, y = sample_batch(rng, train_data, m, a.seq, dev)
                loss, _ = trainer.micro_loss(x, y, 1)
                loss.backward()
                trainer._join_weight_gradients()
                del x, y, loss
            torch.cuda.synchronize(dev)
            peak = torch.cuda.max_memory_allocated(dev)
        except torch.cuda.OutOfMemoryError:
            pass
        trainer.engine.zero_grad()
        gc.collect()
        torch.cuda.empty_cache()
        fits = peak is not None and peak + reserve <= a.probe_mem_frac * total
        if world > 1:
            flag = torch.tensor(int(fits), device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            fits = bool(flag.item())
        trials.append(dict(micro_bs=m, peak_bytes=peak, reserve_bytes=reserve, fits=fits))
        shown = f"peak {peak / 2**30:.2f}G + optimizer {reserve / 2**30:.2f}G" if peak is not None else "OOM"
        log0(f"micro_bs probe {m}: {shown} / {a.probe_mem_frac:.0%} x {total / 2**30:.1f}G -> {'fits' if fits else 'too large'}")
        if fits:
            chosen = m
            break
    torch.set_rng_state(saved[0])
    torch.cuda.set_rng_state(saved[1], dev)
    torch.cuda.reset_peak_memory_stats(dev)
    if not chosen:
        raise RuntimeError("micro_bs=1 does not fit in GPU memory")
    return chosen, trials


def write_checkpoint(state, path):
    """Atomic checkpoint write: serialise to ``<path>.tmp``, then rename.  A crash or a failed write leaves the previous
    checkpoint in place; a leftover ``.tmp`` file is never read by a resume."""
    tmp = f"{path}.tmp"
    try:
        torch.save(state, tmp)
    except BaseException:
        with contextlib.suppress(OSError):
            os.remove(tmp)
        raise
    os.replace(tmp, path)


def export_hf(model, tokenizer, out_dir):
    """bf16 HF directory: weights, config with auto_map, tokenizer and the two model source files."""
    from .models.export import save_hf
    save_hf(model, out_dir, tokenizer=tokenizer, dtype=torch.bfloat16)


def _check_resume(a, plan, fc, tok_sha, sampler):
    previous = json.load(open(f"{a.run_dir}/run_config.json"))
    validate_resume_accounting(previous, fc)
    if previous.get("tokenizer_sha256", tok_sha) != tok_sha:
        raise ValueError("Unsafe resume: tokenizer contents changed; use a new run_dir")
    for key in RESUME_KEYS:
        fallback = previous.get("seed", 0) if key == "data_seed" else NEW_RESUME_DEFAULTS.get(key)
        if previous.get(key, fallback) != vars(a)[key]:
            raise ValueError(f"Unsafe resume: {key} changed; use a new run_dir")
    if "data_identity" in previous and previous["data_identity"] != plan["data_identity"]:
        raise ValueError("Unsafe resume: corpus identity changed")
    if sampler and previous.get("sampling") != plan["sampling"]:
        raise ValueError("Unsafe resume: shuffled block order changed")


def main(argv=None):
    a = parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    tok, cfg, fc, train_data, eval_data, final_data, sampler, plan = prepare_inputs(a, world)
    if a.dry_run:
        print(json.dumps(plan, indent=2, ensure_ascii=False))
        return plan
    os.makedirs(a.run_dir, exist_ok=True)
    ddp = world > 1
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dev = pick_device(a.device, local_rank)
    if dev.type == "cuda":
        torch.cuda.set_device(dev)
    rank = 0
    if ddp:
        dist.init_process_group("nccl" if dev.type == "cuda" else "gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(a.seed + rank)

    def log0(*items):
        if rank == 0:
            print(*items, flush=True)

    tok_sha = tokenizer_sha256(a.tokenizer)
    log0(f"Tokenizer: {a.tokenizer}, vocab={len(tok)}, bos={tok.bos_token_id}, eos={tok.eos_token_id}, pad={tok.pad_token_id}")
    trainer = Trainer(cfg, a, dev, rank, world)
    model, opt = trainer.model, trainer.opt
    log0("Model source:", source_info()["module"], "| gradient engine:", trainer.engine.describe())
    n_all = sum(p.numel() for p in model.parameters())
    n_total_nv = n_all - model.get_input_embeddings().weight.numel()
    n_active_nv = fc["active_nonvocab_params"]
    flops_per_token = fc["train_flops_per_token"]
    assert (fc["total_nonvocab_params"], fc["active_nonvocab_params"]) == (n_total_nv, n_active_nv), \
        "flops.py param count drifted from the model"
    log0(f"layers {cfg.layer_types}\nparams total={n_all / 1e6:.2f}M non-vocab total={n_total_nv / 1e6:.2f}M "
         f"active={n_active_nv / 1e6:.3f}M | train {flops_per_token / 1e6:.1f} MFLOP/token | "
         f"budget {a.tokens:.3e} tokens = {flops_per_token * a.tokens:.3e} FLOPs")
    log0(f"data: train {len(train_data) / 1e9:.2f}B tokens, validation {len(eval_data) / 1e6:.1f}M tokens "
         f"({a.val_data or 'tail of train.bin'}), world={world}")

    if a.auto_micro_bs:
        key = dict(world=world, gpu=torch.cuda.get_device_name(dev) if dev.type == "cuda" else "cpu",
                   gpu_bytes=torch.cuda.get_device_properties(dev).total_memory if dev.type == "cuda" else 0,
                   torch=torch.__version__, fast_paths=1, reserve="optimizer_state", probe_mem_frac=a.probe_mem_frac,
                   grad_ckpt=a.grad_ckpt, max_micro_bs=a.micro_bs, seq=a.seq, batch_tokens=a.batch_tokens,
                   model_sha256=hashlib.sha256(json.dumps(cfg.to_dict(), sort_keys=True).encode()).hexdigest())
        probe_path = Path(a.run_dir) / "micro_bs_probe.json"
        cached = torch.tensor(0, device=dev)
        if rank == 0 and probe_path.exists():
            previous = json.loads(probe_path.read_text())
            if previous.get("key") == key:
                cached.fill_(previous["micro_bs"])
        if ddp:
            dist.broadcast(cached, 0)
        if cached.item():
            a.micro_bs = int(cached.item())
            log0(f"micro_bs {a.micro_bs} (cached in {probe_path})")
        else:
            a.micro_bs, trials = probe_micro_bs(trainer, train_data, a, log0)
            if rank == 0:
                probe_path.write_text(json.dumps(dict(key=key, micro_bs=a.micro_bs, trials=trials), indent=1) + "\n")
    per_micro = a.micro_bs * a.seq * world
    if a.batch_tokens % per_micro:
        raise ValueError(f"batch_tokens {a.batch_tokens} must be divisible by micro_bs*seq*world={per_micro}")
    steps, accum = a.tokens // a.batch_tokens, a.batch_tokens // per_micro
    stop_step = min(steps, a.max_steps) if a.max_steps else steps
    rng = np.random.default_rng(a.data_seed + rank)
    lr_at = lr_schedule(a, steps)

    ckpt_path = f"{a.run_dir}/ckpt.pt"
    resuming = bool(a.resume) and os.path.exists(ckpt_path)
    if resuming:
        _check_resume(a, plan, fc, tok_sha, sampler)
    if ddp:
        dist.barrier()
    metrics = None
    if rank == 0:
        record = {**vars(a), "tokenizer_sha256": tok_sha, "data_dtype": TOKEN_DTYPE.str, "model_code": source_info(),
                  "data_identity": plan["data_identity"], "sampling": plan["sampling"], "config_sha256": plan["config_sha256"],
                  "n_params": n_all, "n_nonvocab_total": n_total_nv, "n_nonvocab_active": n_active_nv,
                  "flops_per_token": flops_per_token, "flops_accounting": fc["accounting_method"],
                  "flops_breakdown": fc["breakdown"], "steps": steps, "accum": accum, "config": cfg.to_dict()}
        with open(f"{a.run_dir}/run_config.json", "w") as f:
            json.dump(record, f, indent=1, ensure_ascii=False)
        metrics_file = open(f"{a.run_dir}/training_metrics.csv", "a" if resuming else "w", newline="")
        metrics = csv.writer(metrics_file)
        if not resuming:
            metrics.writerow(METRIC_COLUMNS)

    t0 = time.time()
    t_last, tok_seen, start_step = t0, 0, 0
    if resuming:
        ck = torch.load(ckpt_path, map_location="cpu", weights_only=False)
        trainer.engine.load_checkpoint(ck["model"], ck["opt"])
        start_step, tok_seen = ck["step"] + 1, ck["tok_seen"]
        if sampler and tok_seen != start_step * a.batch_tokens:
            raise ValueError("Checkpoint step/token count does not match the deterministic data stream")
        if len(ck.get("rank_rng", [])) == world:            # same world size: exact per-rank sample stream
            state = ck["rank_rng"][rank]
            rng.bit_generator.state = state["numpy"]
            torch.set_rng_state(state["torch"])
            if dev.type == "cuda" and state.get("cuda") is not None:
                torch.cuda.set_rng_state(state["cuda"], dev)
        elif rank == 0:
            rng.bit_generator.state = ck["rng"]
        else:
            rng = np.random.default_rng([a.data_seed + rank, start_step])
        if ck.get("world", 1) != world:
            log0("World size changed: global shuffled-block order is preserved" if sampler else
                 "World size changed: optimizer/token count restored; random sample stream differs")
        log0(f"resumed from {ckpt_path}: step {start_step}, tok_seen {tok_seen}")
        del ck
    tb = None
    if rank == 0 and a.tensorboard:                          # purge_step drops events logged past the restored checkpoint
        from torch.utils.tensorboard import SummaryWriter
        tb = SummaryWriter(f"{a.run_dir}/tb", purge_step=start_step if resuming else None)
        if not resuming:
            tb.add_text("run_config", f"```\n{json.dumps(vars(a), indent=1, ensure_ascii=False)}\n```")

    def save_ckpt(step):
        state = {"numpy": rng.bit_generator.state, "torch": torch.get_rng_state(),
                 "cuda": torch.cuda.get_rng_state(dev) if dev.type == "cuda" else None}
        states = [None] * world
        if ddp:
            dist.all_gather_object(states, state)
        else:
            states[0] = state
        trainer.engine.check_canaries()                                 # no peer wrote past the end of an arena since the last checkpoint
        model_state, opt_state = trainer.engine.checkpoint_state()      # collective: owners publish their optimizer shards
        if rank == 0:
            write_checkpoint({"model": model_state, "opt": opt_state, "step": step, "tok_seen": tok_seen,
                              "rng": rng.bit_generator.state, "rank_rng": states, "world": world}, ckpt_path)
        if ddp:
            # Serialising tens of GB takes longer than the bounded waits of the peer-memory barriers: nobody starts the next
            # step (and pushes parameters into rank 0's arena) before the file is complete.
            dist.barrier()

    log0(f"steps {steps} accum {accum} micro_bs {a.micro_bs} warmup {a.warmup} lr {a.lr}")
    pinned = dev.type == "cuda"
    for step in range(start_step, stop_step):
        batches = []
        for mi in range(accum):
            offsets = sampler.micro_offsets(step, mi, rank, world, a.micro_bs, a.batch_tokens) if sampler else None
            batches.append(host_batch(rng, train_data, a.micro_bs, a.seq, offsets, pinned=pinned))
        result = trainer.train_step(batches, lr=lr_at(step), dense=bool(a.dense_warmup and step < a.warmup))
        tok_seen += accum * per_micro
        loss_acc, aux_acc, mtp_acc, kl_acc, gn = trainer.read_step(result)   # the only host sync of the step; raises on a device error
        if tb:
            for name, value in (("loss", loss_acc), ("aux", aux_acc), ("mtp_loss", mtp_acc), ("indexer_kl", kl_acc),
                                ("lr", lr_at(step)), ("grad_norm", gn), ("tokens", tok_seen)):
                tb.add_scalar(f"train/{name}", value, step)
        if a.ckpt_every and step > 0 and step % a.ckpt_every == 0:
            save_ckpt(step)
        logging_step = step % a.log_every == 0 or step == stop_step - 1
        due = logging_step and ((step % a.eval_every == 0 and step > 0) or step == stop_step - 1)
        vl = ""
        if due:
            # Every rank takes part (disjoint windows, one all-reduce): no rank runs ahead into the next step's peer-memory
            # barriers while another is still scoring, and expert-parallel runs evaluate with every rank's experts.
            trainer.engine.gather_experts()
            vl = evaluate(model, eval_data, a.seq, dev, a.eval_sampling, distributed=ddp)
        if logging_step and rank == 0:
            now = time.time()
            tps = min(a.log_every, step - start_step + 1) * accum * per_micro / max(1e-6, now - t_last)
            metrics.writerow([step, tok_seen, f"{loss_acc:.8f}", f"{aux_acc:.8f}", f"{lr_at(step):.8e}", f"{gn:.6f}", f"{tps:.0f}",
                              f"{now - t0:.3f}", f"{vl:.8f}" if vl != "" else "", n_active_nv, n_total_nv,
                              f"{mtp_acc:.8f}", f"{kl_acc:.8f}"])
            metrics_file.flush()
            mem = torch.cuda.max_memory_allocated(dev) / 2**30 if dev.type == "cuda" else 0.0
            print(f"step {step}/{steps} tok {tok_seen / 1e6:.0f}M loss {loss_acc:.4f} mtp {mtp_acc:.3f} kl {kl_acc:.4f} "
                  f"aux {aux_acc:.3f} lr {lr_at(step):.2e} gn {gn:.2f} {tps:.0f} tok/s {(now - t0) / 60:.1f}min mem {mem:.1f}G"
                  + (f" | val {vl:.4f}" if vl != "" else ""), flush=True)
            if tb:
                tb.add_scalar("perf/tok_per_s", tps, step)
                tb.add_scalar("perf/max_mem_gib", mem, step)
                if vl != "":
                    tb.add_scalar("val/loss", vl, step)
                tb.flush()
            t_last = time.time()                             # validation time is not training throughput

    if stop_step > start_step:
        save_ckpt(stop_step - 1)
    final_loss = None
    if final_data is not None:
        trainer.engine.gather_experts()
        final_loss = evaluate(model, final_data, a.seq, dev, "sequential", distributed=ddp)
        if rank == 0:
            with open(f"{a.run_dir}/final_eval.json", "w") as f:
                json.dump(dict(loss=final_loss, metric="pure_cross_entropy", scored_tokens=len(final_data) - 1,
                               train_flops=flops_per_token * tok_seen, flops_accounting=fc["accounting_method"],
                               offset=a.final_eval_offset, tokenizer_sha256=tok_sha, tokens_trained=tok_seen,
                               completed_budget=tok_seen >= steps * a.batch_tokens), f, indent=2)
            log0(f"Final fixed validation CE: {final_loss:.8f} ({len(final_data) - 1:,} targets)")
    if tb:
        tb.close()
    if ddp:
        dist.barrier()
    if rank == 0:
        if a.export_hf:
            export_hf(model, tok, f"{a.run_dir}/hf")
        with open(f"{a.run_dir}/summary.json", "w") as f:
            json.dump({"tokens_trained": tok_seen, "train_flops": flops_per_token * tok_seen, "active_nonvocab": n_active_nv,
                       "flops_accounting": fc["accounting_method"], "total_nonvocab": n_total_nv,
                       "elapsed_s": time.time() - t0, "world": world, "completed_budget": tok_seen >= steps * a.batch_tokens,
                       "final_eval_loss": final_loss, "sampling": plan["sampling"]}, f, indent=1)
        with open(f"{a.run_dir}/flops.json", "w") as f:
            json.dump({**fc, "train_tokens": tok_seen, "train_flops": flops_per_token * tok_seen}, f, indent=2)
        print("DONE", f"{a.run_dir}/hf" if a.export_hf else a.run_dir, flush=True)
    trainer.close()
    if ddp:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
