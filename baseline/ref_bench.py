"""Reference arm of ``bench.py``: times the UNMODIFIED reference (``baseline/_ref``) through its own public code.

The step is the body of the reference's training loop (q38/train.py ``main``): ``Qwen3_8MoeForCausalLM(cfg)`` in fp32
→ ``install_fast_paths`` (FLA Gated DeltaNet + conv, ``grouped_mm`` experts, compiled norms) → ``LossModel`` (Liger
fused linear cross-entropy) → ``HybridOptimizer`` (Muon + AdamW) → ``DistributedDataParallel`` with
``gradient_as_bucket_view`` and ``no_sync`` on all but the last micro-step → bf16 autocast → ``clip_grad_norm_`` →
``opt.step()`` → one loss read-back per optimizer step.  Nothing of this repository's ``q38`` package is imported: the
process sees the reference's ``q38`` only, and no in-tree shared object is loaded.

Same preset, sequence length, micro batch, global batch, phase, synthetic stream, warm-up/steps protocol and JSON keys
as the repository's own arm.
"""
import importlib.util
import json
import os
import sys
import time
import traceback
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent


def _load_by_path(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def _clock_sampler():
    # q38/utils/timing.py of the repository has no package-relative imports; load it as a plain file.
    return _load_by_path("_bench_timing", ROOT / "q38" / "utils" / "timing.py").ClockSampler


def unavailable(reason):
    print(json.dumps({"impl": "reference", "unavailable": " ".join(str(reason).split())[:400]}), flush=True)
    return 0


def run(a):
    sys.path.insert(0, str(HERE))
    import ref_compat
    if not ref_compat.available():
        return unavailable("baseline/_ref is absent: copy the reference's q38/, configs/ and tokenizer/ there")
    try:
        ref_compat.activate()
        import numpy as np
        import torch
        import torch.distributed as dist
        import q38.train as T
        from q38.flops import count
        from q38.models.qwen3_8_moe import Qwen3_8MoeForCausalLM
        from q38.muon import HybridOptimizer
        from q38.presets import load_preset, model_config
    except Exception as exc:      # an import failure of the reference stack, not a GPU problem
        return unavailable(f"reference import failed: {type(exc).__name__}: {exc}")
    synthetic = _load_by_path("_bench_synthetic", ROOT / "q38" / "utils" / "synthetic.py")
    ClockSampler = _clock_sampler()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank, local_rank = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    ddp = world > 1
    if ddp:
        dist.init_process_group("nccl", device_id=dev)
    preset = load_preset(a.preset)
    train = {**T.TRAIN_DEFAULTS, **preset["train"]}
    micro_bs = a.micro_bs or train["micro_bs"]
    batch_tokens = a.batch_tokens or train["batch_tokens"]
    per_micro = micro_bs * a.seq * world
    if batch_tokens % per_micro:
        raise SystemExit(f"global batch {batch_tokens} is not divisible by micro_bs*seq*gpus = {per_micro}")
    accum = batch_tokens // per_micro
    vocab, eos = 10112, 53
    shape = dict(preset["model"])
    notes = []
    if os.environ.get("Q38_REF_EXPERTS"):
        shape["experts_impl"] = os.environ["Q38_REF_EXPERTS"]
    cfg = model_config(shape, vocab, a.seq, bos_token_id=1, eos_token_id=eos, pad_token_id=0)
    fc = count(cfg.to_dict(), a.seq)
    grad_ckpt = train.get("grad_ckpt", 0) if a.grad_ckpt < 0 else a.grad_ckpt
    torch.manual_seed(0 + rank)
    model = Qwen3_8MoeForCausalLM(cfg).to(dev, dtype=torch.float32)
    model.model.gradient_checkpointing = bool(grad_ckpt)
    try:
        gdn = T.gdn_kernel()
    except RuntimeError as exc:
        gdn = f"torch fallback ({exc})"
        notes.append(gdn)
    fast = T.install_fast_paths(model)
    lm = T.LossModel(model, shape["experts"], shape["topk"])
    opt = HybridOptimizer(model, lr=train["lr"], weight_decay=train["wd"], muon=bool(train["muon"]))
    if ddp:
        for p in model.parameters():
            p.grad = torch.zeros_like(p)
        lm = torch.nn.parallel.DistributedDataParallel(lm, device_ids=[local_rank], find_unused_parameters=True,
                                                       gradient_as_bucket_view=True)
    model.train()
    model.model.qsa_dense = a.phase == "dense"
    import contextlib

    stream = synthetic.packed_stream(1 << 22, vocab, eos, mean_doc=1024, zipf=a.zipf, seed=1234 + rank)
    rng = np.random.default_rng(99 + rank)

    def host_batches():
        out = []
        for _ in range(accum):
            x, y = synthetic.batch_from_stream(stream, micro_bs, a.seq, rng)
            out.append((torch.from_numpy(x).pin_memory(), torch.from_numpy(y).pin_memory()))
        return out

    pool = [host_batches() for _ in range(a.warmup + 2 * a.steps)]          # a fresh batch for every step, as in the repository's arm
    device_pool = [[(x.to(dev), y.to(dev)) for x, y in batches] for batches in pool]
    lr = train["lr"]
    aux_coef, mtp_coef, kl_coef, clip = shape["aux_coef"], train["mtp_coef"], train["kl_coef"], train["clip"]

    def train_step(batches):
        for g in opt.param_groups:
            g["lr"] = lr
        totals = torch.zeros(4, dtype=torch.float32, device=dev)
        for mi, (x, y) in enumerate(batches):
            x, y = x.to(dev, non_blocking=True), y.to(dev, non_blocking=True)
            sync = lm.no_sync() if (ddp and mi < accum - 1) else contextlib.nullcontext()
            with sync, torch.autocast("cuda", dtype=torch.bfloat16):
                ce, aux, mtp_loss, kl = lm(x, y)
                loss = (ce + aux_coef * aux + mtp_coef * mtp_loss + kl_coef * kl) / accum
            loss.backward()
            totals += torch.stack([ce.detach(), torch.as_tensor(aux, device=dev).detach(), mtp_loss.detach(), kl.detach()]).float() / accum
        grad_norm = torch.nn.utils.clip_grad_norm_(model.parameters(), clip)
        opt.step()
        opt.zero_grad(set_to_none=not ddp)
        if ddp:
            dist.all_reduce(totals)
            totals /= world
        return torch.cat([totals, grad_norm.detach().reshape(1)])

    def barrier():
        if ddp:
            dist.barrier()
        torch.cuda.synchronize(dev)

    cursor = [0]

    def run_steps(steps, batches_pool, read_back):
        last = None
        for _ in range(steps):
            out = train_step(batches_pool[cursor[0] % len(batches_pool)])
            cursor[0] += 1
            last = out.tolist() if read_back else out
        return last

    t_compile = time.time()
    run_steps(a.warmup, device_pool, True)
    barrier()
    cold = time.time() - t_compile

    def timed(batches_pool, read_back):
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        last = run_steps(a.steps, batches_pool, read_back)
        stop.record()
        barrier()
        ms = torch.tensor(start.elapsed_time(stop), device=dev, dtype=torch.float64)
        if ddp:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item(), last

    with ClockSampler(local_rank) as clocks:
        wall0 = time.time()
        ms_dev, last = timed(device_pool, False)
        ms_e2e, last_host = timed(pool, True)
        wall = time.time() - wall0
    last = last.tolist() if hasattr(last, "tolist") else last
    tokens = a.steps * batch_tokens
    value = tokens / (ms_dev / 1e3)
    e2e = tokens / (ms_e2e / 1e3)
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    peaks = json.loads(peaks_path.read_text()) if peaks_path.exists() else {}
    peak_tflops = peaks.get("bf16_tflops_sustained", 1400.0)
    if rank == 0:
        print(json.dumps({
            "metric": f"train tokens/sec, {a.preset} seq {a.seq}", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": ms_dev / a.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic packed stream (uniform ids, EOS at geometric(1024) boundaries; a fresh batch every step), random-init weights",
            "impl": "reference",
            "config": {"model": a.preset, "global_batch": batch_tokens // a.seq, "seq_len": a.seq, "micro_bs": micro_bs,
                       "accum": accum, "parallelism": f"dp{world}", "phase": a.phase, "grad_sync": "DDP all-reduce (NCCL)",
                       "grad_ckpt": int(grad_ckpt), "zipf": a.zipf,
                       "l2": "no flush: one step streams >10 GB of activations and 1.3 GB of fp32 weights, far above the 126 MB L2",
                       "train_flops_per_token": fc["train_flops_per_token"]},
            "mfu_of_measured_sustained_peak": value * fc["train_flops_per_token"] / (world * peak_tflops * 1e12),
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / a.steps,
                    "h2d_bytes_per_step": accum * 2 * micro_bs * a.seq * 8, "d2h_bytes_per_step": 5 * 4},
            "gpu_launches": 0, "clocks": clocks.summary(), "losses_last_step": last, "losses_last_step_e2e": last_host,
            "reference": {"path": "baseline/_ref (unmodified copy)", "gdn_kernel": gdn, "fast_paths": fast, "notes": notes,
                          "cold_start_s": cold, "torch": torch.__version__},
            "timed_wall_s": wall,
        }), flush=True)
    if ddp:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main(a):
    try:
        return run(a)
    except SystemExit:
        raise
    except Exception as exc:
        traceback.print_exc()
        if int(os.environ.get("RANK", "0")) == 0:
            unavailable(f"reference stock path raised {type(exc).__name__}: {exc}")
        return 0
