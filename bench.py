"""Headline benchmark: training tokens/second of the q38_c2 preset at sequence length 4096.

  python bench.py --gpus 1 --steps 3 --warmup 3
  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P bench.py --gpus 8 ...

One step is one optimizer step of the preset's global batch (262,144 tokens = 64 sequences), i.e.
``64 / (micro_bs * gpus)`` micro-steps of forward+backward per GPU followed by gradient synchronisation, clipping,
the Muon/AdamW update and the parameter publish: strong scaling, exactly what `python -m q38.train --preset q38_c2`
runs in its sparse-attention phase.  Data is a synthetic packed stream (uniform ids over the 10,112-token
vocabulary, EOS at geometric(mean 1024) document boundaries); weights are the preset's random initialisation.

The timed region is K steps between two barriers + device synchronisations, measured with CUDA events and
reduced with MAX over ranks.  Two numbers are reported: ``value`` with the micro-batches already resident on the
device, and ``e2e`` through the public `Trainer.train_step` API with every micro-batch copied from pinned host
memory inside the step and the step's loss vector read back to the host.
"""
import argparse
import json
import os
import sys
import time
from pathlib import Path
from types import SimpleNamespace

ROOT = Path(__file__).resolve().parent


def parse():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--preset", default="q38_c2")
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--micro_bs", type=int, default=0, help="sequences per GPU per micro-step (0 = the preset's)")
    ap.add_argument("--batch_tokens", type=int, default=0, help="global batch in tokens (0 = the preset's)")
    ap.add_argument("--phase", default="sparse", choices=("sparse", "dense"), help="QSA phase: block-sparse (steady state) or dense warm-up")
    ap.add_argument("--grad_sync", default="auto", choices=("auto", "p2p", "collective"))
    ap.add_argument("--zipf", type=float, default=0.0, help="Zipf exponent of the token distribution (0 = uniform)")
    ap.add_argument("--grad_ckpt", type=int, default=-1)
    ap.add_argument("--expert_parallel", type=int, default=0, help="1: split the experts over the GPUs (needs --gpus > 1)")
    ap.add_argument("--ep_capacity", type=float, default=4.0)
    ap.add_argument("--fp8_ffn", type=int, default=0, help="1: routed experts on block-scaled MXFP8 GEMMs (bf16 master weights, bf16 weight gradients)")
    ap.add_argument("--overlap_wgrad", type=int, default=1, help="0: weight-gradient GEMMs on the main stream instead of a second one")
    ap.add_argument("--cuda_graphs", type=int, default=1)
    return ap.parse_args()


def reference_arm(a):
    """Run the unmodified reference (baseline/_ref) in this process; this repository's q38 package is never imported."""
    sys.path[:] = [p for p in sys.path if Path(p or ".").resolve() != ROOT]
    sys.path.insert(0, str(ROOT / "baseline"))
    import ref_bench
    return ref_bench.main(a)


def main():
    a = parse()
    if a.impl == "reference":
        return reference_arm(a)
    sys.path.insert(0, str(ROOT))
    import numpy as np
    import torch
    import torch.distributed as dist
    from q38 import ops
    from q38.flops import count
    from q38.presets import load_preset, model_config
    from q38.train import TRAIN_DEFAULTS, Trainer
    from q38.utils.synthetic import batch_from_stream, packed_stream
    from q38.utils.timing import ClockSampler

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank, local_rank = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    if world != a.gpus:
        if world == 1 and a.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    preset = load_preset(a.preset)
    train = {**TRAIN_DEFAULTS, **preset["train"]}
    micro_bs = a.micro_bs or train["micro_bs"]
    batch_tokens = a.batch_tokens or train["batch_tokens"]
    per_micro = micro_bs * a.seq * world
    if batch_tokens % per_micro:
        raise SystemExit(f"global batch {batch_tokens} is not divisible by micro_bs*seq*gpus = {per_micro}")
    accum = batch_tokens // per_micro
    vocab, eos = 10112, 53
    cfg = model_config(preset["model"], vocab, a.seq, bos_token_id=1, eos_token_id=eos, pad_token_id=0)
    fc = count(cfg.to_dict(), a.seq)
    args = SimpleNamespace(**{**train, "aux_coef": preset["model"]["aux_coef"], "grad_sync": a.grad_sync, "micro_bs": micro_bs, "seq": a.seq,
                              "expert_parallel": a.expert_parallel, "fp8_ffn": a.fp8_ffn, "ep_capacity": a.ep_capacity, "overlap_wgrad": a.overlap_wgrad, "cuda_graphs": a.cuda_graphs,
                              "grad_ckpt": train.get("grad_ckpt", 0) if a.grad_ckpt < 0 else a.grad_ckpt})
    torch.manual_seed(0)
    trainer = Trainer(cfg, args, dev, rank, world)
    backend = ops.install()

    stream = packed_stream(1 << 22, vocab, eos, mean_doc=1024, zipf=a.zipf, seed=1234 + rank)
    rng = np.random.default_rng(99 + rank)

    def host_batches():
        out = []
        for _ in range(accum):
            x, y = batch_from_stream(stream, micro_bs, a.seq, rng)
            out.append((torch.from_numpy(x).pin_memory(), torch.from_numpy(y).pin_memory()))
        return out

    # fresh batches for every step (drawn before the timed region): the model never sees a sequence twice, so the timed steps
    # run on the statistics of random-init weights on random data rather than on a memorised pair of batches
    total_steps = a.warmup + 2 * a.steps
    pool = [host_batches() for _ in range(total_steps)]
    device_pool = [[(x.to(dev), y.to(dev)) for x, y in batches] for batches in pool]
    dense = a.phase == "dense"
    lr = train["lr"]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    cursor = [0]

    def run(steps, batches_pool, read_back):
        last = None
        for _ in range(steps):
            out = trainer.train_step(batches_pool[cursor[0] % len(batches_pool)], lr=lr, dense=dense)
            cursor[0] += 1
            last = trainer.read_step(out) if read_back else out
        return last

    run(a.warmup, device_pool, False)
    ops.check_errors()
    barrier()

    def timed(batches_pool, read_back):
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = ops.launch_count() + trainer.replayed_launches
        start.record()
        last = run(a.steps, batches_pool, read_back)
        stop.record()
        barrier()
        ms = torch.tensor(start.elapsed_time(stop), device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item(), ops.launch_count() + trainer.replayed_launches - launches0, last

    with ClockSampler(local_rank) as clocks:
        wall0 = time.time()
        ms_dev, launches, last = timed(device_pool, False)
        ms_e2e, _, last_host = timed(pool, True)
        wall = time.time() - wall0
    ops.check_errors()
    last = last.tolist() if hasattr(last, "tolist") else last
    tokens = a.steps * batch_tokens
    value = tokens / (ms_dev / 1e3)
    e2e = tokens / (ms_e2e / 1e3)
    peaks = {}
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    if peaks_path.exists():
        peaks = json.loads(peaks_path.read_text())
    peak_tflops = peaks.get("bf16_tflops_sustained", 1400.0)
    h2d = accum * 2 * micro_bs * a.seq * 8
    published = None          # the reference publishes no B200 number for this config
    phases = trainer.engine.phase_times()
    comm = trainer.engine.comm_report()

    def modeling_backend_report():
        from q38.models import modeling
        live = modeling.get_backend()
        return live.describe() if live is not None else backend

    if rank == 0:
        print(json.dumps({
            "metric": f"train tokens/sec, {a.preset} seq {a.seq}", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": ms_dev / a.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": published, "dtype": "bf16", "data": "synthetic packed stream (uniform ids, EOS at geometric(1024) boundaries; a fresh batch every step), random-init weights",
            "impl": "ours",
            "config": {"model": a.preset, "global_batch": batch_tokens // a.seq, "seq_len": a.seq, "micro_bs": micro_bs,
                       "accum": accum, "parallelism": f"dp{world}" + (f"+ep{world}" if a.expert_parallel and world > 1 else ""), "phase": a.phase, "grad_sync": trainer.engine.describe_transport(),
                       "grad_ckpt": int(args.grad_ckpt), "zipf": a.zipf, "fp8_ffn": int(a.fp8_ffn),
                       "l2": "no flush: one step streams >10 GB of activations and 1.3 GB of fp32 weights, far above the 126 MB L2",
                       "train_flops_per_token": fc["train_flops_per_token"]},
            "mfu_of_measured_sustained_peak": value * fc["train_flops_per_token"] / (world * peak_tflops * 1e12),
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / a.steps, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 5 * 4},
            "gpu_launches": launches, "peak_mem_gib": round(torch.cuda.max_memory_allocated(dev) / 2**30, 2), "clocks": clocks.summary(), "losses_last_step": last, "losses_last_step_e2e": last_host,
            "backend": modeling_backend_report(), "timed_wall_s": wall, "finish_step_phase_ms": phases, **comm,
        }), flush=True)
    trainer.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
