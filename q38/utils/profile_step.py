"""Single-GPU training / inference step profile on synthetic tokens.

  python -m q38.utils.profile_step --preset q38_c2 --mode train --out profile.json

Reports ``forward_ms / backward_ms / optimizer_ms`` (CUDA events, median of ``--repeats`` after ``--warmup`` untimed
iterations, eager launches so that the phases can be separated), the tokens per second they imply, and the device time of every
kernel of one step (torch.profiler), grouped by kernel name.  ``--mode infer`` times the forward pass under ``no_grad``.
(Reference: scripts/profile_q38.py:1-53.)
"""
import argparse
import json
import statistics
from types import SimpleNamespace

import torch


def build_trainer(preset_name, seq, micro_bs, grad_ckpt=0):
    from ..presets import load_preset, model_config
    from ..train import ENGINE_DEFAULTS, TRAIN_DEFAULTS, Trainer
    preset = load_preset(preset_name)
    train = {**TRAIN_DEFAULTS, **ENGINE_DEFAULTS, **preset["train"]}
    train.update(aux_coef=preset["model"].get("aux_coef", 0.001), seq=seq or train["seq"], micro_bs=micro_bs or train["micro_bs"], grad_ckpt=grad_ckpt, cuda_graphs=0, grad_sync="collective")
    cfg = model_config(preset["model"], 10112, train["seq"], bos_token_id=1, eos_token_id=53, pad_token_id=0)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    return Trainer(cfg, SimpleNamespace(**train), dev), train


def timed(fn):
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    out = fn()
    stop.record()
    torch.cuda.synchronize()
    return out, start.elapsed_time(stop)


def kernel_table(run, limit):
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
        run()
        torch.cuda.synchronize()
    rows = []
    for e in prof.key_averages():
        t = getattr(e, "self_device_time_total", 0) or 0
        if t > 0 and e.device_type.name == "CUDA":
            rows.append(dict(kernel=e.key[:160], ms=round(t / 1e3, 4), launches=e.count))
    rows.sort(key=lambda r: -r["ms"])
    return dict(total_ms=round(sum(r["ms"] for r in rows), 3), kernels=rows[:limit])


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--preset", default="q38_c2")
    ap.add_argument("--mode", choices=("train", "infer"), default="train")
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--micro_bs", type=int, default=0)
    ap.add_argument("--grad_ckpt", type=int, default=0)
    ap.add_argument("--dense", type=int, default=0, help="1: dense attention (warm-up phase)")
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--repeats", type=int, default=3)
    ap.add_argument("--top", type=int, default=40)
    ap.add_argument("--out", default="")
    a = ap.parse_args(argv)
    from .. import ops
    tr, train = build_trainer(a.preset, a.seq, a.micro_bs, a.grad_ckpt)
    bs, seq = train["micro_bs"], train["seq"]
    x = torch.randint(1, 10112, (bs, seq), device=tr.dev)
    y = x.roll(-1, 1)
    tr.model.model.qsa_dense = bool(a.dense)
    phases = dict(forward_ms=[], backward_ms=[], optimizer_ms=[])

    def forward():
        if a.mode == "infer":
            with torch.no_grad():
                return tr.micro_loss(x, y, 1)[0]
        return tr.micro_loss(x, y, 1)[0]

    def step(record):
        loss, f = timed(forward)
        b = o = 0.0
        if a.mode == "train":
            _, b = timed(lambda: (loss.backward(), tr._join_weight_gradients()))
            _, o = timed(lambda: tr.engine.finish_step(train["clip"]))
        if record:
            phases["forward_ms"].append(f), phases["backward_ms"].append(b), phases["optimizer_ms"].append(o)

    for _ in range(a.warmup):
        step(False)
    launches = ops.launch_count()
    for _ in range(a.repeats):
        step(True)
    launches = (ops.launch_count() - launches) // a.repeats
    med = {k: round(statistics.median(v), 3) for k, v in phases.items()}
    total = sum(med.values())
    report = dict(preset=a.preset, mode=a.mode, micro_bs=bs, seq=seq, dense=bool(a.dense), grad_ckpt=a.grad_ckpt, **med, step_ms=round(total, 3),
                  tok_per_s=round(bs * seq / total * 1e3, 1), extension_launches_per_step=launches, device=torch.cuda.get_device_name(0),
                  profile=kernel_table(lambda: step(False), a.top))
    text = json.dumps(report, indent=1)
    if a.out:
        with open(a.out, "w") as f:
            f.write(text)
    print(json.dumps({k: v for k, v in report.items() if k != "profile"}))
    for row in report["profile"]["kernels"][:a.top]:
        print(f"{row['ms']:9.3f} ms  x{row['launches']:<5d} {row['kernel'][:120]}")
    tr.close()


if __name__ == "__main__":
    main()
