"""One command to start training, evaluation or a smoke run on the GPUs of this node.

  python -m q38.launch train --gpus 8 -- --preset q38_c2                 # torchrun -m q38.train on 8 GPUs
  python -m q38.launch eval  --gpus 8 -- --model runs/q38_c2/hf --data eval.jsonl
  python -m q38.launch smoke                                             # tiny synthetic train run, one GPU (or CPU)

It sets the environment the runs expect (``PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True``, ``OMP_NUM_THREADS``),
uses a loopback rendezvous (container hostnames do not always resolve), tees the output to ``logs/<name>.log`` and
returns the child's exit code.  (Reference: scripts/env.sh:6-15, scripts/train.sh:1-12, scripts/eval.sh:1-12, scripts/smoke.sh.)
"""
import argparse
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def environment(gpus):
    env = dict(os.environ)
    env.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    env.setdefault("OMP_NUM_THREADS", str(max(1, (os.cpu_count() or 8) // max(gpus, 1))))
    env.setdefault("MASTER_ADDR", "127.0.0.1")
    env["PYTHONPATH"] = f"{ROOT}{os.pathsep}{env['PYTHONPATH']}" if env.get("PYTHONPATH") else str(ROOT)
    return env


def command(module, gpus, port, rest):
    if gpus <= 1:
        return [sys.executable, "-m", module, *rest]
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}", "--master-addr", "127.0.0.1",
            "--master-port", str(port), "-m", module, *rest]


def smoke_arguments(run_dir):
    """A few optimizer steps of a tiny model on a synthetic packed corpus: exercises data, model, optimizer, checkpoint and export."""
    from .data import DEFAULT_TOKENIZER, prepare_synthetic
    run_dir.mkdir(parents=True, exist_ok=True)
    data = run_dir / "synthetic.bin"
    if not data.exists():
        prepare_synthetic(DEFAULT_TOKENIZER, data, 65536, mean_doc=256, seed=0)
    return ["--run_dir", str(run_dir), "--data", str(data), "--val_data", "", "--tokenizer", str(DEFAULT_TOKENIZER), "--layers", "4", "--hidden", "128",
            "--heads", "4", "--kv_heads", "2", "--lin_k_heads", "2", "--lin_v_heads", "4", "--experts", "8", "--topk", "2", "--moe_ffn", "32",
            "--shared_ffn", "32", "--ngram_rows", "1024", "--qsa_blocks", "2", "--mhc_iters", "5", "--seq", "256", "--micro_bs", "2",
            "--batch_tokens", "1024", "--tokens", "8192", "--eval_tokens", "2048", "--warmup", "2", "--log_every", "1", "--ckpt_every", "4",
            "--tensorboard", "0", "--resume", "0"]


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=("train", "eval", "smoke"))
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--port", type=int, default=29500)
    ap.add_argument("--log", default=None, help="log file (default logs/<what>.log); '-' disables the tee")
    ap.add_argument("--print", action="store_true", help="print the command line and exit")
    argv = list(sys.argv[1:] if argv is None else argv)
    rest = []
    if "--" in argv:                                   # everything after the first -- belongs to the module
        cut = argv.index("--")
        argv, rest = argv[:cut], argv[cut + 1:]
    a = ap.parse_args(argv)
    module = {"train": "q38.train", "eval": "q38.evaluate", "smoke": "q38.train"}[a.what]
    if a.what == "smoke":
        rest = smoke_arguments(ROOT / "runs" / "smoke") + rest
    cmd = command(module, a.gpus, a.port, rest)
    if a.print:
        print(" ".join(cmd))
        return 0
    log = None
    if a.log != "-":
        path = Path(a.log) if a.log else ROOT / "logs" / f"{a.what}.log"
        path.parent.mkdir(parents=True, exist_ok=True)
        log = open(path, "a")
    proc = subprocess.Popen(cmd, env=environment(a.gpus), cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    for line in proc.stdout:
        sys.stdout.write(line)
        if log:
            log.write(line)
            log.flush()
    if log:
        log.close()
    return proc.wait()


if __name__ == "__main__":
    raise SystemExit(main())
