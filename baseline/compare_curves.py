"""Loss curves of this repository's trainer math against the UNMODIFIED reference over N optimizer steps (CPU, fp32).

    python baseline/compare_curves.py --steps 200 --out profiles/loss_curve_vs_reference.md

Both sides start from the reference's initial weights (the reference side runs in a child process, `baseline/ref_oracle.py
curve`, because its package is also called ``q38``), see the same seeded synthetic batches (uniform ids, EOS at geometric
document boundaries), use the loss ``ce + 0.001 aux + 0.3 mtp + 0.05 kl``, gradient clipping at 1.0 and Muon + AdamW, with
dense attention for the first ``--dense_steps`` steps and block-sparse QSA afterwards.  The table lists both curves every
``--every`` steps and the largest relative difference of the main cross-entropy.
"""
import argparse
import json
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent

SHAPE = {"layers": 5, "hidden": 128, "heads": 4, "kv_heads": 2, "head_dim": 32, "lin_k_heads": 2, "lin_v_heads": 6, "experts": 16, "topk": 3,
         "moe_ffn": 32, "shared_ffn": 32, "n_branch": 4, "mhc_iters": 5, "qsa_blocks": 2, "indexer_heads": 4, "indexer_head_dim": 32,
         "ngram_rows": 2048, "mtp": 1}


def synthetic_tokens(vocab, eos, batch, seq, mean_doc, seed):
    """Same generator as `ref_oracle.synthetic_tokens` (kept in step by the test of the first batch below)."""
    rng = np.random.default_rng(seed)
    ids = rng.integers(1, vocab, (batch, seq + 1), dtype=np.int64)
    flat = ids.reshape(-1)
    position = -1
    while True:
        position += int(rng.geometric(1.0 / mean_doc))
        if position >= flat.size:
            break
        flat[position] = eos
    ids = torch.from_numpy(ids)
    return ids[:, :-1].contiguous(), ids[:, 1:].contiguous()


class PlainCE(torch.nn.Module):
    def forward(self, weight, hidden, labels):
        return F.cross_entropy(F.linear(hidden, weight), labels)


def own_curve(spec, init_state):
    sys.path.insert(0, str(ROOT))
    from q38.losses import LossModel
    from q38.models import Q38ForCausalLM
    from q38.muon import HybridOptimizer
    from q38.presets import model_config
    cfg = model_config(dict(spec["shape"]), spec["vocab"], spec["seq"], eos_token_id=spec["eos"], pad_token_id=0)
    model = Q38ForCausalLM(cfg).train()
    model.load_state_dict(init_state)
    wrapped = LossModel(model, spec["shape"]["experts"], spec["shape"]["topk"], ce=PlainCE())
    opt = HybridOptimizer(model, lr=spec["lr"], weight_decay=spec["wd"])
    rows = []
    for step in range(spec["steps"]):
        x, y = synthetic_tokens(spec["vocab"], spec["eos"], spec["batch"], spec["seq"], spec["mean_doc"], 1000 + step % spec["distinct_batches"])
        model.model.qsa_dense = step < spec["dense_steps"]
        parts = wrapped(x, y)
        (parts[0] + spec["shape"].get("aux_coef", 0.001) * parts[1] + spec["mtp_coef"] * parts[2] + spec["kl_coef"] * parts[3]).backward()
        gn = torch.nn.utils.clip_grad_norm_(model.parameters(), spec["clip"])
        opt.step()
        opt.zero_grad()
        rows.append([step] + [float(p) for p in parts] + [float(gn)])
    return rows


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--every", type=int, default=20)
    ap.add_argument("--dense_steps", type=int, default=10)
    ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    spec = dict(shape=SHAPE, vocab=10112, eos=53, seq=a.seq, batch=a.batch, steps=a.steps, lr=2e-3, wd=0.1, clip=1.0, mtp_coef=0.3, kl_coef=0.05,
                mean_doc=96, distinct_batches=16, dense_steps=a.dense_steps, seed=0)
    with tempfile.TemporaryDirectory() as tmp:
        out = Path(tmp) / "ref_curve.json"
        done = subprocess.run([sys.executable, str(HERE / "ref_oracle.py"), "curve", str(out), json.dumps(spec)], cwd="/tmp", capture_output=True, text=True)
        if done.returncode:
            raise SystemExit(done.stderr[-3000:])
        ref_rows = json.loads(out.read_text())["rows"]
        init = torch.load(str(out) + ".init.pt", weights_only=False)
    own_rows = own_curve(spec, init)
    worst = max(abs(o[1] - r[1]) / max(abs(r[1]), 1e-9) for o, r in zip(own_rows, ref_rows))
    lines = ["# Loss curve against the unmodified reference", "",
             f"`python baseline/compare_curves.py --steps {a.steps} --seq {a.seq} --batch {a.batch} --dense_steps {a.dense_steps}` (CPU, fp32, "
             f"{SHAPE['layers']} layers, hidden {SHAPE['hidden']}, {SHAPE['experts']} experts top-{SHAPE['topk']}, QSA budget {SHAPE['qsa_blocks']} blocks; "
             f"16 synthetic batches revisited; both sides start from the reference's initial weights).", "",
             f"Largest relative difference of the main cross-entropy over {a.steps} steps: **{worst:.2e}**.", "",
             "| step | ce (ours) | ce (reference) | mtp (ours) | mtp (ref) | kl (ours) | kl (ref) | aux (ours) | aux (ref) | grad norm (ours) | grad norm (ref) |",
             "|---|---|---|---|---|---|---|---|---|---|---|"]
    for o, r in zip(own_rows, ref_rows):
        if o[0] % a.every == 0 or o[0] == a.steps - 1:
            lines.append(f"| {o[0]} | {o[1]:.5f} | {r[1]:.5f} | {o[3]:.5f} | {r[3]:.5f} | {o[4]:.6f} | {r[4]:.6f} | {o[2]:.4f} | {r[2]:.4f} | {o[5]:.4f} | {r[5]:.4f} |")
    text = "\n".join(lines) + "\n"
    print(text)
    if a.out:
        Path(a.out).write_text(text)
    return 0 if worst < 2e-2 else 1


if __name__ == "__main__":
    sys.exit(main())
