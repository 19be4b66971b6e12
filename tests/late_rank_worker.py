"""Worker of the late-rank test (launched with torch.distributed.run on 2 to 4 GPUs, NVLS off).

Rank 0 sleeps on the host between two steps for longer than the (shortened) bounded wait of the peer-memory barrier.
Nothing faults and nothing hangs: the other ranks' barrier wait runs out, they record the error and raise every peer's
abort word; rank 0 finds the abort word when it arrives.  Every rank must then get a clean RuntimeError from
`Trainer.read_step`, with parameters and optimizer state exactly as they were before the step, and the CUDA context must
still work."""
import os
import sys
import time
from pathlib import Path
from types import SimpleNamespace

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def main():
    from q38 import ops
    from q38.presets import model_config
    from q38.train import TRAIN_DEFAULTS, Trainer
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    shape = dict(layers=4, hidden=128, heads=4, kv_heads=2, lin_k_heads=2, lin_v_heads=6, experts=8, topk=2, moe_ffn=32, shared_ffn=32,
                 ngram_rows=1024, mhc_iters=5, qsa_blocks=2)
    cfg = model_config(shape, 512, 256, eos_token_id=7, pad_token_id=0)
    torch.manual_seed(0)
    args = SimpleNamespace(**{**TRAIN_DEFAULTS, "aux_coef": 0.001, "lr": 3e-3, "grad_sync": "p2p", "cuda_graphs": 0, "micro_bs": 2, "seq": 256})
    trainer = Trainer(cfg, args, dev, rank, world)
    assert trainer.engine.transport.wait_seconds <= 2.0, "run this worker with Q38_PEER_WAIT_SECONDS=1"
    gen = torch.Generator().manual_seed(100 + rank)
    x = torch.randint(1, 512, (2, 256), generator=gen).pin_memory()
    y = x.roll(-1, 1).pin_memory()
    for _ in range(2):
        trainer.read_step(trainer.train_step([(x, y)], lr=3e-3))
    arena = trainer.engine.arena
    torch.cuda.synchronize(dev)
    before = [t.clone() for t in (arena.params, arena.exp_avg, arena.exp_avg_sq, arena.muon_buf, arena.shadow)]
    dist.barrier()
    if rank == 0:
        time.sleep(3.0)                                   # a host-side stall between steps, longer than the bounded wait
    raised = False
    try:
        trainer.read_step(trainer.train_step([(x, y)], lr=3e-3))
    except RuntimeError as exc:
        raised = "not applied" in str(exc)
    torch.cuda.synchronize(dev)
    assert raised, f"rank {rank}: the step with a late peer did not raise"
    for now, then, name in zip((arena.params, arena.exp_avg, arena.exp_avg_sq, arena.muon_buf, arena.shadow), before,
                               ("params", "exp_avg", "exp_avg_sq", "muon_buf", "shadow")):
        assert torch.equal(now, then), f"rank {rank}: {name} changed although the step was aborted"
    assert torch.ones(8, device=dev).sum().item() == 8.0          # the context is still usable
    dist.barrier()                                                  # every rank is between steps, nothing in flight
    if rank == 0:
        print(f"LATE_RANK_OK world={world}", flush=True)
    trainer.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
