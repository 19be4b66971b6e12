"""Worker of the multi-GPU tests (launched with torch.distributed.run, one rank per GPU).

Runs a few optimizer steps of a small model with the peer-memory transport and with the library collectives from the
same initial weights and data, and checks: (1) both transports end with the same parameters, (2) the replicas of all
ranks are bit-identical, (3) the loss decreases."""
import os
import sys
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
    results = {}
    for mode in ("p2p", "collective"):
        torch.manual_seed(0)
        args = SimpleNamespace(**{**TRAIN_DEFAULTS, "aux_coef": 0.001, "lr": 3e-3, "grad_sync": mode, "cuda_graphs": 0})
        trainer = Trainer(cfg, args, dev, rank, world)
        assert trainer.engine.mode == mode
        gen = torch.Generator().manual_seed(100 + rank)
        x = torch.randint(1, 512, (2, 256), generator=gen).pin_memory()
        y = x.roll(-1, 1).pin_memory()
        losses = [trainer.train_step([(x, y)], lr=3e-3, dense=(i == 0)).tolist() for i in range(5)]
        ops.check_errors()
        params = trainer.engine.arena.params.clone()
        gathered = [torch.empty_like(params) for _ in range(world)]
        dist.all_gather(gathered, params)
        for other in gathered:
            assert torch.equal(other, params), f"{mode}: replicas differ"
        assert torch.equal(trainer.engine.arena.shadow, params.to(torch.bfloat16)), f"{mode}: bf16 shadow out of sync"
        assert losses[-1][0] < losses[0][0], (mode, losses)
        results[mode] = (params, losses)
        trainer.engine.close()
    a, b = results["p2p"][0], results["collective"][0]
    rel = ((a - b).norm() / b.norm()).item()
    first = abs(results["p2p"][1][0][0] - results["collective"][1][0][0])
    assert first < 1e-4, f"first-step losses differ: {first}"                 # same weights, same data, before any update
    # later steps differ by bf16 / atomic-accumulation noise amplified through Newton-Schulz; a transport bug would be O(1)
    assert rel < 1e-2, f"p2p and collective transports disagree: {rel}"
    if rank == 0:
        print(f"MULTI_GPU_OK world={world} rel={rel:.2e} loss {results['p2p'][1][0][0]:.4f} -> {results['p2p'][1][-1][0]:.4f}", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
