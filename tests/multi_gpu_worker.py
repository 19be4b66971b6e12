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
    for mode in ("p2p", "p2p_pull", "p2p_push", "collective", "ep", "ep_graph"):
        # "p2p" takes the default reduce-scatter (the NVSwitch multimem kernels when a multicast mapping exists); the other
        # two force the peer-load and the push variants on CUDA IPC allocations
        os.environ["Q38_RS_ALGO"] = {"p2p_pull": "pull", "p2p_push": "push"}.get(mode, "auto")
        os.environ["Q38_PEER_ALLOC"] = "ipc" if mode in ("p2p_pull", "p2p_push") else "auto"
        torch.manual_seed(0)
        args = SimpleNamespace(**{**TRAIN_DEFAULTS, "aux_coef": 0.001, "lr": 3e-3, "grad_sync": "collective" if mode == "collective" else "p2p",
                                  "cuda_graphs": int(mode == "ep_graph"), "expert_parallel": int(mode.startswith("ep")), "micro_bs": 2, "seq": 256})
        trainer = Trainer(cfg, args, dev, rank, world)
        assert trainer.engine.mode == args.grad_sync
        if rank == 0 and trainer.engine.transport is not None:
            print(f"[{mode}] peer allocations: {trainer.engine.transport.alloc_backend}, reduce-scatter: {trainer.engine.transport.rs_algo}", flush=True)
        gen = torch.Generator().manual_seed(100 + rank)
        x = torch.randint(1, 512, (2, 256), generator=gen).pin_memory()
        y = x.roll(-1, 1).pin_memory()
        losses = [trainer.train_step([(x, y)], lr=3e-3, dense=(i == 0)).tolist() for i in range(5)]
        ops.check_errors()
        if mode == "ep_graph":
            assert trainer.use_graphs and trainer._graphs and trainer.replayed_launches > 0, "the expert-parallel micro-step was not replayed from a CUDA graph"
        state, _ = trainer.engine.checkpoint_state()           # assembles expert slices when the experts are split over ranks
        params = torch.cat([v.detach().float().reshape(-1) for k, v in sorted(state.items())])
        gathered = [torch.empty_like(params) for _ in range(world)]
        dist.all_gather(gathered, params)
        for other in gathered:
            if not torch.equal(other, params):
                offset, bad = 0, []
                for key, value in sorted(state.items()):
                    n = value.numel()
                    if not torch.equal(other[offset:offset + n], params[offset:offset + n]):
                        bad.append((key, (other[offset:offset + n] - params[offset:offset + n]).abs().max().item()))
                    offset += n
                raise AssertionError(f"{mode}: replicas differ in {bad[:8]} ({len(bad)} tensors)")
        arena = trainer.engine.arena
        assert torch.equal(arena.shadow, arena.params.to(torch.bfloat16)), f"{mode}: bf16 shadow out of sync"
        assert losses[-1][0] < losses[0][0], (mode, losses)
        results[mode] = (params, losses)
        transport = trainer.engine.transport
        if transport is not None:
            transport.check_canaries()                          # nothing wrote past the end of a peer-mapped buffer
            if mode == "p2p":                                   # and the check does see a guard byte that changed
                torch.cuda.synchronize()
                guard = transport.local["grads"]
                guard[-1] = 0
                try:
                    transport.check_canaries()
                    raise AssertionError("a changed guard byte went unnoticed")
                except RuntimeError as exc:
                    assert "overrun" in str(exc)
                guard[-1] = 0xA5
        trainer.close()
    for variant in ("p2p_pull", "p2p_push"):
        rel_v = ((results[variant][0] - results["collective"][0]).norm() / results["collective"][0].norm()).item()
        assert rel_v < 1e-2, f"{variant} disagrees with the collective transport: {rel_v}"
    a, b = results["p2p"][0], results["collective"][0]
    rel = ((a - b).norm() / b.norm()).item()
    first = abs(results["p2p"][1][0][0] - results["collective"][1][0][0])
    assert first < 1e-4, f"first-step losses differ: {first}"                 # same weights, same data, before any update
    # later steps differ by bf16 / atomic-accumulation noise amplified through Newton-Schulz; a transport bug would be O(1)
    assert rel < 1e-2, f"p2p and collective transports disagree: {rel}"
    for mode in ("ep", "ep_graph"):
        c = results[mode][0]
        rel_ep = ((c - b).norm() / b.norm()).item()
        first_ep = abs(results[mode][1][0][0] - results["collective"][1][0][0])
        assert first_ep < 1e-4, f"{mode}: first-step loss differs from the replicated-expert run: {first_ep}"
        assert rel_ep < 1e-2, f"{mode}: expert-parallel run disagrees with the replicated-expert run: {rel_ep}"
    if rank == 0:
        print(f"MULTI_GPU_OK world={world} rel={rel:.2e} loss {results['p2p'][1][0][0]:.4f} -> {results['p2p'][1][-1][0]:.4f}", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
