"""Forward-only evaluation of an HF export: JSONL -> packed stream -> bits per byte and EvalTime.

  torchrun --standalone --nproc_per_node=<gpus> -m q38.evaluate --dataset-path eval.jsonl --model-path run/hf

* Packing: every document becomes ``EOS, tokens...``; sequences are consecutive windows of the stream; a
  target is scored iff it is a text token (the inserted EOS is input only).  Right padding follows all
  valid targets, so it cannot influence them.
* bpb = total NLL / (ln 2 * UTF-8 bytes of the texts).
* EvalTime = forward seconds / (non-vocabulary active parameters in 1e9 * scored tokens in 1e6).  Only the
  forward pass including the vocabulary projection is timed; every step contributes the maximum over
  ranks.  Each batch shape is warmed five times before the timed pass.
* ``--profile-dir`` exports a short torch.profiler trace of the warmed forward (``--profile-only`` stops there).

Behaviour and result file follow the reference evaluator (q38/evaluate.py:26-71, 145-298).  The model runs
through this framework's kernels (`q38.ops`); the cross-entropy of the timed logits is computed outside the
timer in fp32 chunks.  Works on CPU with the gloo backend for tests (``--device cpu``).
"""
import argparse
import json
import math
import os
import tempfile
import time
from itertools import islice
from pathlib import Path

import numpy as np

TEXTS_PER_CALL = 128
SCORE_ROWS = 512


def pack_jsonl(dataset_path, tokenizer, cache_dir):
    """Write ``tokens.bin`` (int32) and ``is_text.bin`` (bool) into `cache_dir`; returns byte/token totals."""
    eos = tokenizer.eos_token_id
    if eos is None:
        raise ValueError("The tokenizer must define eos_token_id for document separation")
    n_bytes = n_tokens = 0
    cache_dir = Path(cache_dir)
    with Path(dataset_path).open(encoding="utf-8") as source, \
            (cache_dir / "tokens.bin").open("wb") as token_file, (cache_dir / "is_text.bin").open("wb") as mask_file:
        texts = (json.loads(line)["text"] for line in source if line.strip())
        while batch := list(islice(texts, TEXTS_PER_CALL)):
            n_bytes += sum(len(t.encode("utf-8")) for t in batch)
            encoded = tokenizer(batch, add_special_tokens=False, truncation=False, return_attention_mask=False,
                                return_token_type_ids=False, verbose=False)["input_ids"]
            for text, ids in zip(batch, encoded):
                if text and not ids:
                    raise ValueError("Tokenizer returned no tokens for nonempty text")
                np.asarray([eos] + list(ids), dtype=np.int32).tofile(token_file)
                flags = np.ones(len(ids) + 1, dtype=np.bool_)
                flags[0] = False
                flags.tofile(mask_file)
                n_tokens += len(ids)
    if not n_bytes or not n_tokens:
        raise ValueError("The dataset must contain nonempty text")
    pad = tokenizer.pad_token_id if tokenizer.pad_token_id is not None else eos
    return dict(total_bytes=n_bytes, total_tokens=n_tokens, pad_token_id=pad)


def packed_batch(tokens, is_text, start, stop, sequence_length, pad_token_id):
    """Inputs and labels (-100 = not scored) of sequences ``start..stop-1`` of the packed stream."""
    inputs = np.full((stop - start, sequence_length), pad_token_id, dtype=np.int64)
    labels = np.full_like(inputs, -100)
    for row, seq_index in enumerate(range(start, stop)):
        o = seq_index * sequence_length
        n = min(sequence_length, len(tokens) - 1 - o)
        inputs[row, :n] = tokens[o:o + n]
        labels[row, :n] = np.where(is_text[o + 1:o + n + 1], tokens[o + 1:o + n + 1], -100)
    return inputs, labels


def active_parameter_count(model):
    """Non-vocabulary parameters active per token: exactly top-k routed experts per layer, two n-gram rows,
    no training-only MTP block (the ledger's evaluation convention)."""
    from .flops import count
    return count(model.config.to_dict(), 4096)["active_nonvocab_params"]


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--dataset-path", type=Path, required=True, help="JSONL with a text field")
    ap.add_argument("--model-path", required=True, help="HF export directory")
    ap.add_argument("--batch-size", type=int, default=1, help="sequences per GPU")
    ap.add_argument("--sequence-length", type=int, default=4096)
    ap.add_argument("--output", type=Path, default=Path("result.json"))
    ap.add_argument("--profile-dir", type=Path, help="export a short forward-only trace before evaluation")
    ap.add_argument("--profile-only", action="store_true", help="stop after profiling")
    ap.add_argument("--device", default="auto", choices=("auto", "cuda", "cpu"))
    a = ap.parse_args(argv)
    if not 1 <= a.sequence_length <= 8192:
        ap.error("--sequence-length must be between 1 and 8192")
    if a.batch_size < 1:
        ap.error("--batch-size must be positive")
    if a.profile_only and a.profile_dir is None:
        ap.error("--profile-only requires --profile-dir")
    if not a.profile_only and a.output.exists():
        ap.error(f"Output already exists: {a.output}; choose a new --output path")
    return a


def profile_forward(forward_only, inputs, device, profile_dir, rank):
    """Trace five warmed forwards of one device-resident batch (wait 1, warm-up 1, active 3)."""
    import torch
    from torch.profiler import ProfilerActivity, profile, record_function, schedule
    profile_dir.mkdir(parents=True, exist_ok=True)
    trace_path, table_path = profile_dir / f"rank{rank}.trace.json", profile_dir / f"rank{rank}.operators.txt"
    activities = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if device.type == "cuda" else [])
    sort_keys = (["self_cuda_time_total"] if device.type == "cuda" else []) + ["self_cpu_time_total"]

    def save(prof):
        prof.export_chrome_trace(str(trace_path))
        head = f"Rank: {rank}\nInput shape: {tuple(inputs.shape)}\nDevice: {device}\nSchedule: wait=1, warmup=1, active=3\n"
        tables = [f"Sorted by {key}\n" + prof.key_averages().table(sort_by=key, row_limit=25) for key in sort_keys]
        table_path.write_text(head + "\n" + "\n\n".join(tables) + "\n")
        print(f"Trace: {trace_path}; operators: {table_path}", flush=True)

    with torch.inference_mode(), profile(activities=activities, schedule=schedule(wait=1, warmup=1, active=3, repeat=1),
                                         on_trace_ready=save) as prof:
        for _ in range(5):
            with record_function("inference_forward"):
                forward_only(inputs)
            prof.step()


def main(argv=None):
    a = parse_args(argv)
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    from transformers import PreTrainedTokenizerFast
    from .models.export import load_hf

    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = a.device == "cuda" or (a.device == "auto" and torch.cuda.is_available())
    device = torch.device("cuda", local_rank) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    own_group = not dist.is_initialized()
    if own_group:
        if "RANK" not in os.environ:            # plain `python -m q38.evaluate`: a single-rank group
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29533")
            os.environ.update(RANK="0", WORLD_SIZE="1")
        dist.init_process_group("nccl" if use_cuda else "gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(0)
    sync = (lambda: torch.cuda.synchronize(device)) if use_cuda else (lambda: None)
    a.output.parent.mkdir(parents=True, exist_ok=True)

    # Rank 0 tokenises into a temporary directory; the other ranks map the same files read-only.
    scratch, shared = None, [None]
    if rank == 0:
        scratch = tempfile.TemporaryDirectory(prefix=".eval-", dir=a.output.parent)
        tokenizer = PreTrainedTokenizerFast.from_pretrained(a.model_path, local_files_only=True)
        meta = pack_jsonl(a.dataset_path, tokenizer, Path(scratch.name).resolve())
        shared[0] = (str(Path(scratch.name).resolve()), meta)
        print(f"Packed {meta['total_tokens']} text tokens", flush=True)
    dist.broadcast_object_list(shared, src=0)
    cache_path, meta = shared[0]
    tokens = np.memmap(Path(cache_path) / "tokens.bin", dtype=np.int32, mode="r")
    is_text = np.memmap(Path(cache_path) / "is_text.bin", dtype=np.bool_, mode="r")
    n_seq = math.ceil((len(tokens) - 1) / a.sequence_length)
    global_bs = a.batch_size * world
    n_steps = math.ceil(n_seq / global_bs)

    model = load_hf(a.model_path, dtype=torch.bfloat16 if use_cuda else torch.float32, device=device)
    from .inference import optimize_for_inference
    print(f"Inference fast paths: {optimize_for_inference(model)}", flush=True)
    n_active = active_parameter_count(model)
    if n_active <= 0:
        raise ValueError("Non-vocabulary active parameter count must be positive")

    def batch_for(step):
        start = step * global_bs + rank * a.batch_size
        stop = min(start + a.batch_size, n_seq)
        if start >= stop:
            return None
        x, y = packed_batch(tokens, is_text, start, stop, a.sequence_length, meta["pad_token_id"])
        return torch.from_numpy(x).to(device), torch.from_numpy(y).to(device), int(np.count_nonzero(y != -100))

    def forward_only(x):
        return model(input_ids=x, use_cache=False).logits

    nll = torch.zeros((), device=device, dtype=torch.float64)
    scored, forward_seconds = 0, 0.0
    with torch.inference_mode():
        last_step = (n_seq - 1 - rank * a.batch_size) // global_bs
        warmed = set()
        for step in (0, last_step):
            batch = batch_for(step) if step >= 0 else None
            if batch is None or tuple(batch[0].shape) in warmed:
                continue
            warmed.add(tuple(batch[0].shape))
            for _ in range(5):
                forward_only(batch[0])
            sync()
        dist.barrier()
        if a.profile_dir is not None:
            batch = batch_for(0)
            if batch is not None:
                profile_forward(forward_only, batch[0], device, a.profile_dir, rank)
            dist.barrier()
        if not a.profile_only:
            for step in range(n_steps):
                batch, elapsed = batch_for(step), 0.0
                if batch is not None:
                    x, y, n_valid = batch
                    sync()                                      # host-to-device copies are not timed
                    started = time.perf_counter()
                    logits = forward_only(x)
                    sync()
                    elapsed = time.perf_counter() - started
                slowest = torch.tensor(elapsed, device=device, dtype=torch.float64)
                dist.all_reduce(slowest, op=dist.ReduceOp.MAX)  # replicas run concurrently: a step costs its slowest rank
                forward_seconds += slowest.item()
                if batch is not None:
                    flat, target = logits.reshape(-1, logits.shape[-1]), y.reshape(-1)
                    for o in range(0, target.numel(), SCORE_ROWS):
                        nll += F.cross_entropy(flat[o:o + SCORE_ROWS].float(), target[o:o + SCORE_ROWS],
                                               ignore_index=-100, reduction="sum").double()
                    scored += n_valid
            if rank == 0:
                print(f"Forward time: {forward_seconds:.3f}s", flush=True)

    result = None
    if not a.profile_only:
        count = torch.tensor(scored, device=device, dtype=torch.int64)
        dist.all_reduce(nll)
        dist.all_reduce(count)
        if count.item() != meta["total_tokens"]:
            raise RuntimeError("Scored token count does not match the original text token count")
        bpb = nll.item() / (math.log(2) * meta["total_bytes"])
        evaltime = forward_seconds / ((n_active / 1e9) * (meta["total_tokens"] / 1e6))
        if not (math.isfinite(bpb) and math.isfinite(evaltime) and evaltime > 0):
            raise RuntimeError("Evaluation produced a non-finite loss or invalid forward time")
        result = dict(model_path=a.model_path, bpb=bpb, evaltime=evaltime)
        if rank == 0:
            a.output.write_text(json.dumps(result, ensure_ascii=False, indent=2) + "\n")
            print(json.dumps(result, ensure_ascii=False), flush=True)
    dist.barrier()
    if own_group:
        dist.destroy_process_group()
    del tokens, is_text
    if scratch is not None:
        scratch.cleanup()
    return result


if __name__ == "__main__":
    main()
