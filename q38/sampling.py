"""Deterministic, world-size independent training stream and evaluation windows.

`ShuffledBlockSampler` cuts the corpus into disjoint blocks of `seq` targets (each block reads
`seq + 1` adjacent tokens), shuffles the block ids once with PCG64 and hands out consecutive slices
of that single permutation.  Which slice a (step, micro-step, rank) triple reads depends only on the
global position, so any world size / micro-batch size consumes the same global stream and a resumed
run continues exactly where it stopped.  Behaviour follows the reference sampler
(q38/sampling.py:9-54); the permutation and its sha256 are bit-identical for equal seeds.
"""
import hashlib

import numpy as np

SAMPLER_VERSION = "pcg64-shuffled-disjoint-sequence-blocks-v1"


class ShuffledBlockSampler:
    def __init__(self, length, seq, seed):
        if seq < 1 or length <= seq:
            raise ValueError("Corpus must contain at least seq+1 tokens")
        self.seq, self.seed = seq, seed
        self.blocks = (length - 1) // seq
        self.order = np.random.default_rng(seed).permutation(self.blocks)
        self.sha256 = hashlib.sha256(self.order.astype("<i8", copy=False).tobytes()).hexdigest()

    def offsets(self, position, count):
        """Token offsets of `count` consecutive blocks of the permutation starting at `position`."""
        if position < 0 or count < 1 or position + count > self.blocks:
            raise ValueError("Training budget exceeds the no-replacement corpus; epoch wrapping is disabled")
        return self.order[position:position + count] * self.seq

    def micro_offsets(self, step, micro, rank, world, micro_bs, batch_tokens):
        if world < 1 or rank < 0 or rank >= world or micro < 0 or step < 0:
            raise ValueError("Invalid distributed sampler coordinates")
        per_micro = world * micro_bs * self.seq
        if batch_tokens % per_micro:
            raise ValueError("Global batch must be divisible by world*micro_bs*seq")
        if micro >= batch_tokens // per_micro:
            raise ValueError("Micro-step exceeds gradient accumulation")
        sequences_per_step = batch_tokens // self.seq
        return self.offsets(step * sequences_per_step + (micro * world + rank) * micro_bs, micro_bs)

    def metadata(self):
        return dict(version=SAMPLER_VERSION, seed=self.seed, blocks=self.blocks, sequence_length=self.seq,
                    order_sha256=self.sha256, replacement=False)


def sequential_windows(length, seq, offset=0, targets=0):
    """`(start, size)` windows that score every target once; the last window may be shorter."""
    available = length - offset - 1
    if seq < 1 or offset < 0 or available < 1 or targets < 0:
        raise ValueError("Invalid validation window")
    count = targets or available
    if count > available:
        raise ValueError("Requested validation targets exceed the available partition")
    end = offset + count
    return [(start, min(seq, end - start)) for start in range(offset, end, seq)]
