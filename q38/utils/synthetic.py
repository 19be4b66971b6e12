"""Synthetic packed token streams of the shapes the benchmarks name.

Ids are uniform over ``[1, vocab)`` (or Zipf(s)-distributed to skew expert routing) and an EOS token is
inserted at document boundaries whose gaps are geometric with the given mean, so n-gram context
resets and MTP target masking are exercised like on a real packed corpus."""
import numpy as np


def packed_stream(tokens, vocab, eos_id, mean_doc=1024, zipf=0.0, seed=0):
    rng = np.random.default_rng(seed)
    if zipf and zipf > 0:
        ranks = np.arange(1, vocab, dtype=np.float64)
        weights = ranks ** -zipf
        ids = rng.choice(np.arange(1, vocab), size=tokens, p=weights / weights.sum()).astype(np.int64)
    else:
        ids = rng.integers(1, vocab, tokens, dtype=np.int64)
    if eos_id is not None and mean_doc > 0:
        position = -1
        while True:
            position += int(rng.geometric(1.0 / mean_doc))
            if position >= tokens:
                break
            ids[position] = eos_id
    return ids


def batch_from_stream(stream, batch, seq, rng):
    """(x, y) int64 arrays ``[batch, seq]`` cut at random offsets; y is x shifted by one token."""
    starts = rng.integers(0, len(stream) - seq - 1, batch)
    x = np.stack([stream[s:s + seq] for s in starts]).astype(np.int64)
    y = np.stack([stream[s + 1:s + seq + 1] for s in starts]).astype(np.int64)
    return x, y
