"""Stream fairness, resume and evaluation windows (counterpart of the reference's tests/test_isoflops.py)."""
import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from q38.sampling import ShuffledBlockSampler, sequential_windows
from q38.train import evaluate, lr_schedule, micro_bs_candidates


def test_global_stream_is_independent_of_world_and_micro_batch():
    sampler = ShuffledBlockSampler(4097, 8, 7)
    expected = sampler.offsets(0, 32)
    for world, micro_bs in [(1, 1), (1, 4), (1, 8), (2, 1), (2, 2), (4, 1), (8, 1)]:
        got = []
        for step in range(4):
            for micro in range(64 // (world * micro_bs * 8)):
                for rank in range(world):
                    got.extend(sampler.micro_offsets(step, micro, rank, world, micro_bs, 64))
        np.testing.assert_array_equal(got, expected)
    targets = np.concatenate([np.arange(o + 1, o + 9) for o in expected])
    assert len(np.unique(targets)) == len(targets)


def test_resume_and_no_wrapping():
    a, b = ShuffledBlockSampler(4097, 8, 42), ShuffledBlockSampler(4097, 8, 42)
    assert a.sha256 == b.sha256
    np.testing.assert_array_equal(a.offsets(80, 8), b.micro_offsets(10, 0, 0, 1, 8, 64))
    assert not np.array_equal(a.order, ShuffledBlockSampler(4097, 8, 43).order)
    with pytest.raises(ValueError):
        a.offsets(a.blocks - 1, 2)
    with pytest.raises(ValueError):
        a.micro_offsets(0, 0, 0, 3, 1, 64)


def test_sequential_evaluation_scores_every_target_once():
    assert sequential_windows(12, 4) == [(0, 4), (4, 4), (8, 3)]

    class Uniform(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.seen = []

        def forward(self, input_ids, use_cache=False):
            self.seen.extend(input_ids[0].tolist())
            return SimpleNamespace(logits=torch.zeros((*input_ids.shape, 32)))

    model = Uniform().train()
    loss = evaluate(model, np.arange(12, dtype="<u4"), 4, torch.device("cpu"), "sequential")
    assert abs(loss - math.log(32)) < 1e-6
    assert model.seen == list(range(11)) and model.training


def test_schedule_endpoints_and_candidates():
    sched = lr_schedule(SimpleNamespace(lr=0.004, warmup=11, min_lr_ratio=0.1), 223)
    assert abs(sched(10) - 0.004) < 1e-12 and abs(sched(222) - 0.0004) < 1e-12
    assert micro_bs_candidates(16, 8) == [8, 4, 2, 1] and micro_bs_candidates(6, 4) == [3, 2, 1]
