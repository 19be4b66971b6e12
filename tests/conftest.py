import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `pytest -m gpu`)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


TINY_SHAPE = dict(layers=4, hidden=32, heads=2, kv_heads=1, lin_k_heads=1, lin_v_heads=2, experts=8, topk=2,
                  moe_ffn=8, shared_ffn=8, ngram_rows=64, qsa_blocks=1)


@pytest.fixture
def tiny_config():
    from q38.presets import model_config
    return model_config(dict(TINY_SHAPE), 128, 128, eos_token_id=0)
