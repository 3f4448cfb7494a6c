import os
import sys
import warnings
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

warnings.filterwarnings("ignore", message=".*fuse_linear_cross_entropy.*")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run on a B200)")
    config.addinivalue_line("markers", "slow: long-running test")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(0)
    yield


TINY_V9 = dict(
    hidden_size=128, num_hidden_layers=2, num_heads=4, num_kv_heads=2, head_dim=32, intermediate_size=384,
    vocab_size=1024, window_size=64, ttt_mode=True, ttt_chunk=16, ttt_visible_chunks=2, ttt_layers=[1],
    ttt_lr=1e-2, fuse_norm=False, fuse_swiglu=False, fuse_cross_entropy=False, ttt_force_grouped_scan=False,
)


@pytest.fixture
def tiny_v9_kwargs():
    return dict(TINY_V9)
