"""Shared pytest configuration: markers, seeding, small fixtures.

GPU tests carry ``@pytest.mark.gpu`` and are skipped automatically when no CUDA device is
present; everything else runs on CPU (multi-process paths use the gloo backend).
"""
import os
import random
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

os.environ.setdefault("WANDB_MODE", "disabled")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    config.addinivalue_line("markers", "slow: long-running test")
    config.addinivalue_line("markers", "integration: end-to-end test")
    config.addinivalue_line("markers", "multigpu: needs more than one CUDA device")


def pytest_collection_modifyitems(config, items):
    has_cuda = torch.cuda.is_available()
    n_gpu = torch.cuda.device_count() if has_cuda else 0
    skip_gpu = pytest.mark.skip(reason="no CUDA device")
    skip_multi = pytest.mark.skip(reason="needs >= 2 CUDA devices")
    for item in items:
        if "gpu" in item.keywords and not has_cuda:
            item.add_marker(skip_gpu)
        if "multigpu" in item.keywords and n_gpu < 2:
            item.add_marker(skip_multi)


@pytest.fixture(autouse=True)
def _seed_everything():
    random.seed(42)
    np.random.seed(42)
    torch.manual_seed(42)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(42)
    yield


@pytest.fixture
def cuda_status():
    """Checks the device status word after a GPU test (bounded waits that ran out set it)."""
    yield
    if torch.cuda.is_available():
        from nanoplm_b200.ops import _lib
        torch.cuda.synchronize()
        _lib.check_status()
