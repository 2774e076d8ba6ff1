import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(ROOT, "tests", "golden", "ref_small.npz")
    return dict(np.load(path))


@pytest.fixture(scope="session")
def golden_int8():
    return dict(np.load(os.path.join(ROOT, "tests", "golden", "ref_int8.npz")))


def bf16_from_bits(arr) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(arr)).view(torch.bfloat16)
