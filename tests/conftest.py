import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); deselect with -m 'not gpu'")


@pytest.fixture(scope="session")
def golden_teal():
    return np.load(os.path.join(GOLDEN, "teal.npz"))


@pytest.fixture(scope="session")
def golden_tq():
    return np.load(os.path.join(GOLDEN, "turboquant.npz"))


@pytest.fixture(scope="session")
def golden_cache():
    return np.load(os.path.join(GOLDEN, "cache_trace.npz"))


@pytest.fixture(scope="session")
def golden_codebooks():
    with open(os.path.join(GOLDEN, "codebooks_d128.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def golden_rotations():
    with open(os.path.join(GOLDEN, "rotations_d128.json")) as f:
        return json.load(f)


def rel_l2(a, b) -> float:
    import torch

    a = torch.as_tensor(a).double().flatten()
    b = torch.as_tensor(b).double().flatten()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))
