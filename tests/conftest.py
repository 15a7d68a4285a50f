import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def golden_bigla():
    return dict(np.load(os.path.join(GOLDEN, "bigla_ref.npz")))


@pytest.fixture(scope="session")
def golden_block():
    return dict(np.load(os.path.join(GOLDEN, "block_ref.npz")))


def rel_err(a, b):
    """max|a-b| / max|b| with b the fp32 reference."""
    import torch
    a = torch.as_tensor(a).double().cpu()
    b = torch.as_tensor(b).double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))
