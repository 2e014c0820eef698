import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100); run with -m gpu on a B200 box")


@pytest.fixture(scope="session")
def gguf_witness():
    return dict(np.load(os.path.join(GOLDEN, "gguf_witness.npz")))


@pytest.fixture(scope="session")
def aten_witness():
    return dict(np.load(os.path.join(GOLDEN, "aten_witness.npz")))


@pytest.fixture(scope="session")
def ctx():
    """One library context on cuda:0 for the whole GPU session."""
    import torch

    import tattletale_b200 as ttq

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    c = ttq.Context(0)
    yield c
    c.check_device_status()  # no kernel gave up a bounded wait during the session
    c.close()


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / den) if den > 0 else float(np.linalg.norm(a - b))
