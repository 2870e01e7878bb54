import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU; run with -m gpu")


@pytest.fixture(scope="session")
def plb():
    """The package; the C-ABI library is built on demand (nvcc cross-compiles without a GPU)."""
    sys.path.insert(0, os.path.join(ROOT, "paddle-lite_b200"))
    import build as plb_build  # paddle-lite_b200/build.py
    plb_build.build()
    return importlib.import_module("paddle-lite_b200")


@pytest.fixture(scope="session")
def ctx(plb):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    c = plb.Context(0)
    yield c
    c.sync()
