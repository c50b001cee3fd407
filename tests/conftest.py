"""Shared test setup: the `gpu` marker, the package loader and the fixtures directory."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests" / "fake_comfy")):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device of compute capability 10.0 (B200)")


@pytest.fixture(scope="session")
def pkg():
    import __graft_entry__ as g
    return g.load_package()


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    def load(name):
        return np.load(GOLDEN / name)
    return load


@pytest.fixture(scope="session")
def cuda_pkg(pkg):
    """The package with its native library loaded on a B200; GPU tests fail loudly otherwise."""
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    pkg._native.load()
    pkg._native.require_device(torch.device("cuda:0"))
    return pkg
