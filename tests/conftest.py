"""Shared fixtures. Tests that need a B200 carry ``@pytest.mark.gpu``; everything else runs on CPU."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests" / "golden"))

# tolerances of the parity contract: relative L2 error against the reference's CPU implementation
TOL_TF32 = 2e-3
TOL_BF16 = 1e-2


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU; runs the CUDA path through the C ABI")


@pytest.fixture(scope="session")
def golden():
    return dict(np.load(ROOT / "tests" / "golden" / "hotpath_golden.npz"))


@pytest.fixture(scope="session")
def lib():
    from grilly_b200 import build

    build.build()  # no-op when the in-tree library is up to date
    from grilly_b200 import _lib

    return _lib.load()


@pytest.fixture(scope="session")
def backend(lib):
    """One Compute() per test session, like the reference's ``gpu_backend`` fixture (tests/conftest.py:17-29) --
    except that a missing GPU is an error here, not a skip: the gpu-marked tests must exercise the CUDA path."""
    import grilly_b200

    b = grilly_b200.Compute()
    yield b
    b.cleanup()


@pytest.fixture(scope="session")
def backend_bf16(lib):
    import grilly_b200

    b = grilly_b200.Compute(precision="bf16")
    yield b
    b.cleanup()
