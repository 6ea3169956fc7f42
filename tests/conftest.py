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


@pytest.fixture(scope="session")
def backend_x3(lib):
    """precision='tf32x3': split tf32 products with fp32-level results, the mode whose indices must be exact."""
    import grilly_b200

    b = grilly_b200.Compute(precision="tf32x3")
    yield b
    b.cleanup()


def index_mismatches(got, ref, k, tie_tol):
    """Compares the top-k column indices (descending) of every row of ``got`` with those of the reference ``ref``.

    Returns (rows that differ, rows that differ although the reference separates its top k+1 values by more than
    ``tie_tol`` x the row's largest magnitude). The second number must be zero: an implementation whose values carry
    a relative error of tie_tol cannot order values closer than that, anything else is a real mismatch."""
    got2, ref2 = got.reshape(-1, got.shape[-1]), np.asarray(ref, dtype=np.float64).reshape(-1, ref.shape[-1])
    top_got = np.argsort(-got2, axis=-1, kind="stable")[:, :k]
    order = np.argsort(-ref2, axis=-1, kind="stable")
    top_ref = order[:, :k]
    differ = (top_got != top_ref).any(-1)
    srt = np.take_along_axis(ref2, order[:, :k + 1], axis=-1)
    gaps = np.abs(np.diff(srt, axis=-1)).min(-1)
    scale = np.abs(ref2).max(-1)
    clear = gaps > tie_tol * scale
    return int(differ.sum()), int((differ & clear).sum())
