"""CPU-side checks: the C-ABI library builds, loads and exports every symbol the header declares; the ctypes
binding covers them all; the product refuses to run without a GPU; the host-side planners behave."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "grilly_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(grilly_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    names = declared_symbols()
    assert len(names) >= 35
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/grilly_b200.h but not exported by the library"


def test_ctypes_binding_matches_header():
    from grilly_b200 import _lib

    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_header_is_plain_c(tmp_path):
    """The boundary is a C ABI: the header must compile as C with no CUDA or C++ types."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("gcc not available")
    src = tmp_path / "t.c"
    src.write_text('#include "grilly_b200.h"\nint main(void){ grilly_encoder_config c; (void)c; return GRILLY_OK; }\n')
    subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-I", str(ROOT / "include"), "-c", str(src), "-o",
                    str(tmp_path / "t.o")], check=True)


def test_null_arguments_are_rejected_without_a_gpu(lib):
    from grilly_b200 import _lib

    assert lib.grilly_sync(None) == _lib.ERR_INVALID_ARG
    assert lib.grilly_linear(None, None, None, None, None, None, 1, 1, 1, 0, 0, 0) == _lib.ERR_INVALID_ARG
    assert lib.grilly_init(0, None) == _lib.ERR_INVALID_ARG
    assert lib.grilly_encoder_forward(None, None, None, 1, 1, None) == _lib.ERR_INVALID_ARG
    assert lib.grilly_last_error(None) == b"null context"


def test_no_cpu_fallback_without_gpu(lib):
    """On a machine without a GPU Compute() raises, as the reference's Compute() raises without Vulkan
    (backend/core.py:18-19); nothing silently computes on the CPU."""
    n = C.c_int(-1)
    rc = lib.grilly_device_count(C.byref(n))
    if rc == 0 and n.value > 0:
        pytest.skip("a GPU is present")
    import grilly_b200

    assert grilly_b200.CUDA_AVAILABLE is False
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        grilly_b200.Compute()


def test_product_does_not_import_the_oracle():
    for path in list((ROOT / "grilly_b200").rglob("*.py")) + list((ROOT / "grilly_b200" / "csrc").glob("*")):
        if path.is_file():
            text = path.read_text(errors="ignore")
            assert not re.search(r"^\s*(from|import)\s+oracle|oracle\.oracle|#include.*oracle", text, flags=re.M), \
                f"{path} uses the oracle"


def test_gemm_tile_choice(lib):
    # a wide output runs swapped (tokens are the MMA's N): many tokens get the widest tile, few get the narrow one
    assert lib.grilly_gemm_pick_tile(131072, 1152, 148) == 256
    assert lib.grilly_gemm_pick_tile(32, 1536, 148) == 64
    assert lib.grilly_gemm_pick_tile(100, 1536, 148) == 128
    # a narrow output stays un-swapped and tiles its own width
    assert lib.grilly_gemm_pick_tile(4096, 64, 148) == 64
    assert lib.grilly_gemm_pick_tile(16384, 16384, 148) == 256
    assert lib.grilly_gemm_pick_tile(0, 5, 148) < 0


def plan(lib, lengths, chunk):
    ln = np.asarray(lengths, dtype=np.int32)
    B = len(ln)
    bounds = np.zeros(B + 1, np.int32)
    cu = np.zeros(2 * B + 2, np.int32)
    tot = C.c_longlong(0)
    n = lib.grilly_plan_chunks(ln.ctypes.data, B, chunk, bounds.ctypes.data, cu.ctypes.data, C.byref(tot))
    assert n > 0
    return n, bounds[: n + 1], cu[: B + n], tot.value


def test_chunk_plan(lib):
    rng = np.random.default_rng(0)
    lengths = rng.integers(16, 129, size=200)
    n, bounds, cu, total = plan(lib, lengths, 1000)
    assert total == lengths.sum() and bounds[0] == 0 and bounds[-1] == 200
    off = 0
    for c in range(n):
        b0, b1 = bounds[c], bounds[c + 1]
        seg = cu[off: off + (b1 - b0) + 1]
        assert seg[0] == 0 and np.array_equal(np.diff(seg), lengths[b0:b1])
        assert seg[-1] <= 1000
        # greedy: the next sentence would not have fitted
        if b1 < 200:
            assert seg[-1] + lengths[b1] > 1000
        off += (b1 - b0) + 1
    # one chunk when the limit is off; an over-long sentence still gets its own chunk; empty sentences are kept
    assert plan(lib, lengths, 0)[0] == 1
    n, bounds, cu, total = plan(lib, [5, 300, 0, 7], 100)
    assert list(bounds) == [0, 1, 2, 4] and total == 312
    bad = np.array([3, -1], np.int32)
    assert lib.grilly_plan_chunks(bad.ctypes.data, 2, 0, bounds.ctypes.data, cu.ctypes.data, None) < 0
