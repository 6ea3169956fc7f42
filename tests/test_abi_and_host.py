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


def test_importing_the_package_maps_no_cuda_library():
    """The CPU arm of the benchmark imports grilly_b200.encoder for the weight container only: that import must
    not load libgrilly_b200.so (checked in a fresh interpreter through /proc/self/maps)."""
    import subprocess
    import sys

    code = ("import grilly_b200, grilly_b200.encoder; "
            "print(any('libgrilly_b200' in line for line in open('/proc/self/maps')))")
    out = subprocess.run([sys.executable, "-c", code], cwd=str(ROOT), capture_output=True, text=True, check=True)
    assert out.stdout.strip() == "False"


def test_pool_stats_have_the_reference_keys():
    """backend.fnn.buffer_pool.get_stats() as tutorials/06_transformer_components.py:142-145 reads it
    (keys of BufferPool.get_stats, backend/buffer_pool.py:627-640)."""
    from grilly_b200.compute import _PoolView

    class FakeDevice:
        def pool_stats(self):
            return {"acquired": 40, "released": 38, "bytes_in_use": 1024, "peak_bytes": 4096, "pool_reserved_bytes": 8192,
                    "tensor_map_hits": 7, "tensor_map_misses": 3, "pool_hits": 30, "cached_weights": 2}

    pool = _PoolView(FakeDevice())
    stats = pool.get_stats()
    line = f"\nBuffer pool: {stats['total_acquired']} ops, {stats['hit_rate']:.1%} hit rate"   # the tutorial's line
    assert line == "\nBuffer pool: 40 ops, 75.0% hit rate"
    for key in ("hits", "misses", "allocations", "evictions", "total_acquired", "total_released", "total_pooled_memory",
                "buckets", "hit_rate", "vma_enabled"):
        assert key in stats
    assert stats["hits"] + stats["misses"] == stats["total_acquired"] and stats["allocations"] == stats["misses"] == 10
    assert stats["total_pooled_memory"] == 8192 - 1024 and stats["cached_weights"] == 2


class _FakeTensor:
    def __init__(self, host):
        self.host, self.freed = np.array(host, copy=True), False
        self.shape = self.host.shape

    def free(self):
        self.freed = True


def _fake_device():
    from grilly_b200.device import Device

    dev = object.__new__(Device)
    dev._weights, dev._pinned, dev._closed = {}, {}, True
    dev.uploads = 0

    def upload(arr, dtype="f32", round_tf32=False):
        dev.uploads += 1
        return _FakeTensor(arr)

    dev.upload = upload
    return dev


def test_weight_cache_follows_the_owner_of_the_buffer():
    """Device.weight caches by buffer identity while the owning ndarray lives, never serves a freed address, and
    does not cache what is not an ndarray."""
    import gc

    dev = _fake_device()
    w = np.arange(12, dtype=np.float32).reshape(3, 4)
    t1 = dev.weight(w)
    assert dev.weight(w) is t1 and dev.uploads == 1
    assert dev.weight(w.T) is not t1 and dev.weight(w.T) is dev.weight(w.T)      # a view: own entry, alive with its root
    n_before = dev.uploads
    assert dev.weight([[1.0, 2.0], [3.0, 4.0]]) is not dev.weight([[1.0, 2.0], [3.0, 4.0]])   # lists are never cached
    assert dev.uploads == n_before + 2 and all(isinstance(k[0], int) for k in dev._weights)
    # the owner dies: the entry is dropped instead of being served to whoever gets the address next
    key = next(k for k in dev._weights if k[0] == w.__array_interface__["data"][0] and k[1] == (3, 4))
    del w
    gc.collect()
    ref, stale = dev._weights[key]
    assert ref() is None
    dev._prune()
    assert key not in dev._weights and stale.freed
    # a pinned array survives its last outside reference until invalidate()
    p = np.ones((2, 2), np.float32)
    ptr = p.__array_interface__["data"][0]
    dev.register_weight(p)
    tp = dev.weight(p)
    del p
    gc.collect()
    assert any(k[0] == ptr and dev._weights[k][0]() is not None for k in dev._weights)
    dev.invalidate(dev._pinned[ptr])
    assert tp.freed and ptr not in dev._pinned
    with pytest.raises(TypeError):
        dev.register_weight([1.0, 2.0])


def test_invalidate_drops_folded_layernorm_weights():
    """Compute.invalidate(W) forgets the LayerNorm->linear folds built from W (or from its gamma/beta/bias), and the
    fold cache is bounded."""
    from collections import OrderedDict

    from grilly_b200.compute import Compute

    b = object.__new__(Compute)
    b.device = _fake_device()
    b._folds = OrderedDict()
    w1, w2, g = np.ones((4, 4), np.float32), np.ones((4, 4), np.float32), np.ones(4, np.float32)
    b._folds[("lnfold", id(w1), id(g), 0, 0, "layer")] = ("wf", "cs", "bf", w1, g, None, None)
    b._folds[("lnfold", id(w2), id(g), 0, 0, "layer")] = ("wf", "cs", "bf", w2, g, None, None)
    b.invalidate(w1)
    assert len(b._folds) == 1 and next(iter(b._folds.values()))[3] is w2
    b.invalidate(g)              # shared gamma: the remaining fold goes too
    assert not b._folds
    assert Compute.MAX_FOLDS >= 8


def test_clock_sampler_without_nvidia_smi(monkeypatch):
    """The clock sampler only queries nvidia-smi; where the tool is absent it reports that instead of failing, and a
    summary over fabricated rows takes the median SM clock of the samples under load and the active throttle reasons."""
    from grilly_b200.clocks import ClockSampler

    monkeypatch.setenv("PATH", "/nonexistent")
    got = ClockSampler(0).start(wait_s=0.2).stop()
    assert got["samples"] == 0 and got["sm_mhz"] is None
    s = ClockSampler(0)
    s.proc = type("P", (), {"terminate": lambda self: None, "wait": lambda self, timeout=None: 0, "kill": lambda self: None})()
    s.rows = [["0", "1965", "1965", "400.0", "Not Active", "Not Active", "Not Active", "Active"],
              ["0", "1800", "1965", "500.0", "Not Active", "Not Active", "Not Active", "Active"],
              ["0", "210", "1965", "90.0", "Not Active", "Not Active", "Not Active", "Not Active"]]
    out = s.stop()
    assert out["samples"] == 3 and out["sm_mhz"] == 1882.5 and out["sm_max_mhz"] == 1965.0 and out["reasons"] == ["sw_power_cap"]
