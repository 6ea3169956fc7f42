"""grilly_layernorm_linear_noalloc: the entry point for callers that may not allocate device memory (its
row-statistics scratch lives in a fixed array inside the library). Collected last on purpose, so that a run that
stops at the first failure has already exercised every other test. Works alone in a fresh process too: it builds
its own context and inputs."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run(dev, lib, L, entry, x, g, bt, w, b, mode, with_scratch):
    M, K = x.shape
    N = w.shape[0]
    xd = dev.upload(x)
    wd, gd, bd, cd = dev.upload(w), dev.upload(g), dev.upload(bt), dev.upload(b)
    wf, cs, bf = dev.empty((N, K)), dev.empty((N,)), dev.empty((N,))
    dev.check(lib.grilly_fold_layernorm_weights(dev.ctx, wd.ptr, gd.ptr, bd.ptr if mode == L.NORM_LAYER else None, cd.ptr,
                                                wf.ptr, cs.ptr, bf.ptr, N, K, L.PREC_TF32))
    y = dev.empty((M, N))
    if with_scratch:
        stats = dev.empty((2 * M,))
        dev.check(entry(dev.ctx, xd.ptr, wf.ptr, cs.ptr, bf.ptr, y.ptr, stats.ptr, M, N, K, 1e-5, mode, L.ACT_NONE, L.PREC_TF32, 0))
    else:
        dev.check(entry(dev.ctx, xd.ptr, wf.ptr, cs.ptr, bf.ptr, y.ptr, M, N, K, 1e-5, mode, L.ACT_NONE, L.PREC_TF32, 0))
    return y.numpy()


def test_noalloc_matches_the_allocating_entry_point_twice_in_a_row(lib):
    from grilly_b200 import _lib as L
    from grilly_b200.device import Device

    dev = Device(0)
    try:
        rng = np.random.default_rng(123)
        # the second call is smaller and uses the other norm: stale statistics of the first call stay in the
        # shared array beyond its rows and must not leak into the result
        cases = [(1000, 512, 384, L.NORM_LAYER), (300, 256, 384, L.NORM_RMS)]
        for M, N, K, mode in cases:
            x = (rng.standard_normal((M, K)) * 2 + 0.5).astype(np.float32)
            g = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32)
            bt = (0.1 * rng.standard_normal(K)).astype(np.float32)
            w = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
            b = rng.standard_normal(N).astype(np.float32)
            ref = _run(dev, lib, L, lib.grilly_layernorm_linear, x, g, bt, w, b, mode, True)
            out = _run(dev, lib, L, lib.grilly_layernorm_linear_noalloc, x, g, bt, w, b, mode, False)
            assert np.isfinite(out).all()
            # same kernels on the same inputs: the tests' tf32 tolerance is 2e-3 rel-L2, these agree to the bit
            err = np.linalg.norm(out.astype(np.float64) - ref) / np.linalg.norm(ref.astype(np.float64))
            assert err < 2e-3, err
            assert np.array_equal(out, ref)
    finally:
        dev.close()


def test_noalloc_at_its_row_limit_and_without_touching_the_pool(lib):
    """M == GRILLY_NOALLOC_MAX_ROWS uses the last element of the mean half and the whole rstd half of the one array;
    and a warmed-up call neither allocates from nor returns anything to the context's pool."""
    from grilly_b200 import _lib as L
    from grilly_b200.device import Device

    dev = Device(0)
    try:
        rng = np.random.default_rng(7)
        M, N, K = 65536, 64, 32
        x = (rng.standard_normal((M, K)) + 0.3).astype(np.float32)
        g = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32)
        bt = (0.1 * rng.standard_normal(K)).astype(np.float32)
        w = (rng.standard_normal((N, K)) * 0.2).astype(np.float32)
        b = rng.standard_normal(N).astype(np.float32)
        ref = _run(dev, lib, L, lib.grilly_layernorm_linear, x, g, bt, w, b, L.NORM_LAYER, True)
        out = _run(dev, lib, L, lib.grilly_layernorm_linear_noalloc, x, g, bt, w, b, L.NORM_LAYER, False)
        assert np.array_equal(out, ref)
        # same shapes again with every buffer made beforehand: the pool counters must not move across the call
        xd, y = dev.upload(x), dev.empty((M, N))
        wd, gd, bd, cd = dev.upload(w), dev.upload(g), dev.upload(bt), dev.upload(b)
        wf, cs, bf = dev.empty((N, K)), dev.empty((N,)), dev.empty((N,))
        dev.check(lib.grilly_fold_layernorm_weights(dev.ctx, wd.ptr, gd.ptr, bd.ptr, cd.ptr, wf.ptr, cs.ptr, bf.ptr, N, K, L.PREC_TF32))
        dev.sync()
        before = dev.pool_stats()
        dev.check(lib.grilly_layernorm_linear_noalloc(dev.ctx, xd.ptr, wf.ptr, cs.ptr, bf.ptr, y.ptr, M, N, K, 1e-5, L.NORM_LAYER,
                                                      L.ACT_NONE, L.PREC_TF32, 0))
        dev.sync()
        after = dev.pool_stats()
        for key in ("acquired", "released", "bytes_in_use", "pool_reserved_bytes"):
            assert after[key] == before[key], key
        assert np.array_equal(y.numpy(), ref)
    finally:
        dev.close()


def test_noalloc_refuses_rows_outside_the_folded_forms_envelope(lib):
    """Row means many standard deviations from zero need the normalise-first form, which needs scratch this entry
    point does not have: it says so instead of returning an inaccurate result; the allocating entry handles them."""
    from grilly_b200 import _lib as L
    from grilly_b200.device import Device

    dev = Device(0)
    try:
        rng = np.random.default_rng(8)
        M, N, K = 256, 64, 128
        x = (rng.standard_normal((M, K)) + 20.0).astype(np.float32)
        g, bt = np.ones(K, np.float32), np.zeros(K, np.float32)
        w, b = (rng.standard_normal((N, K)) * 0.1).astype(np.float32), np.zeros(N, np.float32)
        xd, y = dev.upload(x), dev.empty((M, N))
        wd, gd, bd, cd = dev.upload(w), dev.upload(g), dev.upload(bt), dev.upload(b)
        wf, cs, bf = dev.empty((N, K)), dev.empty((N,)), dev.empty((N,))
        dev.check(lib.grilly_fold_layernorm_weights(dev.ctx, wd.ptr, gd.ptr, bd.ptr, cd.ptr, wf.ptr, cs.ptr, bf.ptr, N, K, L.PREC_TF32))
        rc = lib.grilly_layernorm_linear_noalloc(dev.ctx, xd.ptr, wf.ptr, cs.ptr, bf.ptr, y.ptr, M, N, K, 1e-5, L.NORM_LAYER,
                                                 L.ACT_NONE, L.PREC_TF32, 0)
        assert rc == L.ERR_UNSUPPORTED and b"accuracy envelope" in lib.grilly_last_error(dev.ctx)
        # RMS mode has no mean term and is accepted for the same rows
        dev.check(lib.grilly_layernorm_linear_noalloc(dev.ctx, xd.ptr, wf.ptr, None, bf.ptr, y.ptr, M, N, K, 1e-5, L.NORM_RMS,
                                                      L.ACT_NONE, L.PREC_TF32, 0))
        dev.sync()
    finally:
        dev.close()


def test_noalloc_rejects_sizes_beyond_its_scratch(lib):
    from grilly_b200 import _lib as L
    from grilly_b200.device import Device

    dev = Device(0)
    try:
        dummy = dev.empty((16,))
        rc = lib.grilly_layernorm_linear_noalloc(dev.ctx, dummy.ptr, dummy.ptr, dummy.ptr, dummy.ptr, dummy.ptr, 65537, 8, 8,
                                                 1e-5, L.NORM_LAYER, L.ACT_NONE, L.PREC_TF32, 0)
        assert rc == L.ERR_INVALID_ARG
        assert b"exceed the built-in scratch" in lib.grilly_last_error(dev.ctx)
        # an unknown precision is an invalid argument here as in the allocating entry point; bf16 is unsupported
        rc = lib.grilly_layernorm_linear_noalloc(dev.ctx, dummy.ptr, dummy.ptr, dummy.ptr, dummy.ptr, dummy.ptr, 8, 8, 8,
                                                 1e-5, L.NORM_LAYER, L.ACT_NONE, 7, 0)
        assert rc == L.ERR_INVALID_ARG
        rc = lib.grilly_layernorm_linear_noalloc(dev.ctx, dummy.ptr, dummy.ptr, dummy.ptr, dummy.ptr, dummy.ptr, 8, 8, 8,
                                                 1e-5, L.NORM_LAYER, L.ACT_NONE, L.PREC_BF16, 0)
        assert rc == L.ERR_UNSUPPORTED
    finally:
        dev.close()
