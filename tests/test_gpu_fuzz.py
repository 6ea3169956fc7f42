"""Seeded random shapes through the hot-path ops, each against the oracle: row counts around the 128- and 256-row tile
edges, feature counts that are and are not multiples of the tile widths, K with and without a 16-byte row pitch,
ragged sequence lengths, both precisions."""
import numpy as np
import pytest

from conftest import TOL_BF16, TOL_TF32
from oracle import oracle as O

pytestmark = pytest.mark.gpu

ROWS = [1, 2, 31, 32, 33, 127, 128, 129, 255, 256, 257, 300, 511, 513, 1000, 1025, 2049]
FEATS = [1, 8, 31, 64, 96, 100, 128, 192, 200, 256, 384, 512, 640, 1000]
KS = [1, 4, 7, 32, 33, 64, 100, 128, 384, 500]


def _pick(rng, xs):
    return int(xs[int(rng.integers(0, len(xs)))])


@pytest.mark.parametrize("seed", range(12))
def test_linear_family_random_shapes(backend, backend_bf16, seed):
    rng = np.random.default_rng(1000 + seed)
    for _ in range(6):
        M, N, K = _pick(rng, ROWS), _pick(rng, FEATS), _pick(rng, KS)
        x = rng.standard_normal((M, K)).astype(np.float32)
        w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
        b = rng.standard_normal(N).astype(np.float32) if rng.random() < 0.7 else None
        act = ("linear", "fused_linear_gelu", "fused_linear_relu", "fused_linear_silu")[int(rng.integers(0, 4))]
        ref = getattr(O, act)(x, w, b)
        for be, tol in ((backend, TOL_TF32), (backend_bf16, TOL_BF16)):
            got = getattr(be.fnn, act)(x, w, b)
            assert got.shape == (M, N) and np.isfinite(got).all(), (act, M, N, K)
            assert O.rel_l2(got, ref) < tol * (3 if K < 8 else 1), (act, M, N, K, be.precision)
        # C = A B on the same operands
        bmat = rng.standard_normal((K, N)).astype(np.float32)
        assert O.rel_l2(backend.fnn.gemm(x, bmat), x.astype(np.float64) @ bmat.astype(np.float64)) < TOL_TF32 * (3 if K < 8 else 1), (M, K, N)


@pytest.mark.parametrize("seed", range(10))
def test_linear_residual_layernorm_random_shapes(backend, backend_bf16, seed):
    rng = np.random.default_rng(2000 + seed)
    for _ in range(5):
        # now and then enough rows that every CTA pair walks several tiles
        M = _pick(rng, ROWS) if rng.random() < 0.8 else _pick(rng, [19001, 40000, 57000])
        K = _pick(rng, [16, 64, 100, 384, 512])
        N = _pick(rng, [128, 256, 384, 512, 96, 640])          # the last two take the two-launch form
        x = rng.standard_normal((M, K)).astype(np.float32)
        w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
        b = rng.standard_normal(N).astype(np.float32)
        res = (rng.standard_normal((M, N)) + rng.standard_normal()).astype(np.float32) if rng.random() < 0.8 else None
        g, bt = (1 + 0.2 * rng.standard_normal(N)).astype(np.float32), (0.2 * rng.standard_normal(N)).astype(np.float32)
        ref = O.layernorm(O.linear(x, w, b) + (res if res is not None else 0), g, bt, 1e-5)
        for be, tol in ((backend, TOL_TF32), (backend_bf16, TOL_BF16)):
            got = be.fnn.linear_residual_layernorm(x, w, b, res, g, bt, 1e-5)
            assert got.shape == (M, N) and np.isfinite(got).all(), (M, N, K)
            assert O.rel_l2(got, ref) < tol, (M, N, K, be.precision)


@pytest.mark.parametrize("seed", range(10))
def test_attention_random_shapes(backend, backend_bf16, seed):
    rng = np.random.default_rng(3000 + seed)
    for _ in range(4):
        B, H = int(rng.integers(1, 4)), int(rng.integers(1, 5))
        S = _pick(rng, [1, 7, 64, 100, 128, 129, 200, 256, 300, 513])
        D = _pick(rng, [32, 64])
        causal = bool(rng.random() < 0.4)
        q, k, v = (rng.standard_normal((B, S, H, D)).astype(np.float32) for _ in range(3))
        mask = None
        if rng.random() < 0.5:
            lens = rng.integers(1, S + 1, size=B)
            mask = (np.arange(S)[None, :] < lens[:, None]).astype(np.float32)
        ref = O.flash_attention2(q, k, v, mask=mask, causal=causal)
        got = backend.attention.flash_attention2(q, k, v, mask=mask, causal=causal)
        assert O.rel_l2(got, ref) < TOL_TF32, (B, S, H, D, causal, mask is not None)
        if D == 64 or (S <= 128 and not causal):
            got16 = backend_bf16.attention.flash_attention2(q, k, v, mask=mask, causal=causal)
            assert O.rel_l2(got16, ref) < TOL_BF16, (B, S, H, D, causal, mask is not None)
