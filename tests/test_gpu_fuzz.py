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


@pytest.mark.parametrize("seed", range(6))
def test_encoder_random_batches(seed):
    """The resident encoder on random models and batches: 1-3 layers, head dims 32 / 64 / 96 / 128, batches with empty
    and one-token sentences, with and without chunking; against the oracle."""
    import grilly_b200

    rng = np.random.default_rng(4000 + seed)
    heads = _pick(rng, [12, 6, 4, 3])
    layers = int(rng.integers(1, 4))
    ffn = _pick(rng, [384, 768, 1536])
    B, S = int(rng.integers(1, 40)), _pick(rng, [1, 5, 32, 64, 100, 128, 150])
    w = grilly_b200.EncoderWeights.random(rng, num_layers=layers, hidden=384, ffn=ffn, vocab=2000, max_pos=max(S, 8))
    ids = rng.integers(0, 2000, size=(B, S))
    lens = rng.integers(0, S + 1, size=B)
    lens[int(rng.integers(0, B))] = S
    mask = (np.arange(S)[None, :] < lens[:, None]).astype(np.float32)
    ref = O.encoder_forward(ids, mask, w.as_dict(), heads)
    for chunk in (0, 97):
        enc = grilly_b200.SentenceEncoder(w, num_heads=heads, chunk_tokens=chunk)
        try:
            got = enc.encode_ids(ids, mask)
        finally:
            enc.close()
        assert got.shape == (B, 384) and np.isfinite(got).all()
        assert O.rel_l2(got, ref) < TOL_TF32, (heads, layers, ffn, B, S, chunk)
        assert np.array_equal(got[lens == 0], np.zeros((int((lens == 0).sum()), 384), np.float32))


@pytest.mark.parametrize("seed", range(6))
def test_search_random_sizes(backend, seed):
    """faiss.search (distances + top-k without the matrix) against top-k of the oracle's distances."""
    rng = np.random.default_rng(5000 + seed)
    nq, ndb, dim = int(rng.integers(1, 70)), _pick(rng, [1, 10, 257, 1000, 5000, 70001]), _pick(rng, [1, 3, 32, 100, 384])
    k = min(ndb, _pick(rng, [1, 5, 10, 100]))
    kind = ("l2", "cosine", "dot")[int(rng.integers(0, 3))]
    q = rng.standard_normal((nq, dim)).astype(np.float32)
    d = rng.standard_normal((ndb, dim)).astype(np.float32)
    idx, val = backend.faiss.search(q, d, k, kind)
    ridx, rval = O.faiss_topk(O.faiss_distances(q, d, kind), k)
    assert idx.shape == (nq, k) and val.shape == (nq, k)
    np.testing.assert_allclose(val, rval, rtol=2e-4, atol=3e-5)
    # indices agree wherever the oracle's neighbouring distances are further apart than fp32 noise
    dist = O.faiss_distances(q, d, kind)
    for r in range(nq):
        srt = np.sort(dist[r])[: k + 1]
        gaps = np.diff(srt) if srt.size > 1 else np.array([1.0])
        if gaps.size and gaps.min() > 1e-4 * max(1.0, float(np.abs(srt).max())):
            assert np.array_equal(idx[r], ridx[r]), (nq, ndb, dim, k, kind, r)


@pytest.mark.parametrize("seed", range(4))
def test_encoder_bf16_and_modernbert_random_batches(seed):
    """The bf16 mode of the post-LN encoder and the pre-norm (ModernBERT) architecture on random batches."""
    import grilly_b200

    rng = np.random.default_rng(6000 + seed)
    heads = _pick(rng, [12, 6])
    B, S = int(rng.integers(1, 30)), _pick(rng, [7, 48, 100, 128])
    ids = rng.integers(0, 2000, size=(B, S))
    lens = rng.integers(1, S + 1, size=B)
    mask = (np.arange(S)[None, :] < lens[:, None]).astype(np.float32)
    w = grilly_b200.EncoderWeights.random(rng, num_layers=2, hidden=384, ffn=768, vocab=2000, max_pos=128)
    enc = grilly_b200.SentenceEncoder(w, num_heads=heads, precision="bf16")
    try:
        got = enc.encode_ids(ids, mask)
    finally:
        enc.close()
    assert O.rel_l2(got, O.encoder_forward(ids, mask, w.as_dict(), heads)) < TOL_BF16, (heads, B, S)
    wm = grilly_b200.EncoderWeights.random_modernbert(rng, num_layers=2, hidden=384, ffn=576, vocab=2000)
    encm = grilly_b200.SentenceEncoder(wm, num_heads=heads, arch="modernbert", rope_base=10000.0)
    try:
        gotm = encm.encode_ids(ids, mask)
    finally:
        encm.close()
    assert O.rel_l2(gotm, O.modernbert_forward(ids, mask, wm.as_dict(), heads)) < TOL_TF32, (heads, B, S)
