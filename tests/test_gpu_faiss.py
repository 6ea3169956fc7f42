"""Vector search through the C ABI: pairwise distances (tensor-core GEMM over tf32 hi/lo splits) and exact top-k.
The reference checks its own GPU result against closed forms at rtol 1e-4 (tests/test_gpu_operations.py:219-283);
the same checks run here, plus the oracle and the stored outputs of the reference's CPU top-k."""
from pathlib import Path

import numpy as np
import pytest

import cases
from oracle import oracle as O

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("kind", ["l2", "cosine", "dot"])
def test_distances_against_oracle(backend, kind):
    c = cases.faiss_search()
    q, d = c["queries"], c["database"]
    got = backend.faiss_compute_distances(q, d, distance_type=kind)
    ref = O.faiss_distances(q, d, kind)
    assert got.shape == (10, 1000) and got.dtype == np.float32
    # fp32-level accuracy, far inside the tf32 tolerance of 2e-3: the split operands carry 21 mantissa bits
    assert O.rel_l2(got, ref) < 5e-6
    np.testing.assert_allclose(got, ref, rtol=1e-4, atol=2e-5)
    if kind == "l2":
        assert np.all(got >= 0)
        np.testing.assert_allclose(got[0], np.sqrt(np.sum((q[0:1] - d) ** 2, axis=1)), rtol=1e-4)
    # nearest neighbours are the same ones, in the same order
    assert np.array_equal(np.argsort(got, axis=1, kind="stable")[:, :10], np.argsort(ref, axis=1, kind="stable")[:, :10])


@pytest.mark.parametrize("nq,ndb,dim", [(1, 1, 1), (5, 100, 128), (3, 50, 64), (130, 1027, 30), (2048, 4096, 384)])
def test_distance_shapes(backend, nq, ndb, dim):
    rng = np.random.default_rng(nq + ndb + dim)
    q = rng.standard_normal((nq, dim)).astype(np.float32)
    d = rng.standard_normal((ndb, dim)).astype(np.float32)
    for kind in ("l2", "cosine"):
        got = backend.faiss.compute_distances(q, d, kind)
        assert got.shape == (nq, ndb)
        np.testing.assert_allclose(got, O.faiss_distances(q, d, kind), rtol=1e-4, atol=5e-5)
    one = backend.faiss.compute_distances(q[0], d, "dot")          # 1-D query
    assert one.shape == (1, ndb)
    with pytest.raises(ValueError):
        backend.faiss.compute_distances(q, d[:, :-1] if dim > 1 else np.zeros((ndb, 2), np.float32))


def test_identical_vectors_and_unknown_type(backend):
    rng = np.random.default_rng(3)
    d = rng.standard_normal((64, 96)).astype(np.float32)
    l2 = backend.faiss.compute_distances(d, d, "l2")
    # the expanded form |q|^2 + |d|^2 - 2 q.d loses the exact zero of (x - x): an error of a few 1e-6 |x|^2 under the
    # square root leaves up to about 2e-3 |x| (the reference's loop over (q - d)^2 gives exactly 0 here)
    assert np.all(np.diag(l2) < 3e-3 * np.linalg.norm(d, axis=1))
    cos = backend.faiss.compute_distances(d, d, "cosine")
    assert np.all(np.abs(np.diag(cos)) < 1e-5)
    assert np.array_equal(backend.faiss.compute_distances(d[:4], d, "something-else"), cos[:4])


def test_topk_against_reference_outputs(backend):
    ref = dict(np.load(ROOT / "tests" / "golden" / "extras_golden.npz"))
    c = cases.faiss_search()
    idx, val = backend.faiss_topk(c["dist"], c["k"])
    assert idx.shape == (10, 20) and idx.dtype == np.uint32 and val.dtype == np.float32
    assert np.array_equal(val, ref["topk_val"])                      # bit-exact: values are selected, not computed
    o_idx, o_val = O.faiss_topk(c["dist"], c["k"])
    assert np.array_equal(idx, o_idx) and np.array_equal(val, o_val)  # ties by ascending index, like the oracle
    assert np.array_equal(idx[3], np.arange(100, 120, dtype=np.uint32))


@pytest.mark.parametrize("nq,ndb,k", [(1, 1, 1), (10, 1000, 20), (7, 257, 257), (3, 5000, 1024), (64, 100000, 10), (2, 33, 500),
                                       (4, 300000, 50), (1, 1000000, 1024)])
def test_topk_sizes(backend, nq, ndb, k):
    rng = np.random.default_rng(ndb + k)
    dist = rng.standard_normal((nq, ndb)).astype(np.float32)
    dist[0, : min(ndb, 9)] = -np.inf                                # infinities and signed zeros order like floats
    dist[-1, ndb // 2] = np.float32(-0.0)
    if ndb >= 100000:
        dist[-1, ::1000] = -10.0                                     # equal minima spread over the segments of a long row
    idx, val = backend.faiss.topk(dist, k)
    o_idx, o_val = O.faiss_topk(dist, k)
    assert idx.shape == (nq, min(k, ndb))
    assert np.array_equal(val, o_val)
    assert np.array_equal(idx, o_idx)
    # the reference's own check: sorted selected values equal the head of the sorted row
    for r in range(nq):
        np.testing.assert_allclose(np.sort(val[r]), np.sort(dist[r])[: min(k, ndb)], rtol=1e-4)


def test_end_to_end_search_on_device(backend):
    """Distances stay on the device between the two calls; indices point at the distances they were taken from."""
    np.random.seed(42)
    queries = np.random.randn(10, 256).astype(np.float32)
    database = np.random.randn(1000, 256).astype(np.float32)
    dd = backend.faiss.compute_distances(backend.to_device(queries, mma_operand=False), database, "cosine")
    idx, val = backend.faiss.topk(dd, 10)
    dist = dd.numpy()
    for i in range(10):
        assert np.array_equal(val[i], dist[i, idx[i]])
    ref_idx, _ = O.faiss_topk(O.faiss_distances(queries, database, "cosine"), 10)
    assert np.array_equal(idx, ref_idx)
    with pytest.raises(Exception):
        backend.faiss.topk(np.zeros((1, 3000), np.float32), 2000)    # k above 1024 is rejected, not truncated


@pytest.mark.parametrize("nq,ndb,dim,k", [(10, 1000, 256, 20), (8192, 5000, 64, 10), (3, 200000, 32, 100), (1, 7, 5, 7), (600, 2500, 384, 1)])
@pytest.mark.parametrize("kind", ["cosine", "l2"])
def test_search_equals_distances_then_topk(backend, nq, ndb, dim, k, kind):
    """faiss.search never writes the (nq, ndb) matrix (the database is walked in chunks that are reduced to their k
    best at once); values, indices and the order of ties are those of compute_distances followed by topk."""
    rng = np.random.default_rng(nq + ndb)
    q = rng.standard_normal((nq, dim)).astype(np.float32)
    d = rng.standard_normal((ndb, dim)).astype(np.float32)
    if ndb >= 100:
        d[ndb // 2] = d[3]              # exact duplicates in different chunks: equal distances, the lower index first
        d[ndb - 1] = d[3]
    idx, val = backend.faiss.search(q, d, k, kind)
    full = backend.faiss.compute_distances(q, d, kind)
    idx2, val2 = backend.faiss.topk(full, k)
    assert idx.dtype == np.uint32 and idx.shape == (nq, k) and val.shape == (nq, k)
    assert np.array_equal(val, val2)
    assert np.array_equal(idx, idx2)
    ref_idx, ref_val = O.faiss_topk(O.faiss_distances(q[:64], d, kind), k)
    np.testing.assert_allclose(val[:64], ref_val, rtol=1e-4, atol=5e-5)


def test_search_flat_alias_and_errors(backend):
    c = cases.faiss_search()
    idx, val = backend.faiss_search(c["queries"], c["database"], 5, "dot")
    want = np.argsort(O.faiss_distances(c["queries"], c["database"], "dot"), axis=1, kind="stable")[:, :5]
    assert np.array_equal(idx, want.astype(np.uint32))
    with pytest.raises(ValueError):
        backend.faiss.search(c["queries"], c["database"][:, :-1], 5)
    with pytest.raises(ValueError):
        backend.faiss.search(c["queries"], c["database"], 0)
