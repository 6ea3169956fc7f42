"""Host-side logic of the multi-GPU paths on CPU ranks (gloo, world size 2 and 3): batch sharding and the
column-split GEMM's partitioning, slab-wise all-gather and re-assembly. The local multiply is replaced by a NumPy
stand-in defined here; the CUDA path of the same functions is covered by tests/test_gpu_dist.py on 2 GPUs."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_shard_range_covers_everything():
    from grilly_b200.dist import shard_by_tokens, shard_range

    for n in (0, 1, 7, 1024, 1025):
        for world in (1, 2, 3, 8):
            spans = [shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)
    rng = np.random.default_rng(0)
    lens = rng.integers(16, 129, size=1024)
    parts = shard_by_tokens(lens, 8)
    assert sorted(np.concatenate(parts).tolist()) == list(range(1024))
    loads = [int(lens[p].sum()) for p in parts]
    assert max(loads) - min(loads) <= 128


class NumpyLocalGemm:
    """CPU stand-in for the per-rank multiply (test only)."""

    def prepare(self, A, B_cols):
        import torch

        self.torch = torch
        self.a, self.b = np.asarray(A, np.float64), np.asarray(B_cols, np.float64)

    def run_slab(self, r0, r1, out):
        out.copy_(self.torch.from_numpy((self.a[r0:r1] @ self.b).astype(np.float32)))

    def empty(self, *shape):
        return self.torch.empty(shape, dtype=self.torch.float32)

    def to_numpy(self, t):
        return t.numpy()


class FakeEncoder:
    hidden = 4

    def encode_ids(self, ids, mask=None):
        ids = np.asarray(ids, np.float32)
        m = np.ones_like(ids) if mask is None else mask
        return np.stack([ids.sum(1), (ids * m).sum(1), m.sum(1), ids[:, 0]], 1).astype(np.float32)


def _worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist

    from grilly_b200.dist import encode_sharded, gemm_nsplit

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(7)
        A = rng.standard_normal((37, 20)).astype(np.float32)
        B = rng.standard_normal((20, 24 * world)).astype(np.float32)
        C = gemm_nsplit(A, B, local=NumpyLocalGemm(), slabs=3)
        ok_gemm = np.allclose(C, A.astype(np.float64) @ B, atol=1e-5)
        C1 = gemm_nsplit(A[:1], B, local=NumpyLocalGemm(), slabs=4)  # fewer rows than slabs
        ok_gemm = ok_gemm and np.allclose(C1, A[:1].astype(np.float64) @ B, atol=1e-5)
        try:
            gemm_nsplit(A, B[:, :5], local=NumpyLocalGemm())
            ok_err = False
        except ValueError:
            ok_err = True
        ids = rng.integers(0, 100, size=(11, 6))
        mask = (rng.random((11, 6)) > 0.3).astype(np.float32)
        out = encode_sharded(FakeEncoder(), ids, mask)
        ok_enc = np.array_equal(out, FakeEncoder().encode_ids(ids, mask))
        q.put((rank, bool(ok_gemm), ok_err, bool(ok_enc)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_nsplit_gemm_and_sharded_encode_over_gloo(world):
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    results = sorted(q.get(timeout=10) for _ in range(world))
    assert results == [(r, True, True, True) for r in range(world)]
