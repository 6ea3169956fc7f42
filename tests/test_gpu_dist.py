"""Two-GPU run of the sharded paths (skipped on a single-GPU box): the column-split GEMM (with an NCCL all-gather, and with the
exchange fused into the epilogue) and the batch-sharded encoder must reproduce the one-GPU results bit for bit. Ranks are child processes; NVLS is off."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"   # plain peer mappings only
    import torch
    import torch.distributed as dist

    import grilly_b200
    from grilly_b200.dist import FusedNsplit, encode_sharded, gemm_nsplit, gemm_nsplit_fused

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    backend = grilly_b200.Compute(device=rank)
    try:
        rng = np.random.default_rng(11)
        A = rng.standard_normal((1000, 512)).astype(np.float32)
        B = rng.standard_normal((512, 1024)).astype(np.float32)
        C = gemm_nsplit(A, B, backend=backend, slabs=3)
        Cf = gemm_nsplit_fused(A, B, backend)          # exchange inside the GEMM epilogue (stores to the peer's C)
        op = FusedNsplit(backend, 1000, 1024, 512)
        op.prepare(A, B[:, rank * 512:(rank + 1) * 512])
        Cc = op.run_copy(slabs=3).cpu().numpy()        # exchange by strided peer copies per row slab
        backend.device.set_stream(None)
        single = backend.fnn.gemm(A, B)
        ref = A.astype(np.float64) @ B.astype(np.float64)
        rel = float(np.linalg.norm(C - ref) / np.linalg.norm(ref))
        w = grilly_b200.EncoderWeights.random(np.random.default_rng(2), num_layers=2, vocab=3000, max_pos=64)
        enc = grilly_b200.SentenceEncoder(w, num_heads=12, device=backend.device)
        ids = rng.integers(0, 3000, size=(37, 48))
        lens = rng.integers(1, 49, size=37)
        mask = (np.arange(48)[None, :] < lens[:, None]).astype(np.float32)
        sharded = encode_sharded(enc, ids, mask)
        whole = enc.encode_ids(ids, mask)
        enc.close()
        q.put((rank, bool(np.array_equal(C, single)) and bool(np.array_equal(Cf, single)) and bool(np.array_equal(Cc, single)), rel < 2e-3,
               bool(np.array_equal(sharded, whole))))
    finally:
        backend.cleanup()
        dist.destroy_process_group()


def test_two_gpu_nsplit_gemm_and_sharded_encoder(lib):
    import ctypes as C

    n = C.c_int(0)
    lib.grilly_device_count(C.byref(n))
    if n.value < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    assert sorted(q.get(timeout=10) for _ in range(2)) == [(0, True, True, True), (1, True, True, True)]
