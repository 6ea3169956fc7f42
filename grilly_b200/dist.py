"""Multi-GPU use of the hot path: one process per GPU, ``torch.distributed`` for the plumbing.

The reference has no multi-GPU code (CHANGELOG.md:75 "Multi-GPU support not yet implemented"); this module adds the
two partitionings the path admits:

* sentences are independent, so the encoder shards its batch across ranks with no data-path collective
  (:func:`shard_range`, :func:`encode_sharded`);
* one large ``gemm`` (backend/fnn.py:104-166) is split by columns of B: rank r multiplies A by its column block and
  the blocks of C are exchanged with one all-gather per slab of rows (:func:`gemm_nsplit`). The all-gather of a slab
  runs on NCCL's stream while the next slab's GEMM runs on the compute stream;
* the same split with the exchange inside the GEMM kernel (:func:`gemm_nsplit_fused`): C lives in symmetric memory,
  every rank's epilogue stores its column block straight into every rank's C (plain stores to peer-mapped memory,
  tile by tile under the main loop), and one barrier ends the step. No staging buffer, no un-permute pass.

The collective layer is injected (``group``, any initialised ``torch.distributed`` backend) and so is the local
multiply, which lets the partitioning and re-assembly logic be tested on CPU ranks over gloo; the default local
multiply is the CUDA library and raises without a GPU.
"""
from __future__ import annotations

import numpy as np


def shard_range(n: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous, balanced [lo, hi) share of n items for ``rank`` (the first n % world ranks get one more)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank must be in [0, world)")
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_by_tokens(lengths, world: int) -> list[np.ndarray]:
    """Indices of the sentences each rank should take so that every rank gets about the same number of valid tokens
    (longest-first greedy); the order inside a rank is the original order."""
    lengths = np.asarray(lengths)
    loads = np.zeros(world, dtype=np.int64)
    buckets: list[list[int]] = [[] for _ in range(world)]
    for i in np.argsort(-lengths, kind="stable"):
        r = int(np.argmin(loads))
        buckets[r].append(int(i))
        loads[r] += int(lengths[i])
    return [np.array(sorted(b), dtype=np.int64) for b in buckets]


def _dist():
    import torch.distributed as dist

    if not dist.is_initialized():
        raise RuntimeError("torch.distributed is not initialised (launch with torch.distributed.run)")
    return dist


def encode_sharded(encoder, input_ids, attention_mask=None, group=None, gather: bool = True):
    """Each rank encodes its contiguous share of the batch; with ``gather`` every rank gets all embeddings back
    (the only communication, outside the model)."""
    import torch

    dist = _dist()
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    ids = np.asarray(input_ids)
    lo, hi = shard_range(ids.shape[0], rank, world)
    mask = None if attention_mask is None else np.asarray(attention_mask)[lo:hi]
    local = encoder.encode_ids(ids[lo:hi], mask) if hi > lo else np.zeros((0, encoder.hidden), np.float32)
    if not gather:
        return local
    parts = [None] * world
    dist.all_gather_object(parts, local, group=group)
    return np.concatenate(parts, axis=0) if parts else torch.empty(0).numpy()


class _StreamBridge:
    """Runs the library's launches on a torch stream of their own, ordered inside torch's current stream: the
    launches wait for what the current stream has queued, and the current stream (hence NCCL and torch ops issued
    after them) waits for the launches. Torch's default stream has the handle 0, which the library reads as "use
    your own stream", so the current stream itself cannot be handed over."""

    def __init__(self, dev, torch, device):
        self.torch, self.device = torch, device
        self.stream = torch.cuda.Stream(device=device)
        dev.set_stream(self.stream.cuda_stream)

    def __enter__(self):
        self.stream.wait_stream(self.torch.cuda.current_stream(self.device))
        return self

    def __exit__(self, *exc):
        self.torch.cuda.current_stream(self.device).wait_stream(self.stream)


class CudaLocalGemm:
    """Local multiply through libgrilly_b200.so on torch-owned CUDA buffers (A and the column block of B are
    uploaded once and kept; C is written into a torch tensor so NCCL can send it without a copy)."""

    def __init__(self, backend):
        import torch

        self.torch = torch
        self.backend = backend
        self.dev = backend.device
        self.device = torch.device("cuda", self.dev.index)
        self.bridge = _StreamBridge(self.dev, torch, self.device)   # torch and NCCL see the library's work in order

    def prepare(self, A: np.ndarray, B_cols: np.ndarray):
        bf16 = self.backend.precision == "bf16"
        self.a = self.backend.to_device(np.ascontiguousarray(A, dtype=np.float32))
        self.b = self.backend.to_device(np.ascontiguousarray(B_cols, dtype=np.float32))
        self.M, self.K = A.shape
        self.n_loc = B_cols.shape[1]
        self.elt = 2 if bf16 else 4
        self.prec = 1 if bf16 else 0

    def run_slab(self, r0: int, r1: int, out):
        """out[(r1-r0), n_loc] (torch, fp32, contiguous) = A[r0:r1] @ B_cols."""
        import ctypes as C

        with self.bridge:
            rc = self.dev.lib.grilly_gemm_mnk(self.dev.ctx, C.c_void_p(self.a.ptr + r0 * self.K * self.elt), C.c_void_p(self.b.ptr),
                                              C.c_void_p(out.data_ptr()), r1 - r0, self.K, self.n_loc, self.prec, 0)
        self.dev.check(rc)

    def empty(self, *shape):
        return self.torch.empty(shape, dtype=self.torch.float32, device=self.device)

    def to_numpy(self, t):
        return t.cpu().numpy()


def gemm_nsplit(A, B, local=None, backend=None, group=None, slabs: int = 4, return_tensor: bool = False,
                prepared: bool = False):
    """C = A @ B with B split by columns across the ranks of ``group`` and one all-gather per row slab.

    A (M, K) and B (K, N) are the full host matrices on every rank (rank r reads only its column block of B).
    N must be divisible by the world size times 4 (16-byte rows for the device kernel). Returns the full C (M, N)
    on every rank. With ``prepared`` the operands already sit in ``local`` (repeated timing runs).
    """
    dist = _dist()
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    A, B = np.asarray(A), np.asarray(B)
    if A.ndim != 2 or B.ndim != 2 or A.shape[1] != B.shape[0]:
        raise AssertionError(f"K mismatch: {A.shape} @ {B.shape}")
    M, N = A.shape[0], B.shape[1]
    if N % (world * 4):
        raise ValueError(f"N = {N} must be a multiple of 4 x world size ({world}) for the column split")
    if local is None:
        if backend is None:
            raise ValueError("give a Compute() backend (or a local multiply for CPU tests)")
        local = CudaLocalGemm(backend)
    n_loc = N // world
    if not prepared:
        local.prepare(A, B[:, rank * n_loc:(rank + 1) * n_loc])
    slabs = max(1, min(slabs, M))
    bounds = [shard_range(M, s, slabs) for s in range(slabs)]
    out = local.empty(M, N)
    out3 = out.view(M, world, n_loc)
    works = []
    for r0, r1 in bounds:
        mine = local.empty(r1 - r0, n_loc)
        local.run_slab(r0, r1, mine)
        staged = local.empty(world * (r1 - r0), n_loc)       # block of rank q lands at rows [q*rows, (q+1)*rows)
        w = dist.all_gather_into_tensor(staged, mine, group=group, async_op=True)
        works.append((w, staged, mine, r0, r1))
    for w, staged, _mine, r0, r1 in works:
        w.wait()
        out3[r0:r1].copy_(staged.view(world, r1 - r0, n_loc).permute(1, 0, 2))   # (g, rows, N/g) -> rows x N
    return out if return_tensor else local.to_numpy(out)


class FusedNsplit:
    """C = A @ B with B split by columns and every rank's epilogue writing its block into all ranks' C.

    Set-up (once per shape): a symmetric (M, N) fp32 buffer and the peers' addresses of it. ``run()`` is then one
    kernel launch per rank plus a barrier. Operands are uploaded by ``prepare``; A is replicated, rank r keeps
    columns [r N/g, (r+1) N/g) of B.
    """

    def __init__(self, backend, M: int, N: int, K: int, group=None):
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # peer mappings are all the kernel needs
        import torch
        import torch.distributed._symmetric_memory as symm_mem

        dist = _dist()
        self.torch, self.dist, self.group = torch, dist, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks (one destination per rank in the kernel's list)")
        if N % (self.world * 32):
            raise ValueError(f"N = {N} must be a multiple of 32 x world size ({self.world})")
        self.backend, self.dev = backend, backend.device
        self.M, self.N, self.K, self.n_loc = M, N, K, N // self.world
        self.device = torch.device("cuda", self.dev.index)
        self.bridge = _StreamBridge(self.dev, torch, self.device)
        self.c = symm_mem.empty((M, N), dtype=torch.float32, device=self.device)
        self.handle = symm_mem.rendezvous(self.c, group if group is not None else dist.group.WORLD)
        # destination i = C of rank (rank + i) % world at this rank's column offset; the own copy first
        col_bytes = self.rank * self.n_loc * 4
        order = [(self.rank + i) % self.world for i in range(self.world)]
        import ctypes as C
        self._ptrs = (C.c_void_p * self.world)(*[int(self.handle.buffer_ptrs[r]) + col_bytes for r in order])

    def prepare(self, A: np.ndarray, B_cols: np.ndarray):
        bf16 = self.backend.precision == "bf16"
        self.a = self.backend.to_device(np.ascontiguousarray(A, dtype=np.float32))
        self.b = self.backend.to_device(np.ascontiguousarray(B_cols, dtype=np.float32))
        self.prec = 1 if bf16 else 0

    def run_copy(self, slabs: int = 4):
        """Same result with the exchange done by strided peer-to-peer copies instead of epilogue stores: the GEMM of
        a row slab writes this rank's column block into its own C, then one copy per peer (on a side stream, rows of
        N/g contiguous floats) puts the slab into the peer's C while the next slab's GEMM runs."""
        import ctypes as C

        torch = self.torch
        if not hasattr(self, "_side"):
            self._side = torch.cuda.Stream(device=self.device)
            # base addresses of the peers' C: peer memory is only ever a destination of copy-engine copies here
            self._peer_ptrs = {r: int(self.handle.buffer_ptrs[r]) for r in range(self.world) if r != self.rank}
        self.handle.barrier()
        cur = torch.cuda.current_stream(self.device)
        c0, c1 = self.rank * self.n_loc, (self.rank + 1) * self.n_loc
        elt = 2 if self.prec else 4
        for s in range(slabs):
            r0, r1 = shard_range(self.M, s, slabs)
            with self.bridge:
                out = self.c.data_ptr() + (r0 * self.N + c0) * 4
                ptr = (C.c_void_p * 1)(out)
                rc = self.dev.lib.grilly_gemm_mnk_multi(self.dev.ctx, C.c_void_p(self.a.ptr + r0 * self.K * elt), C.c_void_p(self.b.ptr),
                                                        ptr, 1, r1 - r0, self.K, self.n_loc, C.c_longlong(self.N), self.prec)
            self.dev.check(rc)
            self._side.wait_stream(cur)
            off = (r0 * self.N + c0) * 4
            self.dev.set_stream(self._side.cuda_stream)
            try:
                for base in self._peer_ptrs.values():
                    self.dev.check(self.dev.lib.grilly_copy_2d(self.dev.ctx, C.c_void_p(base + off), self.N * 4,
                                                               C.c_void_p(self.c.data_ptr() + off), self.N * 4,
                                                               self.n_loc * 4, r1 - r0))
            finally:
                self.dev.set_stream(self.bridge.stream.cuda_stream)
        cur.wait_stream(self._side)
        self.handle.barrier()
        return self.c

    def run(self):
        """One step: every rank's C holds the full product when this returns (device-side: after the barrier)."""
        import ctypes as C

        self.handle.barrier()        # nobody still reads the C of the previous step
        with self.bridge:
            rc = self.dev.lib.grilly_gemm_mnk_multi(self.dev.ctx, C.c_void_p(self.a.ptr), C.c_void_p(self.b.ptr), self._ptrs,
                                                    self.world, self.M, self.K, self.n_loc, C.c_longlong(self.N), self.prec)
        self.dev.check(rc)
        self.handle.barrier()        # all ranks' stores have landed before anyone reads C
        return self.c


def gemm_nsplit_fused(A, B, backend, group=None, return_tensor: bool = False, exchange: str = "stores"):
    """C = A @ B, column-split over symmetric memory (see :class:`FusedNsplit`): ``exchange="stores"`` writes every
    tile to all ranks from the GEMM epilogue (whole 128-byte lines), ``"copies"`` moves row slabs with strided peer
    copies under the next slab's GEMM. On two GPUs the first is ahead at 8192^3, the second slightly at 16384^3."""
    A, B = np.asarray(A), np.asarray(B)
    if A.ndim != 2 or B.ndim != 2 or A.shape[1] != B.shape[0]:
        raise AssertionError(f"K mismatch: {A.shape} @ {B.shape}")
    op = FusedNsplit(backend, A.shape[0], B.shape[1], A.shape[1], group)
    op.prepare(A, B[:, op.rank * op.n_loc:(op.rank + 1) * op.n_loc])
    c = op.run_copy() if exchange == "copies" else op.run()
    return c if return_tensor else c.cpu().numpy()
