"""Single-kernel micro-benchmarks through the C ABI: ``python -m grilly_b200.microbench <op> [options]``.

    linear     y = act(x W^T + b) (+ residual)      --m --n --k --act {none,gelu,silu,relu} --residual --precision
    gemm       C = A B, row-major                    --m --n --k --precision
    attention  flash_attention2 on packed sentences  --b --s --h --d (lengths uniform in [16, s]) --causal --rope
    linear_ln  y = LayerNorm(x W^T + b + residual)   --m --n --k --precision (one kernel for n in 128/256/384/512)
    layernorm  y = LayerNorm(x)                      --m --n
    faiss      cosine distances (--m queries, --n database vectors, --k dim) and top-k (--topk) of the result

Inputs are seeded synthetic data already resident on the GPU; the op is launched ``--warmup`` times, then ``--reps``
launches are timed with CUDA events on the launching stream and the average is printed with the algorithmic
TFLOP/s and GB/s. With ``--reps 1`` the last launch is the only timed one, which is the form used for ncu captures
(``-k regex:<kernel> -s <warmup> -c 1``).
"""
from __future__ import annotations

import argparse
import math

import numpy as np

from . import _lib as L
from .clocks import ClockSampler
from .device import Device


LAST_CLOCKS = {}


def _time(dev, fn, warmup, reps):
    """ms per launch (CUDA events on the library's stream); the SM clocks sampled over the timed launches are left in
    LAST_CLOCKS and printed with the number."""
    for _ in range(warmup):
        fn()
    dev.sync()
    sampler = ClockSampler(getattr(dev, "index", 0)).start()
    dev.timer_start()
    for _ in range(reps):
        fn()
    ms = dev.timer_stop() / reps
    LAST_CLOCKS.clear()
    LAST_CLOCKS.update(sampler.stop())
    return ms


def _clk() -> str:
    c = LAST_CLOCKS
    return f"[SM {c.get('sm_mhz')} of {c.get('sm_max_mhz')} MHz, reasons {c.get('reasons')}, {c.get('samples')} samples]"


def _nsplit(a):
    """C = A B with B column-split across the ranks (one process per GPU, NCCL all-gather of C per row slab)."""
    import os

    import torch
    import torch.distributed as dist

    from .compute import Compute
    from .dist import CudaLocalGemm, gemm_nsplit

    rank_local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(rank_local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank_local))
    world = dist.get_world_size()
    backend = Compute(device=rank_local, precision=a.precision)
    rng = np.random.default_rng(4)
    A = rng.standard_normal((a.m, a.k)).astype(np.float32)
    B = rng.standard_normal((a.k, a.n)).astype(np.float32)
    n_loc = a.n // world
    if a.fused:
        from .dist import FusedNsplit
        op = FusedNsplit(backend, a.m, a.n, a.k)
        op.prepare(A, B[:, dist.get_rank() * n_loc:(dist.get_rank() + 1) * n_loc])
        step = op.run_copy if a.p2p_copy else op.run
    else:
        local = CudaLocalGemm(backend)
        local.prepare(A, B[:, dist.get_rank() * n_loc:(dist.get_rank() + 1) * n_loc])
        step = lambda: gemm_nsplit(A, B, local=local, return_tensor=True, prepared=True)  # noqa: E731
    for _ in range(a.warmup):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    sampler = ClockSampler(rank_local).start() if dist.get_rank() == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.reps):
        step()
    e1.record()
    torch.cuda.synchronize()
    if sampler is not None:
        LAST_CLOCKS.clear()
        LAST_CLOCKS.update(sampler.stop())
    t = torch.tensor([e0.elapsed_time(e1) / a.reps], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if dist.get_rank() == 0:
        ms = t.item()
        sent = (world - 1) / world * a.m * a.n * 4.0
        how = ("peer copies" if a.p2p_copy else "epilogue stores to peers") if a.fused else "all-gather"
        print(f"gemm n-split x{world} {a.m}x{a.n}x{a.k} {a.precision}: {ms * 1e3:.1f} us (max over ranks)  "
              f"{2.0 * a.m * a.n * a.k / ms / 1e9:.1f} TFLOP/s aggregate  {how} {sent / ms / 1e6:.1f} GB/s sent per GPU  {_clk()}")
    backend.cleanup()
    dist.destroy_process_group()


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("op", choices=["linear", "linear_ln", "gemm", "attention", "layernorm", "faiss"])
    ap.add_argument("--m", "--dim-m", dest="m", type=int, default=18432)
    ap.add_argument("--n", "--dim-n", dest="n", type=int, default=1536)
    ap.add_argument("--k", "--dim-k", dest="k", type=int, default=384)
    ap.add_argument("--act", default="none", choices=["none", "gelu", "silu", "relu"])
    ap.add_argument("--residual", action="store_true")
    ap.add_argument("--out-bf16", action="store_true", help="linear in bf16 mode: bf16 output (as between the layers of the bf16 encoder)")
    ap.add_argument("--precision", default="tf32", choices=["tf32", "bf16"])
    ap.add_argument("--b", type=int, default=256)
    ap.add_argument("--s", type=int, default=128)
    ap.add_argument("--h", type=int, default=12)
    ap.add_argument("--d", type=int, default=32)
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--rope", action="store_true")
    ap.add_argument("--full-length", action="store_true", help="attention: every sentence has length s")
    ap.add_argument("--topk", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--p2p-copy", action="store_true", help="with --nsplit --fused: exchange by strided peer copies per row slab")
    ap.add_argument("--fused", action="store_true", help="with --nsplit: exchange C inside the GEMM epilogue (peer stores)")
    ap.add_argument("--nsplit", action="store_true",
                    help="gemm: split B by columns over the ranks of a torch.distributed.run launch and all-gather C")
    a = ap.parse_args(argv)
    if a.nsplit:
        return _nsplit(a)

    dev = Device(a.device)
    lib, ctx = dev.lib, dev.ctx
    rng = np.random.default_rng(0)
    bf16 = a.precision == "bf16"
    prec = L.PREC_BF16 if bf16 else L.PREC_TF32
    dt = "bf16" if bf16 else "f32"
    elt = 2 if bf16 else 4
    try:
        if a.op == "linear":
            x = dev.upload(rng.standard_normal((a.m, a.k)).astype(np.float32), dt, round_tf32=True)
            w = dev.upload((rng.standard_normal((a.n, a.k)) * 0.05).astype(np.float32), dt, round_tf32=True)
            b = dev.upload(np.zeros(a.n, np.float32))
            r = dev.upload(np.zeros((a.m, a.n), np.float32)) if a.residual else None
            out16 = bf16 and a.out_bf16
            y = dev.empty((a.m, a.n), "bf16" if out16 else "f32")
            act = {"none": L.ACT_NONE, "gelu": L.ACT_GELU, "silu": L.ACT_SILU, "relu": L.ACT_RELU}[a.act]
            flags = L.FLAG_OUT_BF16 if out16 else L.FLAG_ROUND_TF32
            fn = lambda: dev.check(lib.grilly_linear(ctx, x.ptr, w.ptr, b.ptr, r.ptr if r else None, y.ptr, a.m, a.n, a.k, act,  # noqa: E731
                                                     prec, flags))
            flops = 2.0 * a.m * a.n * a.k
            nbytes = elt * (a.m * a.k + a.n * a.k) + (2.0 if out16 else 4.0) * a.m * a.n + (4.0 * a.m * a.n if a.residual else 0.0)
        elif a.op == "linear_ln":
            x = dev.upload(rng.standard_normal((a.m, a.k)).astype(np.float32), dt, round_tf32=True)
            w = dev.upload((rng.standard_normal((a.n, a.k)) * 0.05).astype(np.float32), dt, round_tf32=True)
            b, g, bt = dev.upload(np.zeros(a.n, np.float32)), dev.upload(np.ones(a.n, np.float32)), dev.upload(np.zeros(a.n, np.float32))
            r = dev.upload(rng.standard_normal((a.m, a.n)).astype(np.float32), dt) if a.residual else None
            y, scratch = dev.empty((a.m, a.n)), dev.empty((a.m, a.n))
            fn = lambda: dev.check(lib.grilly_linear_layernorm(ctx, x.ptr, w.ptr, b.ptr, r.ptr if r else None, g.ptr, bt.ptr, y.ptr,  # noqa: E731
                                                               scratch.ptr, a.m, a.n, a.k, 1e-5, prec, L.FLAG_ROUND_TF32 if not bf16 else 0))
            flops = 2.0 * a.m * a.n * a.k
            nbytes = elt * (a.m * a.k + a.n * a.k) + 4.0 * a.m * a.n + (elt * a.m * a.n if a.residual else 0)
        elif a.op == "gemm":
            A = dev.upload(rng.standard_normal((a.m, a.k)).astype(np.float32), dt, round_tf32=True)
            B = dev.upload(rng.standard_normal((a.k, a.n)).astype(np.float32), dt, round_tf32=True)
            Cm = dev.empty((a.m, a.n))
            fn = lambda: dev.check(lib.grilly_gemm_mnk(ctx, A.ptr, B.ptr, Cm.ptr, a.m, a.k, a.n, prec, 0))  # noqa: E731
            flops = 2.0 * a.m * a.n * a.k
            nbytes = elt * (a.m * a.k + a.n * a.k) + 4.0 * a.m * a.n
        elif a.op == "attention":
            lens = np.full(a.b, a.s) if a.full_length else rng.integers(min(16, a.s), a.s + 1, size=a.b)
            cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
            T = int(cu[-1])
            F = a.h * a.d
            qkv = dev.upload(rng.standard_normal((T, 3 * F)).astype(np.float32), dt, round_tf32=True)
            cud = dev.upload(cu, "i32")
            out = dev.empty((T, F))
            rope = L.ROPE_INTERLEAVED if a.rope else L.ROPE_NONE
            fn = lambda: dev.check(lib.grilly_flash_attention(  # noqa: E731
                ctx, qkv.ptr, qkv.ptr + elt * F, qkv.ptr + 2 * elt * F, out.ptr, a.b, int(lens.max()), a.h, a.d, 3 * F, F, cud.ptr, T,
                None, 1.0 / math.sqrt(a.d), int(a.causal), rope, 10000.0, 1.0, prec, 0))
            flops = 4.0 * a.h * a.d * float((lens.astype(np.float64) ** 2).sum()) * (0.5 if a.causal else 1.0)
            nbytes = T * F * (3.0 * elt + 4.0)
        elif a.op == "faiss":
            q = dev.upload(rng.standard_normal((a.m, a.k)).astype(np.float32))
            db = dev.upload(rng.standard_normal((a.n, a.k)).astype(np.float32))
            dist = dev.empty((a.m, a.n))
            idx = dev.empty((a.m, a.topk), "i32")
            val = dev.empty((a.m, a.topk))
            fn = lambda: dev.check(lib.grilly_faiss_distances(ctx, q.ptr, db.ptr, dist.ptr, a.m, a.n, a.k, L.DIST_COSINE))  # noqa: E731
            ms = _time(dev, fn, a.warmup, a.reps)
            print(f"faiss distances {a.m} x {a.n} x {a.k}: {ms * 1e3:.1f} us/launch  {2.0 * a.m * a.n * a.k / ms / 1e9:.1f} TFLOP/s "
                  f"(fp32 dot products; the split GEMM does 3x that)  {4.0 * (a.m * a.k + a.n * a.k + a.m * a.n) / ms / 1e6:.1f} GB/s (algorithmic)  {_clk()}")
            fn = lambda: dev.check(lib.grilly_faiss_topk(ctx, dist.ptr, a.m, a.n, a.topk, idx.ptr, val.ptr))  # noqa: E731
            flops = 0.0
            nbytes = 4.0 * a.m * a.n                       # every distance read once
        else:
            x = dev.upload(rng.standard_normal((a.m, a.n)).astype(np.float32))
            g = dev.upload(np.ones(a.n, np.float32))
            bt = dev.upload(np.zeros(a.n, np.float32))
            y = dev.empty((a.m, a.n))
            fn = lambda: dev.check(lib.grilly_layernorm(ctx, x.ptr, None, g.ptr, bt.ptr, y.ptr, a.m, a.n, 1e-5, L.NORM_LAYER, 0))  # noqa: E731
            flops = 8.0 * a.m * a.n
            nbytes = 8.0 * a.m * a.n
        ms = _time(dev, fn, a.warmup, a.reps)
        dev.sync()
        print(f"{a.op} {vars(a)}\n  {ms * 1e3:.1f} us/launch  {flops / ms / 1e9:.1f} TFLOP/s  {nbytes / ms / 1e6:.1f} GB/s (algorithmic)  {_clk()}")
    finally:
        dev.close()


if __name__ == "__main__":
    main()
