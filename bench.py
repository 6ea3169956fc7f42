"""Headline benchmark: MiniLM-L6-shaped sentence-encoder forward, sentences per second.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched once per GPU by torch.distributed.run)
    python bench.py --impl reference ...                     (the reference's own CPU code for the path, on host cores)

Workload (per GPU, weak scaling): batch 1024 x seq 128 token ids uniform in [1000, 30000), valid lengths uniform
in [16, 128], 6 post-LN layers, hidden 384, 12 heads, FFN 1536 GELU, vocab 30522, random-init weights (std 0.02),
mean-pool + L2 normalise. One step = one forward of that batch. Rank 0 prints ONE JSON line.

`value`   : sentences/s with token ids already in HBM (device-timed, kernels only).
`e2e`     : the same through the public API with host buffers (ids copied host->device from pinned memory and the
            embeddings copied back, both inside the timed region).
`roofline`: the tcgen05 GEMM kernels (the dominant kernel class), algorithmic FLOPs / event-timed kernel time, against
            the measured BURST peak (the timed region is a fraction of a second); the sustained figure is given beside it.
`cpu_baseline`: the reference's own `_forward_layer` NumPy path (or, without the reference copy, the NumPy port) on a
            bounded sample of the same workload.
Further keys put the rest of the metric ("GEMM & attention TFLOP/s") into the same record, each timed launch by
launch with CUDA events, the L2 flushed between launches and its own clock samples:
`linear_cfg0`, `attention_cfg1`, `attention_cfg3`, `gemm_mnk_sweep` at N = 1; `strong` (global batch 1024 split
over the ranks) and `gemm_nsplit` (column-split product, NCCL all-gather and in-kernel peer stores) at N > 1.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

from grilly_b200.clocks import ClockSampler

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CFG = dict(num_layers=6, hidden=384, heads=12, ffn=1536, vocab=30522, max_pos=512, batch=1024, seq=128)
WORKLOAD = "minilm_l6_h384_encoder_forward_b1024_s128_per_gpu"
# DRAM bytes (read + write) per algorithmic byte of a GEMM launch of this workload, from one ncu capture of the QKV
# launch (74 884 x 1152 x 384: 116.9 MB read + 288.8 MB written for 461.9 MB algorithmic; the tail of the output is
# still in L2 when the kernel ends). roofline.traffic scales it by the algorithmic bytes of the run's average launch.
NCU_GEMM_DRAM_PER_ALGORITHMIC_BYTE = 405.7 / 461.9


def make_batch(rank: int):
    rng = np.random.default_rng(2 + 1000 * rank)
    ids = rng.integers(1000, 30000, size=(CFG["batch"], CFG["seq"])).astype(np.int32)
    lens = rng.integers(16, CFG["seq"] + 1, size=CFG["batch"]).astype(np.int32)
    mask = (np.arange(CFG["seq"])[None, :] < lens[:, None]).astype(np.float32)
    return ids, lens, mask


def encoder_flops(lens) -> float:
    """Valid-token FLOPs of one forward: 6 layers x [2 L (4 h^2 + 2 h ffn) + 4 L^2 h] per sentence of length L."""
    h, f, nl = CFG["hidden"], CFG["ffn"], CFG["num_layers"]
    lens = np.asarray(lens, dtype=np.float64)
    return float((nl * (2 * lens * (4 * h * h + 2 * h * f) + 4 * lens * lens * h)).sum())


def load_peaks() -> dict:
    """Measured peaks of this pool's B200s (HBM copy GB/s, cuBLAS bf16 TFLOP/s burst and sustained); the stated
    fallback when the file is absent. tf32 MMA runs at half the bf16 rate, so tf32 peaks are half the bf16 ones."""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        p = json.loads(path.read_text())
        return {"hbm": p["hbm_gbs"], "bf16_burst": p["bf16_tflops"], "bf16_sustained": p["bf16_tflops_sustained"], "basis": "measured"}
    return {"hbm": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "basis": "fallback"}


# ------------------------------------------------------------------------------------------------ CPU arm
def cpu_encoder(sample_sentences: int):
    """One pass of the reference's CPU encoder path over the first `sample_sentences` sentences of the workload.

    With the reference copy present (oracle/_ref, made by oracle/make_ref.py) this is the reference's own
    ``VulkanSentenceTransformer._forward_layer`` (its NumPy branches: float32 products on all BLAS threads), kind
    "reference"; otherwise the NumPy restatement in oracle/oracle.py (float64 accumulation), kind "port".
    Returns (seconds, kind). This function and run_reference() are the only places bench.py executes oracle/."""
    from oracle import ref_encoder as R
    from grilly_b200.encoder import EncoderWeights   # weight container only: importing the package maps no CUDA library

    rng = np.random.default_rng(2)
    w = EncoderWeights.random(rng, CFG["num_layers"], CFG["hidden"], CFG["ffn"], CFG["vocab"], CFG["max_pos"]).as_dict()
    ids, lens, mask = make_batch(0)
    ids, mask = ids[:sample_sentences], mask[:sample_sentences]
    if R.available():
        fwd, kind = (lambda i, m: R.encoder_forward(i, m, w, CFG["heads"])), "reference"
    else:
        from oracle import oracle as O
        fwd, kind = (lambda i, m: O.encoder_forward(i, m, w, CFG["heads"])), "port"
    fwd(ids[:2], mask[:2])  # warm-up (imports, BLAS threads, page faults)
    t0 = time.perf_counter()
    fwd(ids, mask)
    return time.perf_counter() - t0, kind


def cpu_baseline_entry(sample: int) -> dict:
    cores = os.cpu_count() or 1
    dt, kind = cpu_encoder(sample)
    what = ("the reference's own VulkanSentenceTransformer._forward_layer NumPy path (float32 BLAS products)" if kind == "reference"
            else "NumPy port of the reference's CPU path (float64 accumulation)")
    return {"value": sample / dt, "unit": "sentences/s", "cores": cores, "kind": kind,
            "sample": f"first {sample} of the 1024 sentences, {what}, {dt:.1f} s on {cores} host threads"}


def run_reference(args, rank: int):
    if rank != 0:
        return
    sample = 32   # about 10 s of host work per step: 20 steps end within a few minutes
    for _ in range(min(args.warmup, 1)):
        cpu_encoder(8)
    times, kind = [], "port"
    for _ in range(args.steps):
        dt, kind = cpu_encoder(sample)
        times.append(dt)
    ms = 1e3 * sum(times) / len(times)
    value = sample / (ms / 1e3)
    cores = os.cpu_count() or 1
    line = {
        "impl": "reference", "metric": "encoder_sentences_per_sec", "value": value, "unit": "sentences/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 (NumPy/BLAS)" if kind == "reference" else "f64-accumulate NumPy", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "CPU path only: the reference's Vulkan shaders cannot run here "
                   "(no graphics stack); each step is a 32-sentence sample of the 1024-sentence batch"},
        "cpu_baseline": {"value": value, "unit": "sentences/s", "cores": cores, "kind": kind,
                         "sample": f"{sample} of 1024 sentences per step, "
                                   + ("the reference's own _forward_layer NumPy path" if kind == "reference" else "NumPy port of it")
                                   + f" on {cores} host threads"},
        "e2e": {"value": value, "unit": "sentences/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ per-kernel extras
class Extras:
    """Single-launch measurements of the other configurations the metric names, through the C ABI on device-resident
    inputs. Every launch is timed alone with CUDA events on the launching stream, after an L2 flush (a 256 MB buffer
    rewritten outside the events), with nvidia-smi sampling the clocks over the whole loop."""

    def __init__(self, dev, gpu_index: int, l2_flush, peaks: dict):
        import ctypes as C
        from grilly_b200 import _lib as L

        self.C, self.L, self.dev, self.lib, self.gpu, self.flush, self.peaks = C, L, dev, dev.lib, gpu_index, l2_flush, peaks

    def _measure(self, fn, est_ms: float) -> dict:
        reps = int(min(2000, max(20, 300.0 / max(est_ms + 0.1, 1e-3))))
        for _ in range(3):
            fn()
        self.dev.sync()
        sampler = ClockSampler(self.gpu).start()
        ms = []
        for _ in range(reps):
            self.flush()
            self.dev.timer_start()
            fn()
            ms.append(self.dev.timer_stop())
        clocks = sampler.stop()
        return {"ms_median": statistics.median(ms), "ms_best": min(ms), "launches_timed": reps, "l2": "flushed before every launch",
                "clocks": clocks}

    def _tensor_entry(self, r: dict, flops: float, nbytes: float, bf16: bool) -> dict:
        t = r["ms_median"] * 1e-3
        burst = self.peaks["bf16_burst"] * (1.0 if bf16 else 0.5)
        sustained = self.peaks["bf16_sustained"] * (1.0 if bf16 else 0.5)
        r.update({"tflops": flops / t / 1e12, "frac_of_burst_peak": flops / t / 1e12 / burst, "burst_peak_tflops": burst,
                  "frac_of_sustained_peak": flops / t / 1e12 / sustained, "algorithmic_gbytes_per_s": nbytes / t / 1e9,
                  "frac_of_hbm_peak": nbytes / t / 1e9 / self.peaks["hbm"]})
        return r

    def linear_cfg0(self) -> dict:
        """configs[0]: fused linear + GELU, x (rows, 384), W (1536, 384), zero bias; rows 32 and 4096; tf32."""
        dev, lib, L = self.dev, self.lib, self.L
        rng = np.random.default_rng(0)
        lim = math.sqrt(6.0 / (384 + 1536))
        w = dev.upload(rng.uniform(-lim, lim, size=(1536, 384)).astype(np.float32), round_tf32=True)
        b = dev.upload(np.zeros(1536, np.float32))
        out = {}
        for rows in (32, 4096):
            x = dev.upload(rng.standard_normal((rows, 384)).astype(np.float32), round_tf32=True)
            y = dev.empty((rows, 1536))
            fn = lambda: dev.check(lib.grilly_linear(dev.ctx, x.ptr, w.ptr, b.ptr, None, y.ptr, rows, 1536, 384, L.ACT_GELU, L.PREC_TF32, 0))  # noqa: E731
            r = self._measure(fn, 0.02)
            out[f"rows_{rows}"] = self._tensor_entry(r, 2.0 * rows * 1536 * 384, 4.0 * (rows * 384 + 1536 * 384 + 1536 + rows * 1536), False)
            x.free(), y.free()
        return out

    def attention(self, B, S, H, D, bf16, causal, rope) -> dict:
        dev, lib, L = self.dev, self.lib, self.L
        rng = np.random.default_rng(1 if not causal else 3)
        dt = "bf16" if bf16 else "f32"
        q, k, v = (dev.upload(rng.standard_normal((B, S, H, D)).astype(np.float32), dt, round_tf32=True) for _ in range(3))
        o = dev.empty((B, S, H, D))
        fn = lambda: dev.check(lib.grilly_flash_attention(  # noqa: E731
            dev.ctx, q.ptr, k.ptr, v.ptr, o.ptr, B, S, H, D, H * D, H * D, None, B * S, None, 1.0 / math.sqrt(D), int(causal),
            L.ROPE_INTERLEAVED if rope else L.ROPE_NONE, 10000.0, 1.0, L.PREC_BF16 if bf16 else L.PREC_TF32, 0))
        flops = 4.0 * B * H * float(S) * S * D * (0.5 if causal else 1.0)
        nbytes = float(B) * S * H * D * (3 * (2 if bf16 else 4) + 4)
        r = self._tensor_entry(self._measure(fn, flops / 4e14 * 1e3), flops, nbytes, bf16)
        r["shape"] = {"batch": B, "seq": S, "heads": H, "head_dim": D, "dtype": "bf16" if bf16 else "tf32", "causal": causal, "rope": rope}
        for t in (q, k, v, o):
            t.free()
        return r

    def gemm_mnk_sweep(self) -> dict:
        """configs[4] on one GPU: C = A B, M = N = K in {1024 .. 16384}, fp32-in/tf32 and bf16-in/fp32-accumulate."""
        dev, lib, L = self.dev, self.lib, self.L
        out = {}
        for n in (1024, 2048, 4096, 8192, 16384):
            rng = np.random.default_rng(4 + int(math.log2(n)))
            a32 = dev.upload(rng.standard_normal((n, n), dtype=np.float32), round_tf32=True)
            b32 = dev.upload(rng.standard_normal((n, n), dtype=np.float32), round_tf32=True)
            c = dev.empty((n, n))
            for mode in ("tf32", "bf16"):
                if mode == "bf16":
                    a, b = dev.empty((n, n), "bf16"), dev.empty((n, n), "bf16")
                    dev.check(lib.grilly_cast_f32_to_bf16(dev.ctx, a32.ptr, a.ptr, n * n))
                    dev.check(lib.grilly_cast_f32_to_bf16(dev.ctx, b32.ptr, b.ptr, n * n))
                else:
                    a, b = a32, b32
                prec = L.PREC_BF16 if mode == "bf16" else L.PREC_TF32
                fn = lambda: dev.check(lib.grilly_gemm_mnk(dev.ctx, a.ptr, b.ptr, c.ptr, n, n, n, prec, 0))  # noqa: E731
                flops = 2.0 * n ** 3
                r = self._measure(fn, flops / (1.2e15 if mode == "bf16" else 6e14) * 1e3)
                out[f"{n}_{mode}"] = self._tensor_entry(r, flops, (8.0 if mode == "bf16" else 12.0) * n * n, mode == "bf16")
                if mode == "bf16":
                    a.free(), b.free()
            for t in (a32, b32, c):
                t.free()
        return out


def nsplit_extra(backends: dict, dist, torch, local_rank: int, peaks: dict) -> dict:
    """configs[4] across the ranks: B split by columns, every rank ends with the full C. Three exchanges: NCCL
    all-gather per row slab, plain stores from the GEMM epilogue into the peers' C (symmetric memory), and row-slab
    peer copies. Times are CUDA events on torch's current stream (the library's launches are ordered inside it),
    max over ranks."""
    from grilly_b200.dist import CudaLocalGemm, FusedNsplit, gemm_nsplit

    world, rank = dist.get_world_size(), dist.get_rank()
    out = {}

    def timed(step, reps):
        for _ in range(2):
            step()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            step()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / reps], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    def one(backend, n, A, B, cols, flops, sent):
        sampler = ClockSampler(local_rank).start()
        # one GPU, whole product, same run (the basis of the efficiency figures)
        full = CudaLocalGemm(backend)
        full.prepare(A, B)
        c_full = full.empty(n, n)
        single_ms = timed(lambda: full.run_slab(0, n, c_full), 5)
        del c_full
        local = CudaLocalGemm(backend)
        local.prepare(A, B[:, cols])
        ag_ms = timed(lambda: gemm_nsplit(A, B, local=local, return_tensor=True, prepared=True), 5)
        fused = FusedNsplit(backend, n, n, n)
        fused.prepare(A, B[:, cols])
        st_ms = timed(fused.run, 5)
        cp_ms = timed(fused.run_copy, 5)
        clocks = sampler.stop()
        single_tf = flops / single_ms / 1e9
        entry = {"single_gpu_ms": single_ms, "single_gpu_tflops": single_tf, "bytes_sent_per_gpu": sent, "clocks": clocks,
                 "nvlink_floor_ms_at_770_gbs": sent / 770e9 * 1e3}
        for name, ms in (("nccl_all_gather", ag_ms), ("in_kernel_peer_stores", st_ms), ("peer_copies", cp_ms)):
            entry[name] = {"ms_max_over_ranks": ms, "aggregate_tflops": flops / ms / 1e9, "gbytes_per_s_sent_per_gpu": sent / ms / 1e6,
                           "efficiency_vs_n_x_single": (flops / ms / 1e9) / (world * single_tf)}
        del full, local, fused
        torch.cuda.empty_cache()
        return entry

    for n in (8192, 16384):
        rng = np.random.default_rng(4 + int(math.log2(n)))
        A = rng.standard_normal((n, n), dtype=np.float32)
        B = rng.standard_normal((n, n), dtype=np.float32)
        n_loc = n // world
        cols = slice(rank * n_loc, (rank + 1) * n_loc)
        flops, sent = 2.0 * n ** 3, (world - 1) / world * n * n * 4.0
        for backend in backends.values():
            out[f"{n}_{backend.precision}"] = one(backend, n, A, B, cols, flops, sent)
    return out


# ------------------------------------------------------------------------------------------------ main arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="grilly_b200", choices=["grilly_b200", "reference"])
    ap.add_argument("--chunk-tokens", type=int, default=int(os.environ.get("GRILLY_CHUNK_TOKENS", "0")))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="only the encoder line (skip the per-kernel / multi-GPU extras)")
    ap.add_argument("--precision", default="tf32", choices=["tf32", "bf16"],
                    help="tf32 (default, the fp32-parity mode the headline is quoted in) or bf16")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world == 1:
        # started without a launcher: start one process per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29531"), __file__] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    dist = torch = None
    if world > 1:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # peer mappings only, no multicast binding
        import torch
        import torch.distributed as dist

        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    import ctypes as C

    import grilly_b200

    dev = grilly_b200.Device(local_rank)
    rng = np.random.default_rng(2)  # same weights on every rank (replicated model)
    weights = grilly_b200.EncoderWeights.random(rng, CFG["num_layers"], CFG["hidden"], CFG["ffn"], CFG["vocab"], CFG["max_pos"])
    enc = grilly_b200.SentenceEncoder(weights, num_heads=CFG["heads"], device=dev, chunk_tokens=args.chunk_tokens,
                                      precision=args.precision)
    ids, lens, mask = make_batch(rank)
    B, S, F = CFG["batch"], CFG["seq"], CFG["hidden"]

    ids_dev = dev.upload(ids, "i32")
    out_dev = dev.empty((B, F))
    flush = dev.empty((64 * 1024 * 1024,))  # 256 MB > 126 MB L2, rewritten between timed steps
    flush_src = dev.empty((64 * 1024 * 1024,))
    lib = dev.lib

    def l2_flush():
        dev.check(lib.grilly_round_tf32(dev.ctx, C.c_void_p(flush_src.ptr), C.c_void_p(flush.ptr), flush.size))

    def barrier():
        dev.sync()
        if dist is not None:
            dist.barrier()

    def step_device():
        enc.forward_device(ids_dev.ptr, lens, B, S, out_dev.ptr)

    # end to end: the ids sit in the encoder's page-locked input buffer (as a tokenizer would leave them there) and the
    # embeddings come back into its page-locked output buffer; both copies run inside every step
    ids_pinned, out_host = enc.io_buffers(B, S)
    ids_pinned[...] = ids

    def step_e2e():
        enc.encode_ids(ids_pinned, mask, out=out_host)

    for _ in range(args.warmup):
        step_device()
        step_e2e()
    barrier()

    # ---- timed region 1: kernels only, inputs resident in HBM, device-timed per step with an L2 flush between
    sampler = ClockSampler(local_rank).start()
    launches0 = dev.launch_count()
    step_ms = []
    barrier()
    for _ in range(args.steps):
        l2_flush()
        dev.timer_start()  # CUDA events on the stream the kernels are launched on
        step_device()
        step_ms.append(dev.timer_stop())
    barrier()
    launches = dev.launch_count() - launches0 - args.steps  # minus the flush launches

    # ---- timed region 2: end to end through the public API (host ids in, host embeddings out)
    e2e_ms = []
    barrier()
    for _ in range(args.steps):
        l2_flush()
        dev.sync()
        t0 = time.perf_counter()
        step_e2e()
        e2e_ms.append((time.perf_counter() - t0) * 1e3)
    barrier()

    # ---- per-kernel-class timing with CUDA events on the launching stream (separate pass, same steps)
    dev.profile_begin()
    for _ in range(args.steps):
        l2_flush()
        step_device()
    prof = dev.profile_end()
    clocks = sampler.stop()  # sampled across the three measurement passes (device-timed, end-to-end, per-kernel)

    total_ms, total_e2e_ms = sum(step_ms), sum(e2e_ms)
    if dist is not None:
        t = torch.tensor([total_ms, total_e2e_ms], dtype=torch.float64, device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, total_e2e_ms = t.tolist()

    peaks = load_peaks()
    line = None
    if rank == 0:
        bf16 = args.precision == "bf16"
        peak_burst = peaks["bf16_burst"] * (1.0 if bf16 else 0.5)
        peak_sustained = peaks["bf16_sustained"] * (1.0 if bf16 else 0.5)
        peak_note = (f"{'' if bf16 else '0.5 x '}{peaks['basis']} BURST bf16 cuBLAS TFLOP/s"
                     f"{'' if bf16 else ' (tf32 MMA rate is half the bf16 rate)'}: the timed region is a fraction of a second at the "
                     f"burst clock; of {peaks['basis']}")
        g = prof["gemm"]
        gemm_tflops = g["flops"] / (g["ms"] * 1e-3) / 1e12 if g["ms"] > 0 else None
        a = prof["attention"]
        valid_flops = encoder_flops(lens)
        ms_per_step = total_ms / args.steps
        value = world * B / (ms_per_step * 1e-3)
        e2e_value = world * B / (total_e2e_ms / args.steps * 1e-3)
        traffic = NCU_GEMM_DRAM_PER_ALGORITHMIC_BYTE * g["bytes"] / max(g["launches"], 1) if g["launches"] else None
        classes = {}
        for k, v in prof.items():
            if v["launches"]:
                t = v["ms"] * 1e-3
                classes[k] = {"launches": v["launches"], "ms_per_step": v["ms"] / args.steps,
                              "algorithmic_gbytes_per_s": v["bytes"] / t / 1e9 if t > 0 and v["bytes"] else None,
                              "frac_of_hbm_peak": v["bytes"] / t / 1e9 / peaks["hbm"] if t > 0 and v["bytes"] else None}
        line = {
            "metric": "encoder_sentences_per_sec", "value": value, "unit": "sentences/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None,
            "dtype": "tf32 (fp32 storage, fp32 accumulate)" if args.precision == "tf32" else "bf16 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": WORKLOAD, "global_batch": world * B, "seq_len": S, "valid_tokens_per_gpu": int(lens.sum()),
                       "parallelism": f"batch-sharded x{world}, no collective", "l2": "256 MB buffer rewritten between timed steps",
                       "chunk_tokens": args.chunk_tokens, "timing": "CUDA events around each step on the launching stream; L2 flush outside the events"},
            "e2e": {"value": e2e_value, "unit": "sentences/s", "h2d_bytes_per_step": int(ids.nbytes),
                    "d2h_bytes_per_step": int(out_host.nbytes)},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": "tcgen05 GEMM kernels (all encoder GEMMs of the step)", "achieved": gemm_tflops,
                         "peak": peak_burst, "unit": "TFLOP/s", "frac": (gemm_tflops / peak_burst) if gemm_tflops else None,
                         "traffic": traffic, "traffic_basis": "scaled from one ncu capture of the QKV launch of this workload by the "
                                                             "algorithmic bytes of the run's average GEMM launch",
                         "peak_basis": peak_note, "peak_sustained": peak_sustained,
                         "frac_of_sustained_peak": (gemm_tflops / peak_sustained) if gemm_tflops else None,
                         "launches": g["launches"], "avg_launch_ms": g["ms"] / max(g["launches"], 1),
                         "algorithmic_gbytes_per_s": g["bytes"] / (g["ms"] * 1e-3) / 1e9 if g["ms"] > 0 else None},
            "kernel_classes": classes,
            "attention_tflops": (a["flops"] / (a["ms"] * 1e-3) / 1e12) if a["ms"] > 0 else None,
            "encoder_valid_tflops": valid_flops / (ms_per_step * 1e-3) / 1e12,
        }

    # ---- the rest of the metric in the same record
    if not args.no_extras:
        if world == 1:
            ex = Extras(dev, local_rank, l2_flush, peaks)
            line["linear_cfg0"] = ex.linear_cfg0()
            line["attention_cfg1"] = ex.attention(32, 64, 8, 64, bf16=False, causal=False, rope=False)
            line["attention_cfg3"] = ex.attention(8, 4096, 16, 64, bf16=True, causal=True, rope=True)
            line["gemm_mnk_sweep"] = ex.gemm_mnk_sweep()
        else:
            # strong scaling: configs[2] as written, ONE batch of 1024 sentences split over the ranks
            from grilly_b200.dist import shard_range

            g_ids, g_lens, _ = make_batch(0)
            lo, hi = shard_range(B, rank, world)
            s_ids = dev.upload(g_ids[lo:hi], "i32")
            s_out = dev.empty((hi - lo, F))
            s_lens = g_lens[lo:hi]
            for _ in range(3):
                enc.forward_device(s_ids.ptr, s_lens, hi - lo, S, s_out.ptr)
            barrier()
            s_sampler = ClockSampler(local_rank).start()
            s_ms = []
            for _ in range(args.steps):
                l2_flush()
                dev.timer_start()
                enc.forward_device(s_ids.ptr, s_lens, hi - lo, S, s_out.ptr)
                s_ms.append(dev.timer_stop())
            s_clocks = s_sampler.stop()
            t = torch.tensor([sum(s_ms)], dtype=torch.float64, device=f"cuda:{local_rank}")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            strong_ms = t.item() / args.steps
            backends = {p: grilly_b200.Compute(device=local_rank, precision=p) for p in ("tf32", "bf16")}
            try:
                nsplit = nsplit_extra(backends, dist, torch, local_rank, peaks)
            finally:
                for b_ in backends.values():
                    b_.cleanup()
            if rank == 0:
                line["strong"] = {"global_batch": B, "sentences_per_gpu": hi - lo, "ms_per_step_max_over_ranks": strong_ms,
                                  "sentences_per_sec": B / (strong_ms * 1e-3), "scaling": "strong", "clocks": s_clocks,
                                  "valid_tokens_rank0": int(s_lens.sum())}
                line["gemm_nsplit"] = nsplit

    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_entry(64)
        print(json.dumps(line), flush=True)

    enc.close()
    dev.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
