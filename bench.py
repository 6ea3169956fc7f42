"""Headline benchmark: MiniLM-L6-shaped sentence-encoder forward, sentences per second.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched once per GPU by torch.distributed.run)
    python bench.py --impl reference ...                     (the CPU implementation of the same path, timed on host cores)

Workload (per GPU, weak scaling): batch 1024 x seq 128 token ids uniform in [1000, 30000), valid lengths uniform
in [16, 128], 6 post-LN layers, hidden 384, 12 heads, FFN 1536 GELU, vocab 30522, random-init weights (std 0.02),
mean-pool + L2 normalise. One step = one forward of that batch. Rank 0 prints ONE JSON line.

`value`   : sentences/s with token ids already in HBM (device-timed, kernels only).
`e2e`     : the same through the public API with host buffers (ids copied host->device from pinned memory and the
            embeddings copied back, both inside the timed region).
`roofline`: the tcgen05 GEMM kernel (the dominant kernel), algorithmic FLOPs / event-timed kernel time.
`cpu_baseline`: the NumPy restatement of the reference's CPU path on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CFG = dict(num_layers=6, hidden=384, heads=12, ffn=1536, vocab=30522, max_pos=512, batch=1024, seq=128)
WORKLOAD = "minilm_l6_h384_encoder_forward_b1024_s128_per_gpu"
NCU_GEMM_TRAFFIC_RATIO = 405.7 / 461.9  # dram bytes (read + write) per algorithmic byte, from the full-size ncu capture


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


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "50"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, mx, reasons = [], None, set()
        for r in self.rows:
            if len(r) < 8:
                continue
            try:
                clocks.append(float(r[1]))
                mx = float(r[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # under load = the upper half of the samples (idle samples before/after the region are dropped)
        clocks.sort()
        loaded = clocks[len(clocks) // 2:] if clocks else []
        return {"sm_mhz": statistics.median(loaded) if loaded else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(clocks)}


def cpu_baseline(sample_sentences: int, repeats: int = 1):
    """Times the CPU restatement of the reference's encoder path (NumPy, float32 products like the reference's
    NumPy branches, all BLAS threads) on the first `sample_sentences` sentences of the workload."""
    from oracle import oracle as O  # the one place bench.py runs the oracle: as the reported CPU baseline
    import grilly_b200.encoder as E

    rng = np.random.default_rng(2)
    w = E.EncoderWeights.random(rng, CFG["num_layers"], CFG["hidden"], CFG["ffn"], CFG["vocab"], CFG["max_pos"])
    ids, lens, mask = make_batch(0)
    ids, mask = ids[:sample_sentences], mask[:sample_sentences]
    O.encoder_forward(ids[:2], mask[:2], w.as_dict(), CFG["heads"])  # warm-up (BLAS threads, page faults)
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        O.encoder_forward(ids, mask, w.as_dict(), CFG["heads"])
        best = min(best, time.perf_counter() - t0)
    return sample_sentences / best, best


def run_reference(args, rank: int, world: int):
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    sample = 64
    times = []
    for _ in range(args.warmup):
        cpu_baseline(8)
    for _ in range(args.steps):
        _, dt = cpu_baseline(sample)
        times.append(dt)
    ms = 1e3 * sum(times) / len(times)
    value = sample / (ms / 1e3)
    line = {
        "impl": "reference", "metric": "encoder_sentences_per_sec", "value": value, "unit": "sentences/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f64-accumulate NumPy", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "CPU path only: the reference's Vulkan shaders cannot run here "
                   "(no graphics stack); each step is a 64-sentence sample of the 1024-sentence batch"},
        "cpu_baseline": {"value": value, "unit": "sentences/s", "cores": cores, "kind": "port",
                         "sample": f"{sample} of 1024 sentences per step, NumPy/BLAS on {cores} host threads"},
        "e2e": {"value": value, "unit": "sentences/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="grilly_b200", choices=["grilly_b200", "reference"])
    ap.add_argument("--chunk-tokens", type=int, default=int(os.environ.get("GRILLY_CHUNK_TOKENS", "0")))
    ap.add_argument("--no-cpu-baseline", action="store_true")
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
        run_reference(args, rank, world)
        return

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist

        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    import ctypes as C

    import grilly_b200
    from grilly_b200 import _lib as L

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

    out_host = np.empty((B, F), dtype=np.float32)

    def step_e2e():
        enc.encode_ids(ids, mask, out=out_host)

    for _ in range(args.warmup):
        step_device()
        step_e2e()
    barrier()

    # ---- timed region 1: kernels only, inputs resident in HBM, device-timed per step with an L2 flush between
    sampler = ClockSampler(local_rank)
    sampler.start()
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

    if rank == 0:
        peaks = {}
        pk_path = ROOT / "MEASURED_PEAKS.json"
        if pk_path.exists():
            peaks = json.loads(pk_path.read_text())
        bf16_sustained = peaks.get("bf16_tflops_sustained")
        peak_tf32 = (bf16_sustained / 2.0) if bf16_sustained else 1590.0 / 2.0 * (1400.0 / 1590.0)
        if args.precision == "bf16":
            peak_tf32 *= 2.0
        peak_note = ("0.5 x measured sustained bf16 cuBLAS TFLOP/s (tf32 MMA rate is half the bf16 rate); of measured"
                     if bf16_sustained else "0.5 x fallback sustained bf16 figure; of fallback")
        if args.precision == "bf16":
            peak_note = "measured sustained bf16 cuBLAS TFLOP/s; of measured" if bf16_sustained else "fallback sustained bf16 figure; of fallback"
        g = prof["gemm"]
        gemm_tflops = g["flops"] / (g["ms"] * 1e-3) / 1e12 if g["ms"] > 0 else None
        a = prof["attention"]
        valid_flops = encoder_flops(lens)
        ms_per_step = total_ms / args.steps
        value = world * B / (ms_per_step * 1e-3)
        e2e_value = world * B / (total_e2e_ms / args.steps * 1e-3)
        # DRAM traffic per launch: the ncu capture of the pair kernel on this run's QKV launch (74 884 x 1152 x 384,
        # profiles/gemm_tcgen05_encoder_shapes_knockout.md) moved 116.9 + 288.8 MB for 461.9 MB of algorithmic
        # bytes (the tail of the output is still in L2 when the kernel ends); that ratio is scaled by the
        # algorithmic bytes of this run's average GEMM launch
        traffic = NCU_GEMM_TRAFFIC_RATIO * g["bytes"] / max(g["launches"], 1) if g["launches"] else None
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
            "roofline": {"bound": "tensor", "kernel": "gemm_tcgen05_pair_kernel + gemm_tcgen05_kernel (all encoder GEMMs)", "achieved": gemm_tflops,
                         "peak": peak_tf32, "unit": "TFLOP/s", "frac": (gemm_tflops / peak_tf32) if gemm_tflops else None,
                         "traffic": traffic, "peak_basis": peak_note,
                         "launches": g["launches"], "avg_launch_ms": g["ms"] / max(g["launches"], 1),
                         "algorithmic_gbytes_per_s": g["bytes"] / (g["ms"] * 1e-3) / 1e9 if g["ms"] > 0 else None},
            "kernel_classes": {k: {"launches": v["launches"], "ms_per_step": v["ms"] / args.steps} for k, v in prof.items() if v["launches"]},
            "attention_tflops": (a["flops"] / (a["ms"] * 1e-3) / 1e12) if a["ms"] > 0 else None,
            "encoder_valid_tflops": valid_flops / (ms_per_step * 1e-3) / 1e12,
        }
        if world == 1 and not args.no_cpu_baseline:
            cores = os.cpu_count() or 1
            sample = 64
            v, dt = cpu_baseline(sample)
            line["cpu_baseline"] = {"value": v, "unit": "sentences/s", "cores": cores, "kind": "port",
                                    "sample": f"first {sample} of the 1024 sentences, NumPy/BLAS restatement of the reference's "
                                              f"CPU path, {dt:.1f} s on {cores} host threads"}
        print(json.dumps(line), flush=True)

    enc.close()
    dev.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
