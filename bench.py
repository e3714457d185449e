#!/usr/bin/env python
"""Benchmark of the packed-NF4 decode linear path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Workload (`config.workload`): the NF4 GEMV decode sweep of the baseline -
batch M in {1, 4, 16} on layers 4096->4096, 4096->14336 and 14336->4096 with
64-element blocks and double-quantised absmax (8-bit scales, FP32 second level
per 256 blocks). One step runs the nine (M, layer) cases once, each on a
different resident weight instance so that no step re-reads weights from L2.
The metric is packed-weight bytes (codes + scale payload) consumed per second.

Prints ONE JSON line (rank 0). See DESIGN.md for the definition of every key.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LAYERS = [(4096, 4096), (14336, 4096), (4096, 14336)]  # (out, in)
BATCHES = [1, 4, 16]
BLOCK, SCALE_BLOCK = 64, 256
L2_BYTES = 126 * 1024 * 1024
METRIC = "nf4_linear_packed_weight_bandwidth"
UNIT = "GB/s"


def packed_bytes(out_f: int, in_f: int) -> int:
    """Algorithmic bytes of one launch: codes + double-quantised scale payload."""
    n = out_f * in_f
    blocks = -(-n // BLOCK)
    return (n + 1) // 2 + blocks + 4 * (-(-blocks // SCALE_BLOCK)) + 4


STEP_BYTES = sum(packed_bytes(o, i) for o, i in LAYERS) * len(BATCHES)


def measured_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """nvidia-smi clock/throttle samples taken while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int) -> None:
        self.device_index = device_index
        self.proc = None
        self.file = None

    def __enter__(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.device_index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        if self.file is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        self.file.flush()
        rows = [r.strip().split(", ") for r in Path(self.file.name).read_text().splitlines() if r.strip()]
        os.unlink(self.file.name)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, flag in zip(names, r[5:9]):
                if flag.strip().lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


# ---- CPU reference arm / baseline ----------------------------------------------------

def cpu_sweep(weights_host: dict, xs_host: dict, cases: list[tuple[int, int, int]], use_all_threads: bool):
    """Runs the given (M, out, in) cases on the host. Returns (seconds, kind, threads).

    With the reference library present its own single-threaded loops are used;
    independent cases then run concurrently on separate threads when
    `use_all_threads` (the loops themselves stay as shipped). Otherwise the C
    restatement runs with OpenMP over independent outputs."""
    import oracle  # checker only; never on the product path

    threads = oracle.host_threads()
    if oracle.ref_available():
        ref = oracle.ref()

        def one(case):
            m, o, i = case
            import ctypes as C
            w = weights_host[(o, i)]
            sec = C.c_double(0)
            x = xs_host[(m, i)]
            import numpy as np
            y = np.empty((m, o), np.float32)
            rc = ref.lib.ref_linear_forward(*ref._wargs(w), oracle._ptr(x, oracle._f32p), oracle._ptr(y, oracle._f32p),
                                            m, C.byref(sec))
            if rc:
                raise RuntimeError(ref.lib.ref_last_error().decode())
            return sec.value

        workers = min(threads, len(cases)) if use_all_threads else 1
        t0 = time.perf_counter()
        if workers > 1:
            with ThreadPoolExecutor(workers) as pool:
                inner = list(pool.map(one, cases))
            seconds = time.perf_counter() - t0
        else:
            inner = [one(c) for c in cases]
            seconds = sum(inner)
        return seconds, "reference", workers
    port = oracle.port()
    use = threads if use_all_threads else 1
    t0 = time.perf_counter()
    for m, o, i in cases:
        port.linear_forward(weights_host[(o, i)], xs_host[(m, i)], threads=use)
    return time.perf_counter() - t0, "port", use


def host_inputs(seed_base: int = 5678):
    import numpy as np
    xs = {}
    for m in BATCHES:
        for _, i in LAYERS:
            if (m, i) not in xs:
                xs[(m, i)] = np.random.default_rng(seed_base + m * 131 + i).standard_normal((m, i)).astype(np.float32)
    return xs


def run_reference(args) -> None:
    """The reference's CPU implementation of the same sweep on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    import oracle

    port = oracle.port()
    rng = np.random.default_rng(1234)
    weights = {}
    for o, i in LAYERS:
        # Packed-domain synthetic payload (same distributions as the GPU arm's).
        n = o * i
        blocks = n // BLOCK
        codes = rng.integers(0, 256, n // 2, dtype=np.uint8)
        scales = np.maximum(0.0479 + 0.0066 * rng.standard_normal(blocks), 0.02).astype(np.float32)
        qs = np.zeros(blocks, np.uint8)
        second = np.zeros(-(-blocks // SCALE_BLOCK), np.float32)
        import ctypes as C
        off = C.c_float(0)
        port.lib.orc_double_quantize_scales(oracle._ptr(scales, oracle._f32p), blocks, SCALE_BLOCK,
                                            oracle._ptr(qs, oracle._u8p), oracle._ptr(second, oracle._f32p), C.byref(off))
        weights[(o, i)] = oracle.Nf4Weight(codes, o, i, BLOCK, scale_codes=qs, second_level=second,
                                           scale_block_size=SCALE_BLOCK, offset=float(off.value))
    xs = host_inputs()
    # Bounded sample per step: the M = 1 and M = 4 cases of every layer (6 of the 9 launches).
    sample = [(m, o, i) for m in (1, 4) for o, i in LAYERS]
    sample_bytes = sum(packed_bytes(o, i) for _, o, i in sample)
    steps = max(1, min(args.steps, 3))
    warm = 1 if args.warmup > 0 else 0
    for _ in range(warm):
        cpu_sweep(weights, xs, sample, True)
    total = 0.0
    kind, workers = "port", 1
    for _ in range(steps):
        sec, kind, workers = cpu_sweep(weights, xs, sample, True)
        total += sec
    value = sample_bytes * steps / total / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": 1e3 * total / steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "nf4_gemv_decode_sweep", "layers": LAYERS, "batches": BATCHES,
                   "block_size": BLOCK, "scale_block_size": SCALE_BLOCK, "scales": "double_quantized_u8"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": workers, "kind": kind,
                         "sample": "M in {1,4} on all three layers per step (6 of 9 launches), "
                                   "independent launches on separate host threads"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---- B200 arm ---------------------------------------------------------------------------

def run_b200(args) -> None:
    import numpy as np
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    import riftco_transformer_b200 as b2
    from riftco_transformer_b200 import synth

    if not b2.is_available():
        raise SystemExit("riftco_b200: " + b2.unavailability_reason())

    # Resident weight instances: enough copies of each layer to exceed 2x L2.
    copies = {}
    weights = {}
    for li, (o, i) in enumerate(LAYERS):
        n_copies = max(3, -(-2 * L2_BYTES // packed_bytes(o, i)))
        copies[(o, i)] = n_copies
        weights[(o, i)] = [synth.packed_weight(o, i, seed=1234 + 97 * li + c + 1000 * rank) for c in range(n_copies)]
    g = torch.Generator(device="cuda")
    g.manual_seed(5678)
    xs = {(m, i): torch.randn((m, i), device="cuda", generator=g) for m in BATCHES for _, i in LAYERS}
    ys = {(m, o): torch.empty((m, o), device="cuda") for m in BATCHES for o, _ in LAYERS}
    cases = [(m, o, i) for m in BATCHES for o, i in LAYERS]

    def step(k: int) -> None:
        for m, o, i in cases:
            w = weights[(o, i)][k % copies[(o, i)]]
            b2.dispatch_quantized_linear_forward(xs[(m, i)], w, ys[(m, o)], (m, i, o, BLOCK))

    # One CUDA graph per weight rotation index so that launches run back to back.
    n_graphs = max(copies.values())
    step(0)
    torch.cuda.synchronize()
    graphs = []
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for k in range(n_graphs):
            gph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gph, stream=side):
                step(k)
            graphs.append(gph)
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for k in range(args.warmup):
        graphs[k % n_graphs].replay()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as sampler:
        start.record()
        for k in range(args.steps):
            graphs[(args.warmup + k) % n_graphs].replay()
        stop.record()
        barrier()
        # keep the GPU busy a little longer so the sampler sees load for short runs
        elapsed_ms = start.elapsed_time(stop)
        t_end = time.perf_counter() + max(0.0, 0.6 - elapsed_ms / 1e3)
        k = 0
        while time.perf_counter() < t_end:
            graphs[k % n_graphs].replay()
            k += 1
        torch.cuda.synchronize()
    clocks = sampler.summary()
    if world > 1:
        t = torch.tensor([elapsed_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    value = STEP_BYTES * world * args.steps / (elapsed_ms / 1e3) / 1e9

    # Per-case kernel durations (CUDA events around back-to-back graph launches of one case).
    per_case = {}
    for m, o, i in cases:
        n_c = copies[(o, i)]
        gph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(gph, stream=side):
                for c in range(n_c):
                    b2.dispatch_quantized_linear_forward(xs[(m, i)], weights[(o, i)][c], ys[(m, o)], (m, i, o, BLOCK))
        torch.cuda.synchronize()
        for _ in range(3):
            gph.replay()
        torch.cuda.synchronize()
        reps = 20
        start.record()
        for _ in range(reps):
            gph.replay()
        stop.record()
        torch.cuda.synchronize()
        us = start.elapsed_time(stop) * 1e3 / (reps * n_c)
        per_case[f"M{m}_{i}to{o}"] = {"us": round(us, 3), "gbps": round(packed_bytes(o, i) / us / 1e3, 1)}

    peaks, peak_kind = measured_peaks()
    launches_per_step = len(cases)
    avg_launch_s = (elapsed_ms / 1e3) / (args.steps * launches_per_step)
    achieved = (STEP_BYTES / launches_per_step) / avg_launch_s / 1e9
    roofline = {
        "kernel": "nf4_gemv_kernel", "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"],
        "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "peak_source": peak_kind, "traffic": None,
        "per_case": per_case,
    }

    # End to end through the host-buffer entry point: pinned host x in, host y out, every launch.
    e2e = None
    xs_pin = {k: v.cpu().pin_memory() for k, v in xs.items()}
    ys_pin = {k: torch.empty(v.shape, dtype=torch.float32).pin_memory() for k, v in ys.items()}
    e2e_steps = max(3, min(args.steps, 50))

    def e2e_step(k: int) -> None:
        for m, o, i in cases:
            w = weights[(o, i)][k % copies[(o, i)]]
            b2.host_quantized_linear_forward(xs_pin[(m, i)], w, ys_pin[(m, o)], m)

    for k in range(3):
        e2e_step(k)
    barrier()
    t0 = time.perf_counter()
    for k in range(e2e_steps):
        e2e_step(k)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e = {"value": STEP_BYTES * world * e2e_steps / e2e_s / 1e9, "unit": UNIT,
           "h2d_bytes_per_step": sum(4 * m * i for m, _, i in cases),
           "d2h_bytes_per_step": sum(4 * m * o for m, o, _ in cases), "steps": e2e_steps}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        host_w = {}
        import oracle
        for (o, i), lst in weights.items():
            p = synth.host_payload(lst[0])
            host_w[(o, i)] = oracle.Nf4Weight(p.codes, o, i, BLOCK, scale_codes=p.scale_codes,
                                              second_level=p.second_level, scale_block_size=SCALE_BLOCK,
                                              offset=p.offset)
        xs_host = {k: v.cpu().numpy() for k, v in xs.items()}
        sample = [(m, o, i) for m in (1, 4) for o, i in LAYERS]
        sec, kind, workers = cpu_sweep(host_w, xs_host, sample, False)
        cpu_baseline = {"value": sum(packed_bytes(o, i) for _, o, i in sample) / sec / 1e9, "unit": UNIT,
                        "cores": workers, "kind": kind,
                        "sample": "one pass of the M in {1,4} cases on all three layers (6 of the 9 launches of a step)"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 mma, f32 accumulate", "data": "synthetic",
            "config": {"workload": "nf4_gemv_decode_sweep", "layers": LAYERS, "batches": BATCHES,
                       "block_size": BLOCK, "scale_block_size": SCALE_BLOCK, "scales": "double_quantized_u8",
                       "l2": "each step reads a different resident weight instance; instances per layer total > 2x L2"},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "clocks": clocks,
            "gpu_launches": launches_per_step * args.steps,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
