#!/usr/bin/env python
"""Benchmark of the NF4-linear + paged-decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Workload (`config.workload`): one full decode step of a 7B-shaped decoder-only
Transformer with random-init weights - 32 layers, d_model 4096, 32 query / 8 KV
heads of width 128, SwiGLU FFN 14336, RMSNorm, RoPE, vocab 32000, every linear
packed NF4 (block 64, double-quantised absmax), batch 32 at context 2048, FP32
paged KV cache (page 16) - sharded by output rows / KV heads over N GPUs with
NCCL all-gathers at the layer boundaries. `value` is decoded tokens per second
of the whole job. One step reads ~21 GB (3.7 GB of packed weights, 17 GB of KV),
far more than L2, so no flush is needed between steps.

At N = 1 the line also carries the per-kernel measurements the headline is made
of (`kernels`): the NF4 GEMV decode sweep of the baseline (M in {1,4,16} on
4096->4096, 4096->14336, 14336->4096) and paged GQA decode attention on 64
sequences of length U[512, 8192], each as achieved HBM GB/s of its algorithmic
bytes against the measured copy bandwidth.

Prints ONE JSON line (rank 0).
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
METRIC = "nf4_7b_decode_tokens_per_second"
UNIT = "tokens/s"
BATCH, CONTEXT = 32, 2048


def packed_bytes(out_f: int, in_f: int) -> int:
    """Algorithmic bytes of one launch: codes + double-quantised scale payload."""
    n = out_f * in_f
    blocks = -(-n // BLOCK)
    return (n + 1) // 2 + blocks + 4 * (-(-blocks // SCALE_BLOCK)) + 4




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



# ---- CPU side: the reference's own loops on a bounded sample -------------------------------

LAYER_LINEARS = [(4096, 4096), (1024, 4096), (1024, 4096), (4096, 4096), (14336, 4096), (14336, 4096),
                 (4096, 14336)]  # q, k, v, o, gate, up, down as (out, in)
LM_HEAD = (32000, 4096)
N_LAYERS = 32
WEIGHTS_PER_LAYER = sum(o * i for o, i in LAYER_LINEARS)
# one token's cost in units of "one layer of one sequence": 32 layers + the LM head's share
LAYER_EQUIVALENTS = N_LAYERS + LM_HEAD[0] * LM_HEAD[1] / WEIGHTS_PER_LAYER


def cpu_layer_sample():
    """Host payloads and inputs of ONE layer for ONE sequence at context 2049
    (synthetic, same distributions as the GPU arm)."""
    import ctypes as C

    import numpy as np
    import oracle  # checker only; never on the product path

    rng = np.random.default_rng(1234)
    port = oracle.port()
    weights = []
    for o, i in LAYER_LINEARS:
        n = o * i
        blocks = n // BLOCK
        codes = rng.integers(0, 256, n // 2, dtype=np.uint8)
        scales = np.maximum(0.0479 + 0.0066 * rng.standard_normal(blocks), 0.02).astype(np.float32)
        qs = np.zeros(blocks, np.uint8)
        second = np.zeros(-(-blocks // SCALE_BLOCK), np.float32)
        off = C.c_float(0)
        port.lib.orc_double_quantize_scales(oracle._ptr(scales, oracle._f32p), blocks, SCALE_BLOCK,
                                            oracle._ptr(qs, oracle._u8p), oracle._ptr(second, oracle._f32p),
                                            C.byref(off))
        weights.append(oracle.Nf4Weight(codes, o, i, BLOCK, scale_codes=qs, second_level=second,
                                        scale_block_size=SCALE_BLOCK, offset=float(off.value)))
    seq = CONTEXT + 1
    pages = -(-seq // 16)
    k = rng.standard_normal((pages, 8, 16, 128)).astype(np.float32)
    v = rng.standard_normal((pages, 8, 16, 128)).astype(np.float32)
    table = rng.permutation(pages).astype(np.uint32)
    q = rng.standard_normal((1, 32, 128)).astype(np.float32)
    xs = [rng.standard_normal((1, i)).astype(np.float32) for _, i in LAYER_LINEARS]
    return weights, xs, (q, k, v, table, seq)


def cpu_layer_seconds(sample) -> tuple[float, str]:
    """Seconds the reference's CPU loops take for the sample (one thread)."""
    import numpy as np
    import oracle

    weights, xs, (q, k, v, table, seq) = sample
    impl = oracle.ref() if oracle.ref_available() else oracle.port()
    t0 = time.perf_counter()
    for w, x in zip(weights, xs):
        impl.linear_forward(w, x, threads=1)
    impl.paged_decode_gqa(q, k, v, table[None, :], np.array([seq], np.uint32), threads=1)
    return time.perf_counter() - t0, impl.kind


def run_reference(args) -> None:
    """The reference's CPU implementation of the decode step's operators on the
    host cores. Each step is a bounded sample - one layer's seven packed linears
    and its paged attention for ONE sequence at context 2049 - run concurrently
    for as many independent sequences as there are host threads; tokens/s scales
    it to a full token (32 layers + LM head)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import oracle

    threads = oracle.host_threads()
    sample = cpu_layer_sample()
    steps = max(1, min(args.steps, 3))
    warm = 1 if args.warmup > 0 else 0
    kind = "port"

    def one_step() -> float:
        nonlocal kind
        t0 = time.perf_counter()
        with ThreadPoolExecutor(threads) as pool:
            kinds = list(pool.map(lambda _: cpu_layer_seconds(sample)[1], range(threads)))
        kind = kinds[0]
        return time.perf_counter() - t0

    for _ in range(warm):
        one_step()
    total = sum(one_step() for _ in range(steps))
    sec_per_layer_seq = total / steps / threads          # aggregate over the concurrent sequences
    value = 1.0 / (sec_per_layer_seq * LAYER_EQUIVALENTS)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": 1e3 * total / steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind,
                         "sample": "per step: one layer (7 packed linears + paged attention) of one sequence at "
                                   "context 2049, on every host thread concurrently; scaled by 32 layers + LM head"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


NCU_ATTENTION_READ_RATIO = 1.0007   # dram__bytes_read.sum / algorithmic bytes, profiles/paged_decode_bulk_8x4096.md


def workload_config(world: int) -> dict:
    return {"workload": "7b_decode_step", "layers": N_LAYERS, "d_model": 4096, "q_heads": 32, "kv_heads": 8,
            "head_dim": 128, "ffn": 14336, "vocab": 32000, "batch": BATCH, "context": CONTEXT,
            "weights": "nf4 block 64, double-quantised scales (u8 + f32 per 256)", "kv": "f32 pages of 16",
            "sharding": f"output rows / kv heads over {world} gpu(s); activations joined at layer boundaries by the "
                        "library's peer-store all-gather kernel over NVLink (B2_PEER_GATHER=0: NCCL all-gather)",
            "l2": "each step reads ~21 GB of weights and KV, far larger than L2"}


# ---- B200 arm ------------------------------------------------------------------------------------

def time_graph(torch, fn, reps: int, inner: int) -> float:
    """Mean microseconds per launch of `fn` (which enqueues `inner` launches),
    replayed from a CUDA graph so that launches are back to back."""
    side = torch.cuda.Stream()
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            fn()
    torch.cuda.synchronize()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        g.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / (reps * inner)


def kernel_measurements(torch, b2, synth, peaks) -> dict:
    """Per-kernel HBM rooflines on the baseline's kernel-level configurations."""
    import numpy as np
    out = {}
    # NF4 GEMV decode sweep: enough resident instances per layer to exceed 2x L2.
    g = torch.Generator(device="cuda")
    g.manual_seed(5678)
    sweep = {}
    for li, (o, i) in enumerate(LAYERS):
        n_copies = max(3, -(-2 * L2_BYTES // packed_bytes(o, i)))
        ws = [synth.packed_weight(o, i, seed=4321 + 97 * li + c) for c in range(n_copies)]
        for m in BATCHES:
            x = torch.randn((m, i), device="cuda", generator=g)
            y = torch.empty((m, o), device="cuda")

            def launch(ws=ws, x=x, y=y, m=m, i=i, o=o):
                for w in ws:
                    b2.dispatch_quantized_linear_forward(x, w, y, (m, i, o, BLOCK))

            us = time_graph(torch, launch, 20, n_copies)
            gbps = packed_bytes(o, i) / us / 1e3
            sweep[f"M{m}_{i}to{o}"] = {"us": round(us, 3), "gbps": round(gbps, 1),
                                       "frac": round(gbps / peaks["hbm_gbs"], 4)}
        del ws
    out["nf4_gemv_sweep"] = {"kernel": "nf4_gemv_tma_kernel", "bound": "hbm", "unit": "GB/s",
                             "bytes": "packed codes + scale payload per launch", "cases": sweep}
    # Paged GQA decode attention: 64 sequences, context U[512, 8192].
    lens = np.random.default_rng(91011).integers(512, 8193, size=64)
    pool, tables, dlens = synth.paged_cache(lens, 8)
    q = torch.randn((64, 32, 128), device="cuda", generator=g)
    ctx = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    mx = int(lens.max())
    from riftco_transformer_b200._lib import lib
    ws = torch.empty(max(lib.b2_paged_decode_workspace_bytes(64, 32, 128, 16, mx), 16), dtype=torch.uint8,
                     device="cuda")
    us = time_graph(torch, lambda: b2.paged_decode_attention(q, pool, tables, dlens, ctx, mx, status=status,
                                                             workspace=ws), 10, 1)
    kv_bytes = int(lens.sum()) * 8 * 128 * 4 * 2
    out["paged_decode_c4"] = {"kernel": "paged_decode_bulk_kernel(+merge)", "bound": "hbm", "unit": "GB/s",
                              "us": round(us, 1), "kv_bytes": kv_bytes, "gbps": round(kv_bytes / us / 1e3, 1),
                              "frac": round(kv_bytes / us / 1e3 / peaks["hbm_gbs"], 4),
                              "status": int(status.item())}
    return out


def run_b200(args) -> None:
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        group = dist.group.WORLD

    import riftco_transformer_b200 as b2
    from riftco_transformer_b200 import synth
    from riftco_transformer_b200.decode import DecoderConfig, synthetic_step

    if not b2.is_available():
        raise SystemExit("riftco_b200: " + b2.unavailability_reason())
    peaks, peak_kind = measured_peaks()

    cfg = DecoderConfig()
    step, inputs = synthetic_step(cfg, BATCH, CONTEXT, rank, world, device, group)
    tokens, positions, seq_lens = inputs["tokens"], inputs["positions"], inputs["seq_lens"]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # Warm up eagerly (library set-up, NCCL channels), then capture the step in a graph.
    barrier()   # ranks finish building their shards at different times; the gathers wait only so long
    step.ops.launches = 0
    step.step(tokens, positions, seq_lens)
    launches_per_step = step.ops.launches
    barrier()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        step.step(tokens, positions, seq_lens)
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            step.step(tokens, positions, seq_lens)
    barrier()
    for _ in range(max(args.warmup, 3)):
        graph.replay()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as sampler:
        start.record()
        for _ in range(args.steps):
            graph.replay()
        stop.record()
        barrier()
        elapsed_ms = max_over_ranks(start.elapsed_time(stop))
        # Keep load on the GPU until the sampler has a few samples. Every rank must replay the step
        # the same number of times (each replay joins the peer all-gathers), so the count comes from
        # the reduced time, never from a local clock.
        extra = 0 if elapsed_ms >= 600.0 else int((600.0 - elapsed_ms) / (elapsed_ms / args.steps)) + 1
        for _ in range(extra):
            graph.replay()
        torch.cuda.synchronize()
    clocks = sampler.summary()
    # a bounded wait that ran out (barrier, peer all-gather) invalidates the measurement
    b2.check_device_errors()
    step.ops.check_peer_status()
    ms_per_step = elapsed_ms / args.steps
    value = BATCH / (ms_per_step / 1e3)

    # End to end: token ids from pinned host memory in, next token ids back to the host, every step.
    host_in = torch.stack([tokens.cpu(), positions.cpu(), seq_lens.cpu()]).pin_memory()
    host_out = torch.empty(BATCH, dtype=torch.int32).pin_memory()
    e2e_steps = max(3, min(args.steps, 20))

    def e2e_step():
        tokens.copy_(host_in[0], non_blocking=True)
        positions.copy_(host_in[1], non_blocking=True)
        seq_lens.copy_(host_in[2], non_blocking=True)
        graph.replay()
        host_out.copy_(step.next_tokens, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(2):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    e2e = {"value": BATCH * e2e_steps / e2e_s, "unit": UNIT, "h2d_bytes_per_step": 3 * BATCH * 4,
           "d2h_bytes_per_step": BATCH * 4, "steps": e2e_steps}

    # Dominant kernel of the step: paged decode attention (17 of the 21 GB). Timed on the step's own
    # 32 layer pools (distinct data, > L2) with CUDA events around back-to-back launches.
    def attention_all_layers():
        for layer in range(cfg.layers):
            step.ops.attention(step.q, step.pools[layer], step.tables, seq_lens, step.ctx_local,
                               step.max_seq_len, step.status, step.workspace)

    attn_us = max_over_ranks(time_graph(torch, attention_all_layers, 5, cfg.layers))
    kv_bytes_launch = inputs["kv_bytes_per_step"] / cfg.layers
    achieved = kv_bytes_launch / attn_us / 1e3
    # DRAM traffic per launch: the ncu capture of a smaller case of this kernel
    # (profiles/paged_decode_bulk_8x4096.md) read 1.0007 x its algorithmic K/V bytes and wrote its
    # split partials and context; both scale with the tokens read, so they are scaled to this launch.
    splits = -(-(CONTEXT + 1) // 256)
    hq_local = cfg.q_heads // world
    traffic = int(kv_bytes_launch * NCU_ATTENTION_READ_RATIO) + BATCH * hq_local * (splits * 130 + 128) * 4
    roofline = {"kernel": "paged_decode_bulk_kernel(+merge)", "bound": "hbm", "achieved": achieved,
                "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                "peak_source": peak_kind, "traffic": traffic, "us_per_launch": attn_us,
                "share_of_step": attn_us * cfg.layers / 1e3 / ms_per_step}
    step_bytes = step.weight_bytes() + inputs["kv_bytes_per_step"]
    step_roofline = {"bytes_per_step_per_gpu": step_bytes, "hbm_floor_ms": step_bytes / peaks["hbm_gbs"] / 1e6,
                     "frac": step_bytes / peaks["hbm_gbs"] / 1e6 / ms_per_step}

    b2.check_device_errors()
    step.ops.check_peer_status()
    if int(step.status.item()) != 0:
        raise SystemExit(f"decode step reported status bits {int(step.status.item())} (bad block table or token id)")

    kernels = None
    cpu_baseline = None
    if rank == 0 and world == 1:
        del graph
        if not args.no_kernels:
            kernels = kernel_measurements(torch, b2, synth, peaks)
        if not args.no_cpu_baseline:
            sec, kind = cpu_layer_seconds(cpu_layer_sample())
            cpu_baseline = {"value": 1.0 / (sec * LAYER_EQUIVALENTS), "unit": UNIT, "cores": 1, "kind": kind,
                            "sample": "one layer (7 packed linears + paged attention) of one sequence at context "
                                      "2049 on one thread, scaled by 32 layers + LM head"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32 (batch-32 linears: bf16 tcgen05 operands, f32 accumulate; the GEMV sweep: f16 mma.sync operands, f32 accumulate)",
            "data": "synthetic", "config": workload_config(world), "roofline": roofline,
            "step_roofline": step_roofline, "kernels": kernels, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "clocks": clocks, "gpu_launches": launches_per_step * args.steps,
        }
        print(json.dumps(line))
    if world > 1:
        # Tearing the NCCL group down while CUDA graphs that captured its collectives are alive hangs;
        # every rank has finished its work here, so leave without the teardown.
        sys.stdout.flush()
        dist.barrier()
        torch.cuda.synchronize()
        os._exit(0)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel sweep measurements")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
