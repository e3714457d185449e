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
4096->4096, 4096->14336, 14336->4096, both scale encodings), the four batch-32
linears of one decoder layer, paged GQA decode attention on 64 sequences of
length U[512, 8192] - each as achieved HBM GB/s of its algorithmic bytes against
the measured copy bandwidth - and the prefill GEMM / QLoRA input-backward of the
baseline (M = 4096, both layers, both encodings) as TFLOP/s against the measured
dense bf16 peak.

Prints ONE JSON line (rank 0).

    python bench.py --only linear --rows 32 --out 14336 --inp 4096 --launches 3
    python bench.py --only attention --seqs 8 --context 4096 --launches 3

run a few launches of one kernel on synthetic data and print their mean device
time (for profilers and quick checks; not the JSON line).
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
        weights.append(port.double_quantize_payload(codes, scales, o, i, BLOCK, SCALE_BLOCK))
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


def cpu_full_cases() -> dict:
    """The reference's CPU loops on the baseline's kernel-level configurations that finish in
    seconds, run IN FULL on one thread: config 1 (X[64,512] x W[1024,512], FP32 scales), the
    M = 1 case of config 2 on all three layers (double-quantised scales) and one config-4
    sequence (context 4352 = the mean of U[512, 8192], 32 query / 8 KV heads)."""
    import numpy as np
    import oracle

    impl = oracle.ref() if oracle.ref_available() else oracle.port()
    port = oracle.port()
    rng = np.random.default_rng(4242)
    out = {"kind": impl.kind, "threads": 1}
    W = (rng.standard_normal((1024, 512)) * 0.02).astype(np.float32)
    w1 = port.quantize_nf4(W, 64)
    x1 = rng.standard_normal((64, 512)).astype(np.float32)
    t0 = time.perf_counter()
    impl.linear_forward(w1, x1, threads=1)
    out["c1_64x512_to_1024_ms"] = round(1e3 * (time.perf_counter() - t0), 3)
    for o, i in LAYERS:
        n = o * i
        blocks = n // BLOCK
        codes = rng.integers(0, 256, n // 2, dtype=np.uint8)
        scales = np.maximum(0.0479 + 0.0066 * rng.standard_normal(blocks), 0.02).astype(np.float32)
        w = port.double_quantize_payload(codes, scales, o, i, BLOCK, SCALE_BLOCK)
        x = rng.standard_normal((1, i)).astype(np.float32)
        t0 = time.perf_counter()
        impl.linear_forward(w, x, threads=1)
        out[f"c2_M1_{i}to{o}_ms"] = round(1e3 * (time.perf_counter() - t0), 3)
    seq = 4352
    pages = -(-seq // 16)
    k = rng.standard_normal((pages, 8, 16, 128)).astype(np.float32)
    v = rng.standard_normal((pages, 8, 16, 128)).astype(np.float32)
    table = rng.permutation(pages).astype(np.uint32)
    q = rng.standard_normal((1, 32, 128)).astype(np.float32)
    t0 = time.perf_counter()
    impl.paged_decode_gqa(q, k, v, table[None, :], np.array([seq], np.uint32), threads=1)
    out["c4_one_sequence_ctx4352_ms"] = round(1e3 * (time.perf_counter() - t0), 3)
    return out


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
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "extrapolated": True,
                         "sample": "per step: one layer (7 packed linears + paged attention) of one sequence at "
                                   "context 2049, on every host thread concurrently; scaled by 32 layers + LM head"},
        "extrapolated": True,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# dram__bytes_read.sum / algorithmic K+V bytes in an ncu capture of the bulk attention kernel (8 sequences x 4096)
NCU_ATTENTION_READ_RATIO = 1.0007


def workload_config(world: int) -> dict:
    return {"workload": "7b_decode_step", "layers": N_LAYERS, "d_model": 4096, "q_heads": 32, "kv_heads": 8,
            "head_dim": 128, "ffn": 14336, "vocab": 32000, "batch": BATCH, "context": CONTEXT,
            "weights": "N(0, 0.02^2) quantised to nf4 block 64, double-quantised scales (u8 + f32 per 256); every "
                       "rank shards the same global payload by output rows", "kv": "f32 pages of 16",
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


def scale_payload_bytes(out_f: int, in_f: int, double_quantized: bool) -> int:
    blocks = out_f * in_f // BLOCK
    return blocks + 4 * (-(-blocks // SCALE_BLOCK)) + 4 if double_quantized else 4 * blocks


def kernel_measurements(torch, b2, synth, peaks, device_index: int) -> dict:
    """Per-kernel rooflines on the baseline's kernel-level configurations (N = 1 only)."""
    import ctypes as C

    import numpy as np
    from riftco_transformer_b200 import _lib
    from riftco_transformer_b200._lib import lib
    from riftco_transformer_b200.backend import _check, _stream_ptr
    out = {}
    g = torch.Generator(device="cuda")
    g.manual_seed(5678)

    # ---- config 2: NF4 GEMV decode sweep; enough resident instances per layer to exceed 2x L2 ----
    sweep = {}
    for dq in (True, False):
        for li, (o, i) in enumerate(LAYERS):
            algorithmic = o * i // 2 + scale_payload_bytes(o, i, dq)
            n_copies = max(3, -(-2 * L2_BYTES // algorithmic))
            ws = [synth.packed_weight(o, i, seed=4321 + 97 * li + c, double_quantized=dq) for c in range(n_copies)]
            for m in BATCHES:
                x = torch.randn((m, i), device="cuda", generator=g)
                y = torch.empty((m, o), device="cuda")

                def launch(ws=ws, x=x, y=y, m=m, i=i, o=o):
                    for w in ws:
                        b2.dispatch_quantized_linear_forward(x, w, y, (m, i, o, BLOCK))

                us = time_graph(torch, launch, 20, n_copies)
                gbps = algorithmic / us / 1e3
                sweep[f"M{m}_{i}to{o}_{'dq' if dq else 'f32'}"] = {
                    "us": round(us, 3), "gbps": round(gbps, 1), "frac": round(gbps / peaks["hbm_gbs"], 4),
                    "route": b2.last_route()}
            del ws
    out["nf4_gemv_sweep"] = {"kernel": "nf4_gemv_tma_kernel (route gemv_tma) / nf4_decode_tmem_kernel<half> with its "
                                       "fp32 -> fp16 pre-pass (route decode_tmem), per case", "bound": "hbm", "unit": "GB/s",
                             "bytes": "packed codes + scale payload per launch (dq: u8 scale codes + f32 per 256 "
                                      "blocks; f32: one f32 scale per block)", "cases": sweep}

    # ---- the four batch-32 linears of one decoder layer, as the decode step issues them ----
    groups = {"q+k+v": [(4096, 4096), (1024, 4096), (1024, 4096)], "o": [(4096, 4096)],
              "gate+up": [(14336, 4096), (14336, 4096)], "down": [(4096, 14336)]}
    b32 = {}
    for name, shapes in groups.items():
        algorithmic = sum(o * i // 2 + scale_payload_bytes(o, i, True) for o, i in shapes)
        n_sets = max(3, -(-2 * L2_BYTES // algorithmic))
        sets = [[synth.packed_weight(o, i, seed=911 + 13 * s + j) for j, (o, i) in enumerate(shapes)]
                for s in range(n_sets)]
        x16 = torch.randn((BATCH, shapes[0][1]), device="cuda", generator=g).to(torch.bfloat16)
        ys = [torch.empty((BATCH, o), device="cuda") for o, _ in shapes]
        ptrs = (C.c_void_p * len(ys))(*[y.data_ptr() for y in ys])
        structs = [(_lib.Nf4WeightStruct * len(ws))(*[w.struct() for w in ws]) for ws in sets]

        def launch(structs=structs, n=len(ys), x16=x16, ptrs=ptrs):
            for st in structs:
                _check(lib.b2_nf4_linear_forward_multi_bf16(st, n, x16.data_ptr(), ptrs, BATCH, _stream_ptr(None)))

        us = time_graph(torch, launch, 10, n_sets)
        gbps = algorithmic / us / 1e3
        b32[name] = {"us": round(us, 3), "bytes": algorithmic, "gbps": round(gbps, 1),
                     "frac": round(gbps / peaks["hbm_gbs"], 4)}
        del sets, structs
    out["nf4_linear_b32"] = {"kernel": "nf4_decode_tmem_kernel", "bound": "hbm", "unit": "GB/s", "rows": BATCH,
                             "input": "bf16 activations handed over by the producing kernel, one launch per group",
                             "cases": b32}

    # ---- config 3: prefill GEMM and QLoRA input-backward, M = 4096, both layers, both encodings ----
    rows = 4096
    c3 = {}
    with ClockSampler(device_index) as sampler:
        for o, i in [(14336, 4096), (4096, 14336)]:
            x = torch.randn((rows, i), device="cuda", generator=g)
            dy = torch.randn((rows, o), device="cuda", generator=g) * 0.01
            y = torch.empty((rows, o), device="cuda")
            dx = torch.empty((rows, i), device="cuda")
            for dq in (True, False):
                w = synth.packed_weight(o, i, seed=31337 + o, double_quantized=dq)
                dims = (rows, i, o, BLOCK)
                for kind, fn in (("forward", lambda: b2.dispatch_quantized_linear_forward(x, w, y, dims)),
                                 ("input_backward", lambda: b2.dispatch_quantized_linear_input_backward(dy, w, dx, dims))):
                    us = min(time_graph(torch, fn, 5, 1) for _ in range(3))   # activations + output exceed L2
                    tflops = 2.0 * rows * o * i / us / 1e6
                    c3[f"{kind}_{i}to{o}_{'dq' if dq else 'f32'}"] = {
                        "us": round(us, 1), "tflops": round(tflops, 1),
                        "frac": round(tflops / peaks["bf16_tflops"], 4)}
            del x, dy, y, dx
        torch.cuda.synchronize()
    out["nf4_gemm_c3"] = {"kernel": "nf4_gemm_tmem_kernel (forward), nf4_dequant_transpose + bf16_gemm (input-backward)",
                          "bound": "tensor", "unit": "TFLOP/s", "rows": rows, "peak": peaks["bf16_tflops"],
                          "peak_kind": "dense bf16, burst", "flops": "2 * rows * out * in per call",
                          "clocks": sampler.summary(), "cases": c3}

    # ---- config 4: paged GQA decode attention, 64 sequences, context U[512, 8192] ----
    lens = np.random.default_rng(91011).integers(512, 8193, size=64)
    pool, tables, dlens = synth.paged_cache(lens, 8)
    q = torch.randn((64, 32, 128), device="cuda", generator=g)
    ctx = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    mx = int(lens.max())
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


# ---- single-kernel runs for profilers --------------------------------------------------------------

def probe_linear(args) -> None:
    """`--launches` calls of the packed-NF4 linear, each on its own weight instance."""
    import torch

    import riftco_transformer_b200 as b2
    from riftco_transformer_b200 import synth
    rows, out_f, in_f = args.rows, args.out, args.inp
    weights = [synth.packed_weight(out_f, in_f, seed=1000 + i, double_quantized=not args.fp32_scales)
               for i in range(args.launches)]
    shape = (rows, in_f, out_f, weights[0].block_size)
    if args.backward:   # dX[rows, in] = dY[rows, out] * W
        x = torch.randn((rows, out_f), device="cuda") * 0.01
        y = torch.empty((rows, in_f), device="cuda")
        call = b2.dispatch_quantized_linear_input_backward
    else:               # Y[rows, out] = X[rows, in] * W^T
        x = torch.randn((rows, in_f), device="cuda")
        y = torch.empty((rows, out_f), device="cuda")
        call = b2.dispatch_quantized_linear_forward
    call(x, weights[0], y, shape)   # library set-up outside the timed launches
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for w in weights:
        call(x, w, y, shape)
    stop.record()
    torch.cuda.synchronize()
    b2.check_device_errors()
    us = start.elapsed_time(stop) * 1e3 / args.launches
    payload = weights[0].resident_payload_bytes()
    print(f"linear {'input-backward' if args.backward else 'forward'} rows={rows} {in_f}->{out_f}: {us:.2f} us/launch "
          f"(eager, launch gaps included), {payload} B of packed weight per launch = {payload / us / 1e3:.1f} GB/s, "
          f"{2.0 * rows * out_f * in_f / us / 1e6:.1f} TFLOP/s")


def probe_attention(args) -> None:
    """`--launches` calls of paged decode attention for a batch on its own KV pool."""
    import torch

    import riftco_transformer_b200 as b2
    from riftco_transformer_b200 import synth
    pool, tables, lens = synth.paged_cache([args.context] * args.seqs, args.kv_heads, 128, 16, seed=7)
    q = torch.randn((args.seqs, args.q_heads, 128), device="cuda")
    ctx = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    b2.paged_decode_attention(q, pool, tables, lens, ctx, args.context, status=status)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.launches):
        b2.paged_decode_attention(q, pool, tables, lens, ctx, args.context, status=status)
    stop.record()
    torch.cuda.synchronize()
    b2.check_device_errors()
    us = start.elapsed_time(stop) * 1e3 / args.launches
    kv_bytes = int(lens.sum().item()) * args.kv_heads * 128 * 4 * 2
    print(f"attention seqs={args.seqs} context={args.context} heads={args.q_heads}/{args.kv_heads}: "
          f"{us:.2f} us/launch, {kv_bytes} B of K/V per launch = {kv_bytes / us / 1e3:.1f} GB/s, "
          f"status {int(status.item())}")


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
    # B2_SHARD_ALL=1 row-shards the o- and down-projections too (four gathers per layer instead of two).
    whole = () if os.environ.get("B2_SHARD_ALL") == "1" else None
    step, inputs = synthetic_step(cfg, BATCH, CONTEXT, rank, world, device, group, whole=whole)
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
    # DRAM traffic per launch: an ncu capture of a smaller case of this kernel (8 sequences x 4096
    # tokens) read 1.0007 x its algorithmic K/V bytes and wrote its split partials and context; both
    # scale with the tokens read, so they are scaled to this launch.
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

    # Correctness witness. The synthetic model is a function of the seed alone (every rank shards the
    # same global payload), so the step's next tokens and logits can be compared across world sizes:
    # the line carries a CRC of the next tokens, and with more than one rank, rank 0 rebuilds the whole
    # model on its own GPU, runs the step unsharded and compares (token ids must agree; logits differ
    # only by the order of FP32 partial sums, which depends on how many tiles a shard has).
    # The tensor-core linears round their operands to bf16, so a difference in the ORDER of FP32
    # partial sums (which depends on how many tiles a shard has) can flip a rounding by one bf16 ulp;
    # through 32 layers of a random model that grows to ~2e-2 in the logits - the same figure two
    # single-GPU kernels with different summation order give. The comparison is therefore made
    # twice: after ONE layer, where it is tight, and at full depth.
    import zlib

    def logits_after(the_step, the_inputs, layers):
        the_step.active_layers = layers
        tok, lg = the_step.step(the_inputs["tokens"], the_inputs["positions"], the_inputs["seq_lens"])
        torch.cuda.synchronize()
        the_step.active_layers = cfg.layers
        return tok.clone(), lg.clone()

    tokens_n, logits_n = logits_after(step, inputs, cfg.layers)
    check = {"next_tokens_crc32": zlib.crc32(tokens_n.cpu().numpy().tobytes())}
    if world > 1:
        _, logits_n1 = logits_after(step, inputs, 1)
        barrier()
        if rank == 0:
            single, single_in = synthetic_step(cfg, BATCH, CONTEXT, 0, 1, device, None)
            _, logits_11 = logits_after(single, single_in, 1)
            tok1, logits1 = logits_after(single, single_in, cfg.layers)

            def rel(a, b):
                return float(((a.double() - b.double()).norm() / b.double().norm()).item())

            check.update({"single_gpu_next_tokens_crc32": zlib.crc32(tok1.cpu().numpy().tobytes()),
                          "tokens_equal_single_gpu_fraction": float((tok1 == tokens_n).float().mean().item()),
                          "logits_rel_l2_vs_single_gpu_after_1_layer": rel(logits_n1, logits_11),
                          "logits_rel_l2_vs_single_gpu": rel(logits_n, logits1),
                          "note": "bf16 operand rounding amplifies FP32 summation-order differences with depth; "
                                  "two single-GPU kernels that differ only in summation order are 1.7e-2 apart at 32 layers"})
            del single, single_in, tok1, logits1, logits_11
            torch.cuda.empty_cache()
        barrier()

    kernels = None
    cpu_baseline = None
    if rank == 0 and world == 1:
        del graph
        if not args.no_kernels:
            kernels = kernel_measurements(torch, b2, synth, peaks, local_rank)
        if not args.no_cpu_baseline:
            sec, kind = cpu_layer_seconds(cpu_layer_sample())
            cpu_baseline = {"value": 1.0 / (sec * LAYER_EQUIVALENTS), "unit": UNIT, "cores": 1, "kind": kind,
                            "extrapolated": True,
                            "sample": "one layer (7 packed linears + paged attention) of one sequence at context "
                                      "2049 on one thread, scaled by 32 layers + LM head",
                            "full_cases": cpu_full_cases()}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32 (batch-32 linears: bf16 tcgen05 operands, f32 accumulate; the GEMV sweep: f16 operands, f32 accumulate)",
            "data": "synthetic", "config": workload_config(world), "roofline": roofline,
            "step_roofline": step_roofline, "check": check, "kernels": kernels, "cpu_baseline": cpu_baseline,
            "e2e": e2e,
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
    ap.add_argument("--only", default="all", choices=["all", "linear", "attention"],
                    help="linear / attention: a few launches of one kernel (for profilers), no JSON line")
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--out", type=int, default=14336)
    ap.add_argument("--inp", type=int, default=4096)
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--fp32-scales", action="store_true")
    ap.add_argument("--backward", action="store_true", help="--only linear: the input-backward dX = dY * W")
    ap.add_argument("--seqs", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--q-heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    args = ap.parse_args()
    if args.only != "all":
        import riftco_transformer_b200 as b2
        if not b2.is_available():
            raise SystemExit("riftco_b200: " + b2.unavailability_reason())
        (probe_linear if args.only == "linear" else probe_attention)(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
