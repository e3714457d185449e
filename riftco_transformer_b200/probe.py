"""Small, self-contained launches of the library's hot kernels on synthetic data,
for profilers and quick timing:

    python -m riftco_transformer_b200.probe linear --rows 1 --out 14336 --inp 4096 --launches 4
    python -m riftco_transformer_b200.probe linear --rows 4096 --backward --launches 2
    python -m riftco_transformer_b200.probe attention --seqs 8 --context 4096 --launches 3

``linear`` runs ``--launches`` calls of the packed-NF4 forward, each on its own
weight instance (so no launch finds its weights in L2); ``attention`` runs the
paged decode attention of a batch on its own KV pool. Both print the mean device
time per launch (CUDA events) and the algorithmic bytes, and check the library's
device error words. Sizes default to a few hundred MB so a profiler capture ends
in seconds.
"""
from __future__ import annotations

import argparse

import torch


def _events():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def probe_linear(args) -> None:
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
    start, stop = _events()
    start.record()
    for w in weights:
        call(x, w, y, shape)
    stop.record()
    torch.cuda.synchronize()
    b2.check_device_errors()
    us = start.elapsed_time(stop) * 1e3 / args.launches
    payload = weights[0].resident_payload_bytes()
    print(f"linear {'input-backward' if args.backward else 'forward'} rows={rows} {in_f}->{out_f}: {us:.2f} us/launch (eager, launch gaps included), "
          f"{payload} B of packed weight per launch = {payload / us / 1e3:.1f} GB/s, "
          f"{2.0 * rows * out_f * in_f / us / 1e6:.1f} TFLOP/s")


def probe_attention(args) -> None:
    import riftco_transformer_b200 as b2
    from riftco_transformer_b200 import synth
    pool, tables, lens = synth.paged_cache([args.context] * args.seqs, args.kv_heads, 128, 16, seed=7)
    q = torch.randn((args.seqs, args.q_heads, 128), device="cuda")
    ctx = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    b2.paged_decode_attention(q, pool, tables, lens, ctx, args.context, status=status)
    torch.cuda.synchronize()
    start, stop = _events()
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


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="what", required=True)
    lin = sub.add_parser("linear")
    lin.add_argument("--rows", type=int, default=1)
    lin.add_argument("--out", type=int, default=14336)
    lin.add_argument("--inp", type=int, default=4096)
    lin.add_argument("--launches", type=int, default=4)
    lin.add_argument("--fp32-scales", action="store_true")
    lin.add_argument("--backward", action="store_true", help="time the input-backward dX = dY * W instead")
    lin.set_defaults(fn=probe_linear)
    att = sub.add_parser("attention")
    att.add_argument("--seqs", type=int, default=8)
    att.add_argument("--context", type=int, default=4096)
    att.add_argument("--q-heads", type=int, default=32)
    att.add_argument("--kv-heads", type=int, default=8)
    att.add_argument("--launches", type=int, default=3)
    att.set_defaults(fn=probe_attention)
    args = ap.parse_args()
    import riftco_transformer_b200 as b2
    if not b2.is_available():
        raise SystemExit("riftco_b200: " + b2.unavailability_reason())
    args.fn(args)


if __name__ == "__main__":
    main()
