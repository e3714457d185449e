"""Cases of the persistent decode-batch linear kernel (1..32 activation rows), shared by the
in-process GPU tests and by the worker that runs them with the kernel forced for every batch
size. Each case is checked against the FP32 CPU oracle through the C ABI."""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

# rows, [out features of the weights applied to one input], in, block, double-quantised
CASES = [
    (32, [4096], 4096, 64, True),            # 32 tiles x 16 rounds over all SMs: every tile is split
    (17, [512], 4096, 64, True),             # 4 tiles, 64 items: fewer CTAs than SMs
    (32, [14336], 4096, 64, True),           # whole tiles and split tiles in one launch
    (32, [4096], 14336, 64, True),           # long contraction, second-level groups straddle rows
    (23, [1000], 1024, 64, True),            # four rounds per tile, ragged last tile
    (32, [640, 128, 136], 1024, 64, True),   # three weights of one input (q / k / v style), ragged tiles
    (32, [4096, 1024, 1024], 4096, 64, True),
    (20, [768], 1024, 128, False),           # FP32 scales, block 128
    (32, [256], 4096, 256, True),            # block 256: four k-blocks share a scale
    (32, [384], 768, 64, False),             # FP32 scales, block 64, three rounds
    (19, [200], 512, 64, False),             # the shortest width taken: two rounds
]
SMALL_ROW_CASES = [
    (1, [4096], 4096, 64, True),
    (4, [14336], 4096, 64, True),
    (16, [4096], 14336, 64, True),
    (9, [1000], 1024, 64, True),
    (5, [640, 128], 512, 64, False),
    (16, [300], 2048, 128, True),
]


def rel_l2(a, e):
    a = np.asarray(a, np.float64)
    e = np.asarray(e, np.float64)
    return float(np.linalg.norm(a - e) / max(np.linalg.norm(e), 1e-30))


def run_case(b2, port, case, tol, shard=None):
    """Runs one case through b2_nf4_linear_forward(_multi) and checks every row."""
    from riftco_transformer_b200 import _lib
    from riftco_transformer_b200._lib import lib
    from riftco_transformer_b200.backend import _check
    rows, outs, in_f, block, dq = case
    rng = np.random.default_rng(rows * 131 + sum(outs) + in_f)
    hosts, weights = [], []
    for o in outs:
        W = (rng.standard_normal((o, in_f)) * 0.02).astype(np.float32)
        hosts.append(port.quantize_nf4_double_quantized(W, block, 256) if dq else port.quantize_nf4(W, block))
        weights.append(b2.PackedNf4Weight.from_host(hosts[-1]))
    x = rng.standard_normal((rows, in_f)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    from conftest import Guarded
    guards = [Guarded((rows, w.out_features)) for w in weights]   # NaN-filled, with guard bands around
    ys = [g.tensor for g in guards]
    structs = (_lib.Nf4WeightStruct * len(weights))(*[w.struct() for w in weights])
    ptrs = (C.c_void_p * len(weights))(*[y.data_ptr() for y in ys])
    for _ in range(2):   # twice: the arrival counters must be back at zero after a launch
        if len(weights) == 1:
            _check(lib.b2_nf4_linear_forward(C.byref(structs[0]), xd.data_ptr(), ys[0].data_ptr(), rows, None, 0, None))
        else:
            _check(lib.b2_nf4_linear_forward_multi(structs, len(weights), xd.data_ptr(), ptrs, rows, None, 0, None))
        assert lib.b2_last_route() == 1, (case, lib.b2_last_route())   # B2_ROUTE_DECODE_TMEM
        b2.check_device_errors()
        for g in guards:
            g.check()
        for host, y in zip(hosts, ys):
            got = y.cpu().numpy()
            want = port.linear_forward(host, x)
            assert np.isfinite(got).all(), case
            assert rel_l2(got, want) <= tol, (case, rel_l2(got, want))
            for r in range(rows):
                assert rel_l2(got[r], want[r]) <= 2 * tol, (case, r, rel_l2(got[r], want[r]))
    return [y.cpu().numpy() for y in ys]
