"""Every kernel family the library can choose is reached by a shape, through the C ABI, and held
to the CPU oracle there. The library picks the kernel from the request alone; ``last_route``
says which one served the call, so a path cannot silently lose its coverage when the selection
rules change. Needs a B200."""
import numpy as np
import pytest
import torch

from conftest import rel_l2
from test_gpu_parity import backward, dev, forward, run_gqa

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def b2():
    import riftco_transformer_b200 as pkg
    assert pkg.is_available(), pkg.unavailability_reason()
    return pkg


def _weight(port, out_f, in_f, block, dq, seed):
    rng = np.random.default_rng(seed)
    W = (rng.standard_normal((out_f, in_f)) * 0.02).astype(np.float32)
    return port.quantize_nf4_double_quantized(W, block, 256) if dq else port.quantize_nf4(W, block)


# (route, rows, out, in, block, double-quantised, tolerance)
FORWARD = [
    ("decode_tmem", 32, 512, 1024, 64, True, 1e-2),    # bf16 operands on tcgen05
    ("decode_tmem", 17, 384, 512, 64, False, 1e-2),    # FP32 scales, ragged last 128-row tile
    ("decode_tmem", 12, 256, 8192, 64, True, 2e-3),    # 9..16 rows on a long contraction: the fp16 form
    ("gemv_tma", 8, 256, 8192, 64, True, 2e-3),        # ... up to 8 rows stay on mma.sync
    ("gemv_tma", 4, 4096, 4096, 64, True, 2e-3),       # fp16 operands on mma.sync
    ("gemv_tma", 16, 1024, 2048, 128, False, 2e-3),
    ("gemv_tile", 3, 1000, 192, 64, True, 2e-3),       # out_features no multiple of the TMA row tile
    ("gemv_tile", 9, 130, 2048 + 64, 64, False, 2e-3),
    ("gemm_tmem", 64, 512, 1024, 64, True, 1e-2),
    ("gemm_tmem", 24, 640, 192, 64, False, 1e-2),      # 17..32 rows, width no multiple of 256
    ("gemm_tmem", 32, 256, 512, 64, True, 1e-2),       # 8 scale codes per row: under one 16-byte TMA box
    ("generic", 5, 33, 96, 32, False, 1e-5),           # block size under 64: FP32 SIMT
    ("generic", 40, 7, 96, 32, True, 1e-5),
]


@pytest.mark.parametrize("route,rows,out_f,in_f,block,dq,tol", FORWARD)
def test_forward_routes(b2, port, route, rows, out_f, in_f, block, dq, tol):
    host = _weight(port, out_f, in_f, block, dq, out_f * 31 + in_f + rows)
    x = np.random.default_rng(rows).standard_normal((rows, in_f)).astype(np.float32)
    y = forward(b2, b2.PackedNf4Weight.from_host(host), dev(x))
    assert b2.last_route() == route
    want = port.linear_forward(host, x)
    assert rel_l2(y, want) <= tol
    for r in range(rows):
        assert rel_l2(y[r], want[r]) <= 2 * tol


@pytest.mark.parametrize("rows,route,tol", [(4, "gemv_tile", 2e-3), (20, "gemv_tile", 2e-3), (40, "generic", 1e-5)])
def test_codes_that_are_only_8_byte_aligned(b2, port, rows, route, tol):
    """The TMA-fed and tcgen05 kernels want 16-byte aligned codes; a weight placed at an address
    that is 8 modulo 16 is served by the kernels that read it with plain loads."""
    host = _weight(port, 512, 1024, 64, True, 99)
    w = b2.PackedNf4Weight.from_host(host)
    shifted = torch.empty(w.codes.numel() + 16, dtype=torch.uint8, device="cuda")
    shifted[8:8 + w.codes.numel()] = w.codes
    w.codes = shifted[8:8 + w.codes.numel()]
    assert w.codes.data_ptr() % 16 == 8
    x = np.random.default_rng(rows).standard_normal((rows, 1024)).astype(np.float32)
    y = forward(b2, w, dev(x))
    assert b2.last_route() == route
    assert rel_l2(y, port.linear_forward(host, x)) <= tol


BACKWARD = [
    ("backward_dense", 512, 768, 320, 64, True, 1e-2),
    ("gemm_smem", 64, 768, 320, 64, True, 1e-2),
    ("gemm_smem", 33, 128, 64, 64, False, 1e-2),
    ("generic", 19, 768, 320, 64, True, 1e-5),         # 32 rows or fewer
    ("generic", 600, 96, 64, 32, False, 1e-5),         # block size under 64
]


@pytest.mark.parametrize("route,rows,out_f,in_f,block,dq,tol", BACKWARD)
def test_input_backward_routes(b2, port, route, rows, out_f, in_f, block, dq, tol):
    host = _weight(port, out_f, in_f, block, dq, out_f * 17 + in_f + rows)
    dy = (np.random.default_rng(rows).standard_normal((rows, out_f)) * 0.01).astype(np.float32)
    dx = backward(b2, b2.PackedNf4Weight.from_host(host), dev(dy))
    assert b2.last_route() == route
    assert rel_l2(dx, port.linear_input_backward(host, dy)) <= tol


@pytest.mark.parametrize("route,hq,hkv,d,bs", [
    ("attention_bulk", 8, 2, 128, 16),
    ("attention_generic", 8, 2, 128, 8),      # page size other than 16
    ("attention_generic", 6, 2, 64, 16),      # head width other than 128, three query heads per KV head
    ("attention_generic", 2, 1, 3, 2),        # the reference test's own shape class
])
def test_attention_routes(b2, port, route, hq, hkv, d, bs):
    rng = np.random.default_rng(hq * 100 + d + bs)
    lens = np.array([1, bs, bs + 1, 5 * bs + 3], np.uint32)
    blocks = -(-lens.astype(np.int64) // bs)
    P = int(blocks.sum()) + 2
    perm = rng.permutation(P)
    tables = np.zeros((len(lens), int(blocks.max())), np.uint32)
    at = 0
    for s, nb in enumerate(blocks):
        tables[s, :nb] = perm[at:at + nb]
        at += nb
    K = rng.standard_normal((P, hkv, bs, d)).astype(np.float32)
    V = rng.standard_normal((P, hkv, bs, d)).astype(np.float32)
    q = rng.standard_normal((len(lens), hq, d)).astype(np.float32)
    got, status = run_gqa(b2, q, K, V, tables, lens)
    assert b2.last_route() == route
    assert status == 0
    assert rel_l2(got, port.paged_decode_gqa(q, K, V, tables, lens)) <= 2e-3


def test_attention_grid_between_one_and_two_waves(b2, port):
    """16 sequences x 4 KV heads x 9 splits = 576 CTAs: the launcher takes the three-slot form of
    the fast kernel there (two CTAs per SM, fewer waves); larger and smaller grids take two slots.
    Same arithmetic either way, so the result is held to the oracle like any other."""
    rng = np.random.default_rng(576)
    hkv, rep, d, bs = 4, 2, 128, 16
    lens = np.full(16, 2049, np.uint32)
    lens[3], lens[11] = 1800, 2047          # fewer splits for two sequences: their spare CTAs exit at once
    blocks = -(-lens.astype(np.int64) // bs)
    P = int(blocks.sum())
    perm = rng.permutation(P)
    tables = np.zeros((len(lens), int(blocks.max())), np.uint32)
    at = 0
    for s, nb in enumerate(blocks):
        tables[s, :nb] = perm[at:at + nb]
        at += nb
    K = rng.standard_normal((P, hkv, bs, d)).astype(np.float32)
    V = rng.standard_normal((P, hkv, bs, d)).astype(np.float32)
    q = rng.standard_normal((len(lens), hkv * rep, d)).astype(np.float32)
    got, status = run_gqa(b2, q, K, V, tables, lens)
    assert b2.last_route() == "attention_bulk" and status == 0
    want = port.paged_decode_gqa(q, K, V, tables, lens)
    for s in range(len(lens)):
        assert rel_l2(got[s], want[s]) <= 2e-3, f"sequence {s}"
