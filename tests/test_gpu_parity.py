"""Parity of the CUDA path (through the C ABI) with the CPU oracle and with the
committed reference vectors. Every test here needs a B200.

Tolerances: dequantised weights and page gathers are bit-exact; linear and
attention outputs are compared by relative L2 error against the FP32 CPU oracle
(<= 2e-3 for the FP32-accumulate decode kernels and attention), and the
reference's own fixtures by its accelerator tolerance of 3e-5 (3e-4 for
attention) relative-with-floor."""
import numpy as np
import pytest
import torch

import cases
from conftest import Guarded, bits, rel_l2, weight_from_golden

pytestmark = pytest.mark.gpu

GEMV_TOL = 2e-3
ATTN_TOL = 2e-3


@pytest.fixture(scope="module")
def b2():
    import riftco_transformer_b200 as pkg
    assert pkg.is_available(), pkg.unavailability_reason()
    return pkg


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def close_with_floor(actual, expected, tol):
    a, e = np.asarray(actual), np.asarray(expected)
    return bool((np.abs(a - e) <= tol * np.maximum(1.0, np.maximum(np.abs(a), np.abs(e)))).all())


def forward(b2, w, x):
    """Through the C ABI into an output placed between guard bands: every caller of this helper
    also checks that the kernel it reached wrote nothing outside its [rows, out] tensor."""
    rows = x.shape[0]
    out = Guarded((rows, w.out_features))
    b2.dispatch_quantized_linear_forward(x, w, out.tensor, (rows, w.in_features, w.out_features, w.block_size))
    out.check()
    return out.tensor.cpu().numpy()


def backward(b2, w, dy):
    rows = dy.shape[0]
    out = Guarded((rows, w.in_features))
    b2.dispatch_quantized_linear_input_backward(dy, w, out.tensor, (rows, w.in_features, w.out_features, w.block_size))
    out.check()
    return out.tensor.cpu().numpy()


# ---- dequantisation: bit-exact ---------------------------------------------------

@pytest.mark.parametrize("prefix", ["kat_codebook", "partial", "dq33", "aligned_fp32", "aligned_dq",
                                    "edge_fp32", "edge_dq"])
def test_dequantize_matches_reference_vectors_bit_exactly(b2, golden, prefix):
    host = weight_from_golden(golden, prefix)
    got = b2.dequantize(b2.PackedNf4Weight.from_host(host)).cpu().numpy()
    assert (bits(got).ravel() == bits(golden[f"{prefix}_dequant"]).ravel()).all()


@pytest.mark.parametrize("shape,block,sblock", [((1024, 512), 64, 256), ((4096, 4096), 64, 256),
                                                ((333, 77), 32, 32), ((64, 14336), 128, 64)])
@pytest.mark.parametrize("dq", [False, True])
def test_dequantize_random_bit_exact(b2, port, shape, block, sblock, dq):
    rng = np.random.default_rng(11)
    W = (rng.standard_normal(shape) * 0.02).astype(np.float32)
    W[1, : min(shape[1], 2 * block)] = 0.0
    host = port.quantize_nf4_double_quantized(W, block, sblock) if dq else port.quantize_nf4(W, block)
    got = b2.dequantize(b2.PackedNf4Weight.from_host(host)).cpu().numpy()
    assert (bits(got) == bits(port.dequantize(host))).all()


def test_dequantize_row_shards_are_bitwise_slices(b2, port):
    rng = np.random.default_rng(12)
    W = (rng.standard_normal((512, 14336)) * 0.02).astype(np.float32)  # 224 blocks per row: groups straddle rows
    host = port.quantize_nf4_double_quantized(W, 64, 256)
    full = b2.PackedNf4Weight.from_host(host)
    want = port.dequantize(host)
    for world in (2, 4, 8):
        for rank in range(world):
            shard = full.row_shard(rank, world)
            got = b2.dequantize(shard).cpu().numpy()
            rows = 512 // world
            assert (bits(got) == bits(want[rank * rows:(rank + 1) * rows])).all()


# ---- linear: the reference's fixtures (generic kernels) ---------------------------

@pytest.mark.parametrize("name", ["aligned", "edge"])
@pytest.mark.parametrize("enc", ["fp32", "dq"])
def test_linear_reference_fixtures(b2, golden, name, enc):
    p = f"{name}_{enc}"
    w = b2.PackedNf4Weight.from_host(weight_from_golden(golden, p))
    y = forward(b2, w, dev(golden[f"{name}_input"]))
    dx = backward(b2, w, dev(golden[f"{name}_upstream"]))
    assert close_with_floor(y, golden[f"{p}_forward"], 3e-5)
    assert close_with_floor(dx, golden[f"{p}_backward"], 3e-5)


def test_linear_config1_against_reference_rows(b2, port, golden):
    c = cases.seeded_cases()
    for dq, key in ((False, "c1_forward_rows0_8"), (True, "c1_dq_forward_rows0_8")):
        host = port.quantize_nf4_double_quantized(c["W1"], 64, 256) if dq else port.quantize_nf4(c["W1"], 64)
        w = b2.PackedNf4Weight.from_host(host)
        y = forward(b2, w, dev(c["X1"]))  # 64 rows: tensor-core path (bf16 operands)
        assert rel_l2(y[:8], golden[key]) <= 1e-2
        y8 = forward(b2, w, dev(c["X1"][:8]))  # 8 rows: decode kernel
        assert rel_l2(y8, golden[key]) <= GEMV_TOL
        if dq:
            dx = backward(b2, w, dev(c["dY1"]))
            assert rel_l2(dx, golden["c1_dq_backward"]) <= 1e-5


# ---- decode GEMV: baseline configuration 2 ----------------------------------------

@pytest.fixture(scope="module")
def c2_weights(port):
    rng = np.random.default_rng(1234)
    out = {}
    for out_f, in_f in ((4096, 4096), (14336, 4096), (4096, 14336)):
        W = (rng.standard_normal((out_f, in_f)) * 0.02).astype(np.float32)
        out[(out_f, in_f)] = port.quantize_nf4_double_quantized(W, 64, 256)
    return out


@pytest.mark.parametrize("shape", [(4096, 4096), (14336, 4096), (4096, 14336)])
@pytest.mark.parametrize("rows", [1, 4, 16, 23, 32])
def test_gemv_config2(b2, port, c2_weights, shape, rows):
    host = c2_weights[shape]
    w = b2.PackedNf4Weight.from_host(host)
    x = np.random.default_rng(5678 + rows).standard_normal((rows, shape[1])).astype(np.float32)
    y = forward(b2, w, dev(x))
    want = port.linear_forward(host, x)
    assert np.isfinite(y).all()
    # up to 16 rows: fp16 operands, FP32 block scales (2e-3); above, the bf16 tensor-core path (1e-2)
    tol = GEMV_TOL if rows <= 16 else 1e-2
    assert rel_l2(y, want) <= tol
    # every row separately, so a wrong batch row cannot hide in the norm
    for r in range(rows):
        assert rel_l2(y[r], want[r]) <= tol


@pytest.mark.parametrize("out_f,in_f,block,rows,dq", [
    (1000, 192, 64, 3, True),      # ragged row tile, 3 steps
    (17, 64, 64, 1, False),        # fewer rows than one MMA tile
    (256, 8192, 4096, 7, True),    # largest block size
    (4096, 4096, 128, 9, False),   # FP32 scales, block 128, two batch tiles
    (130, 2048 + 64, 64, 20, True),
])
def test_gemv_edge_shapes(b2, port, out_f, in_f, block, rows, dq):
    rng = np.random.default_rng(out_f * 7 + in_f)
    W = (rng.standard_normal((out_f, in_f)) * 0.05).astype(np.float32)
    host = port.quantize_nf4_double_quantized(W, block, 32) if dq else port.quantize_nf4(W, block)
    x = rng.standard_normal((rows, in_f)).astype(np.float32)
    y = forward(b2, b2.PackedNf4Weight.from_host(host), dev(x))
    # up to 16 rows the fp16 decode kernel (2e-3); more rows go to the bf16 tensor-core kernel (1e-2)
    assert rel_l2(y, port.linear_forward(host, x)) <= (GEMV_TOL if rows <= 16 else 1e-2)


def test_gemv_is_linear_and_deterministic(b2, port, c2_weights):
    host = c2_weights[(4096, 4096)]
    w = b2.PackedNf4Weight.from_host(host)
    rng = np.random.default_rng(3)
    a = rng.standard_normal((4, 4096)).astype(np.float32)
    b = rng.standard_normal((4, 4096)).astype(np.float32)
    ya, yb, yab = forward(b2, w, dev(a)), forward(b2, w, dev(b)), forward(b2, w, dev(a + b))
    assert rel_l2(yab, ya + yb) <= 2 * GEMV_TOL
    assert (bits(forward(b2, w, dev(a))) == bits(ya)).all()


def test_gemv_row_shards_concatenate(b2, port, c2_weights):
    host = c2_weights[(14336, 4096)]
    full = b2.PackedNf4Weight.from_host(host)
    x = np.random.default_rng(9).standard_normal((8, 4096)).astype(np.float32)
    want = port.linear_forward(host, x)
    parts = [forward(b2, full.row_shard(r, 8), dev(x)) for r in range(8)]
    assert rel_l2(np.concatenate(parts, axis=1), want) <= GEMV_TOL


# ---- input backward ------------------------------------------------------------------

@pytest.mark.parametrize("dq", [False, True])
def test_input_backward_random(b2, port, dq):
    rng = np.random.default_rng(21)
    W = (rng.standard_normal((768, 320)) * 0.02).astype(np.float32)
    host = port.quantize_nf4_double_quantized(W, 64, 256) if dq else port.quantize_nf4(W, 64)
    dy = (rng.standard_normal((19, 768)) * 0.01).astype(np.float32)
    dx = backward(b2, b2.PackedNf4Weight.from_host(host), dev(dy))
    assert rel_l2(dx, port.linear_input_backward(host, dy)) <= 1e-5


# ---- validation mirrors the reference's dispatch layer -------------------------------

def test_linear_rejects_bad_requests(b2, golden):
    w = b2.PackedNf4Weight.from_host(weight_from_golden(golden, "aligned_fp32"))
    x = dev(golden["aligned_input"])
    y = torch.empty((2, 3), dtype=torch.float32, device="cuda")
    with pytest.raises(RuntimeError):
        b2.dispatch_quantized_linear_forward(x, w, torch.empty(5, device="cuda"), (2, 32, 3, 32))
    with pytest.raises(ValueError):
        b2.dispatch_quantized_linear_forward(x, w, y, (2, 32, 3, 0))
    with pytest.raises(ValueError):
        b2.dispatch_quantized_linear_forward(x.cpu(), w, y, (2, 32, 3, 32))
    same = torch.empty(64, dtype=torch.float32, device="cuda")
    from riftco_transformer_b200 import _lib
    import ctypes as C
    ws = w.struct()
    assert _lib.lib.b2_nf4_linear_forward(C.byref(ws), same.data_ptr(), same.data_ptr(), 2, None, 0, None) \
        == _lib.STATUS_INVALID_ARGUMENT
    assert b"alias" in _lib.lib.b2_last_error()
    assert _lib.lib.b2_nf4_linear_forward(C.byref(ws), x.data_ptr(), y.data_ptr(), 0, None, 0, None) \
        == _lib.STATUS_INVALID_ARGUMENT


# ---- paged decode attention ----------------------------------------------------------

def test_paged_decode_reference_fixture(b2, golden):
    # table {3,0,4}, head width 3, block size 2, unused slots poisoned with -+777
    heads, width = golden["paged_query"].shape
    ctx = torch.empty((heads, width), dtype=torch.float32, device="cuda")
    b2.dispatch_paged_decode_attention_forward(
        dev(golden["paged_query"]), dev(golden["paged_key_pages"]), dev(golden["paged_value_pages"]),
        golden["paged_table"], ctx, (heads, width, 2, 5, int(golden["paged_seq_len"][0])))
    got = ctx.cpu().numpy()
    assert close_with_floor(got, golden["paged_expected_causal_last_row"], 3e-4)
    assert close_with_floor(got, golden["paged_reference_context"], 3e-4)


def test_paged_decode_contract_and_special_values(b2):
    # tests/core/backend/test_nn_backend.cpp:2218-2403 restated
    q = torch.ones((1, 1), device="cuda")
    keys = dev(np.array([1, 2, 3, 4], np.float32).reshape(2, 1, 2, 1))
    values = dev(np.array([0.5, 1, 1.5, 2], np.float32).reshape(2, 1, 2, 1))
    ctx = torch.empty((1, 1), device="cuda")
    dims = (1, 1, 2, 2, 1)
    f = b2.dispatch_paged_decode_attention_forward
    with pytest.raises(ValueError):
        f(q, keys, values, [0], ctx, (0, 1, 2, 2, 1))
    with pytest.raises(ValueError):
        f(q, keys, values, [], ctx, dims)
    with pytest.raises(IndexError):
        f(q, keys, values, [2], ctx, dims)
    with pytest.raises(RuntimeError):
        f(q, keys[:1].contiguous(), values, [0], ctx, dims)
    with pytest.raises(ValueError):
        f(q, keys, values, [0], q, dims)
    with pytest.raises(OverflowError):
        f(q, keys, values, [0], ctx, (1, 1, 2, 2 ** 32 + 2, 1))
    f(q, keys, values, [0], ctx, dims)
    assert abs(ctx.item() - 0.5) < 1e-6
    one = torch.ones((1, 1, 1, 1), device="cuda")
    for bad in (float("nan"), float("inf"), float("-inf")):
        with pytest.raises(b2.DomainError):
            f(torch.full((1, 1), bad, device="cuda"), one, one.clone(), [0], torch.empty((1, 1), device="cuda"),
              (1, 1, 1, 1, 1))


def run_gqa(b2, q, K, V, tables, lens):
    n_seq, hq, d = q.shape
    out = Guarded((n_seq, hq, d))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    pool = b2.PagedKvPool(dev(K), dev(V))
    b2.paged_decode_attention(dev(q), pool, dev(tables.view(np.int32)), dev(lens.view(np.int32)), out.tensor,
                              int(lens.max()), status=status)
    out.check()
    return out.tensor.cpu().numpy(), int(status.item())


def test_paged_decode_gqa_golden_sequence(b2, golden):
    c = cases.seeded_cases()
    got, status = run_gqa(b2, c["q"], c["K"], c["V"], c["table"][None, :], np.array([c["seq_len"]], np.uint32))
    assert status == 0
    assert rel_l2(got, golden["gqa_context"]) <= ATTN_TOL


@pytest.mark.parametrize("rep", [1, 2, 4, 8])
def test_paged_decode_batched_ragged(b2, port, rep):
    rng = np.random.default_rng(91011 + rep)
    hkv, d, bs = 4, 128, 16
    lens = np.array([1, 15, 16, 17, 255, 256, 257, 300, 1024, 2049], np.uint32)
    blocks = -(-lens.astype(np.int64) // bs)
    P = int(blocks.sum()) + 3
    perm = rng.permutation(P)
    tables = np.zeros((len(lens), int(blocks.max())), np.uint32)
    at = 0
    for s, nb in enumerate(blocks):
        tables[s, :nb] = perm[at:at + nb]
        at += nb
    K = rng.standard_normal((P, hkv, bs, d)).astype(np.float32)
    V = rng.standard_normal((P, hkv, bs, d)).astype(np.float32)
    # poison the unused tail of every last page: it must never reach the result
    for s, n in enumerate(lens):
        tail = int(n) % bs
        if tail:
            K[tables[s, blocks[s] - 1], :, tail:] = np.nan
            V[tables[s, blocks[s] - 1], :, tail:] = np.inf
    q = rng.standard_normal((len(lens), hkv * rep, d)).astype(np.float32)
    got, status = run_gqa(b2, q, K, V, tables, lens)
    assert status == 0
    want = port.paged_decode_gqa(q, np.nan_to_num(K, nan=0.0), np.nan_to_num(V, posinf=0.0), tables, lens)
    assert np.isfinite(got).all()
    for s in range(len(lens)):
        assert rel_l2(got[s], want[s]) <= ATTN_TOL, f"sequence {s} (len {lens[s]})"


def test_paged_decode_config4_sample(b2, port):
    # 8 of the 64 sequences of the baseline's paged-decode configuration
    rng = np.random.default_rng(91011)
    hq, hkv, d, bs = 32, 8, 128, 16
    lens = rng.integers(512, 8193, size=8).astype(np.uint32)
    blocks = -(-lens.astype(np.int64) // bs)
    P = int(blocks.sum())
    perm = rng.permutation(P)
    tables = np.zeros((8, int(blocks.max())), np.uint32)
    at = 0
    for s, nb in enumerate(blocks):
        tables[s, :nb] = perm[at:at + nb]
        at += nb
    K = rng.standard_normal((P, hkv, bs, d)).astype(np.float32)
    V = rng.standard_normal((P, hkv, bs, d)).astype(np.float32)
    q = rng.standard_normal((8, hq, d)).astype(np.float32)
    got, status = run_gqa(b2, q, K, V, tables, lens)
    assert status == 0
    assert rel_l2(got, port.paged_decode_gqa(q, K, V, tables, lens)) <= ATTN_TOL


def test_paged_decode_config4_all_64_sequences(b2, port):
    """The baseline's paged-decode configuration in full: 64 sequences with context U[512, 8192],
    32 query / 8 KV heads, permuted pages (2.2 GB of K/V), every sequence against the oracle."""
    rng = np.random.default_rng(91011)
    hq, hkv, d, bs = 32, 8, 128, 16
    lens = rng.integers(512, 8193, size=64).astype(np.uint32)
    blocks = -(-lens.astype(np.int64) // bs)
    P = int(blocks.sum())
    perm = rng.permutation(P)
    tables = np.zeros((64, int(blocks.max())), np.uint32)
    at = 0
    for s, nb in enumerate(blocks):
        tables[s, :nb] = perm[at:at + nb]
        at += nb
    K = rng.standard_normal((P, hkv, bs, d), dtype=np.float32)
    V = rng.standard_normal((P, hkv, bs, d), dtype=np.float32)
    q = rng.standard_normal((64, hq, d), dtype=np.float32)
    got, status = run_gqa(b2, q, K, V, tables, lens)
    assert status == 0
    want = port.paged_decode_gqa(q, K, V, tables, lens, threads=0)
    assert rel_l2(got, want) <= ATTN_TOL
    for s in range(64):
        assert rel_l2(got[s], want[s]) <= ATTN_TOL, f"sequence {s} (len {lens[s]})"


def test_device_encoder_matches_the_oracle_bit_for_bit(b2, port):
    """synth.quantize - the reference's NF4 encoder restated in torch, which produces the benchmark's
    weights on the device - against the C restatement of pack_nf4 / double_quantize_scales: same
    codes (ties to the lower index, zero blocks -> scale 0 / code 7), same scales, same offset."""
    from riftco_transformer_b200 import synth
    rng = np.random.default_rng(31)
    W = (rng.standard_normal((384, 1024)) * 0.02).astype(np.float32)
    W[5, 64:128] = 0.0                      # a zero block
    W[7, :64] = np.float32(0.02) * port.codebook()[np.arange(64) % 16] * np.float32(1.0)   # exact codebook points
    W[9, 0:2] = (0.5, -0.5)                 # a value halfway between two levels after scaling
    for dq in (True, False):
        dev_w = synth.quantize(torch.from_numpy(W).cuda(), double_quantized=dq)
        host = port.quantize_nf4_double_quantized(W, 64, 256) if dq else port.quantize_nf4(W, 64)
        assert np.array_equal(dev_w.codes.cpu().numpy(), host.codes)
        if dq:
            assert np.array_equal(dev_w.primary.cpu().numpy(), host.scale_codes)
            assert (bits(dev_w.secondary.cpu().numpy()) == bits(host.second_level)).all()
            assert np.float32(dev_w.offset) == np.float32(host.offset)
        else:
            assert (bits(dev_w.primary.cpu().numpy()) == bits(host.fp32_scales)).all()
        assert (bits(b2.dequantize(dev_w).cpu().numpy()) == bits(port.dequantize(host))).all()


def test_rope_append_refuses_a_position_past_the_table(b2):
    """A position whose page index lies past the sequence's table row is treated like a bad block:
    the status bit is set and no page is written (the neighbouring row is never read)."""
    from riftco_transformer_b200._lib import lib
    from riftco_transformer_b200.backend import _check
    heads, d, bs = 2, 128, 16
    q = torch.randn((2, heads, d), device="cuda")
    k = torch.randn((2, heads, d), device="cuda")
    v = torch.randn((2, heads, d), device="cuda")
    K = torch.full((4, heads, bs, d), 7.0, device="cuda")
    V = torch.full((4, heads, bs, d), -7.0, device="cuda")
    tables = torch.tensor([[0, 1], [2, 3]], dtype=torch.int32, device="cuda")
    positions = torch.tensor([32, 5], dtype=torch.int32, device="cuda")    # 32 / 16 = 2: past a row of 2 entries
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _check(lib.b2_rope_append_kv(q.data_ptr(), k.data_ptr(), v.data_ptr(), positions.data_ptr(), tables.data_ptr(),
                                 K.data_ptr(), V.data_ptr(), 2, heads, heads, d, bs, 4, 2, 1e4, status.data_ptr(), None))
    torch.cuda.synchronize()
    assert int(status.item()) & 4
    # sequence 1 appended normally (page 2, slot 5); nothing else changed, in particular not page 2's
    # slot 0, which is where sequence 0 would have landed through its neighbour's table row
    assert torch.equal(V[2, :, 5], v[1])
    untouched = torch.ones((4, bs), dtype=torch.bool, device="cuda")
    untouched[2, 5] = False
    assert (V.permute(0, 2, 1, 3)[untouched] == -7.0).all() and (K.permute(0, 2, 1, 3)[untouched] == 7.0).all()


def test_paged_decode_flags_bad_block_without_touching_it(b2):
    q = torch.randn((1, 8, 128), device="cuda")
    pool = b2.PagedKvPool(torch.randn((2, 8, 16, 128), device="cuda"), torch.randn((2, 8, 16, 128), device="cuda"))
    ctx = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    table = torch.tensor([[1, 7]], dtype=torch.int32, device="cuda")  # 7 is outside the pool of 2
    b2.paged_decode_attention(q, pool, table, torch.tensor([20], dtype=torch.int32, device="cuda"), ctx, 20,
                              status=status)
    torch.cuda.synchronize()
    assert int(status.item()) & 4


# ---- host-buffer seam -----------------------------------------------------------------

def test_host_seam_from_two_threads_at_once(b2, port, c2_weights):
    """The host-buffer forms share one staging buffer per device; concurrent callers must not see
    each other's data (each call holds the device's lock from its first copy to its last)."""
    import threading
    host = c2_weights[(4096, 4096)]
    w = b2.PackedNf4Weight.from_host(host)
    rng = np.random.default_rng(12)
    xs = [rng.standard_normal((4, 4096)).astype(np.float32) for _ in range(2)]
    wants = [forward(b2, w, dev(x)) for x in xs]
    errors = []

    def worker(i):
        try:
            torch.cuda.set_device(0)
            y = np.empty((4, 4096), np.float32)
            for _ in range(40):
                b2.host_quantized_linear_forward(xs[i], w, y, 4)
                if not (bits(y) == bits(wants[i])).all():
                    errors.append(f"thread {i}: output of another call")
                    return
        except Exception as e:   # noqa: BLE001
            errors.append(repr(e))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    assert not errors, errors


def test_host_seam_matches_device_path(b2, port, c2_weights):
    host = c2_weights[(4096, 4096)]
    w = b2.PackedNf4Weight.from_host(host)
    x = np.random.default_rng(4).standard_normal((4, 4096)).astype(np.float32)
    y = np.empty((4, 4096), np.float32)
    b2.host_quantized_linear_forward(x, w, y, 4)
    assert (bits(y) == bits(forward(b2, w, dev(x)))).all()
    dy = np.random.default_rng(5).standard_normal((2, 4096)).astype(np.float32)
    dx = np.empty((2, 4096), np.float32)
    b2.host_quantized_linear_input_backward(dy, w, dx, 2)
    assert rel_l2(dx, port.linear_input_backward(host, dy)) <= 1e-5

    c = cases.seeded_cases()
    pool = b2.PagedKvPool(dev(c["K"]), dev(c["V"]))
    ctx = np.empty_like(c["q"])
    b2.host_paged_decode_attention_forward(c["q"], pool, c["table"][None, :], np.array([c["seq_len"]], np.uint32), ctx)
    want = port.paged_decode_gqa(c["q"], c["K"], c["V"], c["table"][None, :], np.array([c["seq_len"]], np.uint32))
    assert rel_l2(ctx, want) <= ATTN_TOL
    bad = c["table"].copy()
    bad[0] = 99
    with pytest.raises(IndexError):
        b2.host_paged_decode_attention_forward(c["q"], pool, bad[None, :], np.array([c["seq_len"]], np.uint32), ctx)


# ---- encoder and payload validation on the device ---------------------------------------------

@pytest.mark.parametrize("shape,block,sblock", [((384, 1024), 64, 256), ((33, 33), 32, 32), ((7, 96), 32, 0),
                                                  ((256, 512), 128, 0), ((1024, 4096), 64, 256)])
def test_device_quantize_matches_the_reference_encoder_bit_for_bit(b2, port, shape, block, sblock):
    """b2_nf4_quantize against the C restatement of pack_nf4 / double_quantize_scales (itself held to
    the reference's vectors): codes incl. ties and an odd tail, zero blocks, scales, offset."""
    rng = np.random.default_rng(shape[0] * 7 + block)
    W = (rng.standard_normal(shape) * 0.02).astype(np.float32)
    flat = W.reshape(-1)
    flat[block:2 * block] = 0.0                                             # a zero block
    flat[:16] = np.float32(0.03) * port.codebook()                          # exact levels once scaled
    flat[16:18] = np.float32(0.03) * np.float32(0.5) * (port.codebook()[3] + port.codebook()[4])   # a midpoint
    flat[18] = 0.03
    dev_w = b2.quantize_nf4(torch.from_numpy(W).cuda(), block, sblock)
    host = port.quantize_nf4_double_quantized(W, block, sblock) if sblock else port.quantize_nf4(W, block)
    assert np.array_equal(dev_w.codes.cpu().numpy(), host.codes)
    if sblock:
        assert np.array_equal(dev_w.primary.cpu().numpy(), host.scale_codes)
        assert (bits(dev_w.secondary.cpu().numpy()) == bits(host.second_level)).all()
        assert np.float32(dev_w.offset).view(np.uint32) == np.float32(host.offset).view(np.uint32)
    else:
        assert (bits(dev_w.primary.cpu().numpy()) == bits(host.fp32_scales)).all()
    b2.validate_payload(dev_w)          # what the encoder writes is canonical
    assert (bits(b2.dequantize(dev_w).cpu().numpy()) == bits(port.dequantize(host))).all()


def test_device_quantize_rejects_non_finite_values(b2):
    W = torch.zeros((4, 64), device="cuda")
    W[2, 5] = float("inf")
    with pytest.raises(ValueError, match="NF4 source values must be finite"):
        b2.quantize_nf4(W, 64, 0)
    W[2, 5] = float("nan")
    with pytest.raises(ValueError, match="NF4 source values must be finite"):
        b2.quantize_nf4(W, 32, 32)


def test_validate_payload_applies_the_canonical_rules(b2, port):
    """require_canonical_payload, src/core/quantization/quantized_weight.cpp:102-174, message by message."""
    import dataclasses
    rng = np.random.default_rng(3)
    W = (rng.standard_normal((8, 96)) * 0.02).astype(np.float32)
    W[1, :32] = 0.0
    plain = b2.PackedNf4Weight.from_host(port.quantize_nf4(W, 32))
    nested = b2.PackedNf4Weight.from_host(port.quantize_nf4_double_quantized(W, 32, 32))
    b2.validate_payload(plain)
    b2.validate_payload(nested)

    def broken(w, **changes):
        return dataclasses.replace(w, **changes)

    with pytest.raises(ValueError, match="packed byte count"):
        b2.validate_payload(broken(plain, codes=plain.codes[:-1].clone()))
    with pytest.raises(ValueError, match="scale count does not match"):
        b2.validate_payload(broken(plain, primary=plain.primary[:-1].clone()))
    with pytest.raises(ValueError, match="scale-code count"):
        b2.validate_payload(broken(nested, primary=nested.primary[:-1].clone()))
    with pytest.raises(ValueError, match="second-level scale count"):
        b2.validate_payload(broken(nested, secondary=torch.cat([nested.secondary, nested.secondary[:1]])))
    bad = plain.primary.clone()
    bad[3] = -1.0
    with pytest.raises(ValueError, match="block scales must be finite and nonnegative"):
        b2.validate_payload(broken(plain, primary=bad))
    bad = plain.primary.clone()
    bad[5] = float("nan")
    with pytest.raises(ValueError, match="block scales must be finite and nonnegative"):
        b2.validate_payload(broken(plain, primary=bad))
    bad = nested.secondary.clone()
    bad[0] = float("inf")
    with pytest.raises(ValueError, match="second-level scales must be finite and nonnegative"):
        b2.validate_payload(broken(nested, secondary=bad))
    codes = plain.codes.clone()            # the zero block (row 1, first 32 weights) must hold code 7 only
    codes[(96 + 4) // 2] = 0x73
    with pytest.raises(ValueError, match="canonical zero code 7"):
        b2.validate_payload(broken(plain, codes=codes))
    odd = b2.PackedNf4Weight.from_host(port.quantize_nf4((rng.standard_normal((3, 11)) * 0.1).astype(np.float32), 32))
    b2.validate_payload(odd)
    codes = odd.codes.clone()
    codes[-1] |= 0x50                      # 33 elements: the last byte's high nibble is unused
    with pytest.raises(ValueError, match="unused high nibble"):
        b2.validate_payload(broken(odd, codes=codes))


@pytest.mark.parametrize("hq,hkv,d,bs", [(8, 2, 128, 16), (6, 2, 64, 16)])
def test_paged_decode_writes_the_bf16_copy_of_its_context(b2, hq, hkv, d, bs):
    """b2_paged_decode_attention_bf16: the FP32 context is the one b2_paged_decode_attention writes,
    bit for bit, and the bf16 copy is its round-to-nearest-even (single-split, merged and generic
    paths)."""
    from riftco_transformer_b200._lib import lib
    from riftco_transformer_b200.backend import _check
    rng = np.random.default_rng(hq + d)
    lens = np.array([3, 200, 256, 257, 1500], np.uint32)
    blocks = -(-lens.astype(np.int64) // bs)
    P = int(blocks.sum())
    perm = rng.permutation(P)
    tables = np.zeros((len(lens), int(blocks.max())), np.uint32)
    at = 0
    for s, nb in enumerate(blocks):
        tables[s, :nb] = perm[at:at + nb]
        at += nb
    K = dev(rng.standard_normal((P, hkv, bs, d)).astype(np.float32))
    V = dev(rng.standard_normal((P, hkv, bs, d)).astype(np.float32))
    q = dev(rng.standard_normal((len(lens), hq, d)).astype(np.float32))
    t, ln = dev(tables.view(np.int32)), dev(lens.view(np.int32))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    plain = torch.empty_like(q)
    both = torch.empty_like(q)
    half = torch.empty(q.shape, dtype=torch.bfloat16, device="cuda")
    args = (len(lens), hq, hkv, d, bs, P, tables.shape[1], int(lens.max()), None, 0, status.data_ptr(), None)
    _check(lib.b2_paged_decode_attention(q.data_ptr(), K.data_ptr(), V.data_ptr(), t.data_ptr(), ln.data_ptr(),
                                         plain.data_ptr(), *args))
    _check(lib.b2_paged_decode_attention_bf16(q.data_ptr(), K.data_ptr(), V.data_ptr(), t.data_ptr(), ln.data_ptr(),
                                              both.data_ptr(), half.data_ptr(), *args))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(plain.view(torch.int32), both.view(torch.int32))
    assert torch.equal(half.view(torch.int16), both.to(torch.bfloat16).view(torch.int16))
    with pytest.raises(ValueError):
        _check(lib.b2_paged_decode_attention_bf16(q.data_ptr(), K.data_ptr(), V.data_ptr(), t.data_ptr(),
                                                  ln.data_ptr(), both.data_ptr(), None, *args))
