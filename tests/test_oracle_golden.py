"""The C restatement in oracle/ against the committed reference vectors
(produced by the reference's own CPU code, see tests/golden/make_golden.py) and
against the known answers written in the reference's tests. CPU only."""
import numpy as np
import pytest

import cases
from conftest import bits, weight_from_golden

import oracle


def same_payload(a, b):
    assert (a.codes == b.codes).all()
    assert a.encoding == b.encoding
    if a.fp32_scales is not None:
        assert (bits(a.fp32_scales) == bits(b.fp32_scales)).all()
    else:
        assert (a.scale_codes == b.scale_codes).all()
        assert (bits(a.second_level) == bits(b.second_level)).all()
        assert np.float32(a.offset) == np.float32(b.offset)


def test_codebook_literals_and_packing_kat(port, golden):
    # tests/core/test_quantization.cpp:61-112
    cb = port.codebook()
    assert (bits(cb) == bits(golden["codebook"])).all()
    assert cb[7] == 0.0 and (np.diff(cb) > 0).all()
    w = port.quantize_nf4(cb.reshape(1, 16), 32)
    assert w.codes.tolist() == [0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE]
    assert w.fp32_scales.tolist() == [1.0]
    assert (bits(port.dequantize(w)) == bits(cb)).all()
    same_payload(w, weight_from_golden(golden, "kat_codebook"))


def test_tie_zero_and_partial_blocks(port, golden):
    # tests/core/test_quantization.cpp:115-153
    tie = port.quantize_nf4(golden["tie_values"].reshape(1, 32), 32)
    assert tie.codes[0] & 0x0F == 7
    same_payload(tie, weight_from_golden(golden, "tie"))

    zeros = port.quantize_nf4(np.zeros((1, 33), np.float32), 32)
    assert zeros.fp32_scales.tolist() == [0.0, 0.0]
    assert all(((zeros.codes[i // 2] >> (4 * (i % 2))) & 15) == 7 for i in range(33))
    assert zeros.codes[-1] == 0x07
    same_payload(zeros, weight_from_golden(golden, "zeros33"))

    part = port.quantize_nf4(golden["partial_values"].reshape(1, 33), 32)
    assert part.fp32_scales.tolist() == [2.0, 10.0]
    assert part.codes[0] & 15 == 0 and part.codes[16] & 15 == 15
    same_payload(part, weight_from_golden(golden, "partial"))
    assert (bits(port.dequantize(part)) == bits(golden["partial_dequant"])).all()


def test_double_quantized_golden_vector(port, golden):
    # tests/core/test_quantization.cpp:155-214
    w = port.quantize_nf4_double_quantized(golden["dq33_values"].reshape(1, -1), 32, 32)
    assert w.second_level.tolist() == [16.0, 16.0] and w.offset == 16.0
    assert (w.scale_codes[0], w.scale_codes[16], w.scale_codes[32]) == (1, 128, 255)
    d = port.dequantize(w).ravel()
    assert (d[0], d[16 * 32], d[32 * 32]) == (0.0, 16.0, 32.0)
    assert len(w.codes) == 528 and w.scale_bytes == 45 and w.payload_bytes == 573
    same_payload(w, weight_from_golden(golden, "dq33"))
    assert (bits(d) == bits(golden["dq33_dequant"]).ravel()).all()


def test_nearest_code_sweep(port, golden):
    got = np.array([port.nearest_code(float(v)) for v in golden["nearest_probes"]], np.uint8)
    assert (got == golden["nearest_codes"]).all()


@pytest.mark.parametrize("name", ["aligned", "edge"])
@pytest.mark.parametrize("enc", ["fp32", "dq"])
def test_linear_fixtures(port, golden, name, enc):
    # tests/core/backend/test_quantized_linear_backend.cpp:89-302
    W = getattr(cases, f"{name}_weight")()
    X = getattr(cases, f"{name}_input")()
    dY = getattr(cases, f"{name}_upstream")()
    assert (bits(W) == bits(golden[f"{name}_weight"])).all()
    w = port.quantize_nf4(W, 32) if enc == "fp32" else port.quantize_nf4_double_quantized(W, 32, 32)
    p = f"{name}_{enc}"
    same_payload(w, weight_from_golden(golden, p))
    if name == "edge":
        assert w.numel % 2 == 1 and w.blocks == 35 and (w.codes[-1] & 0xF0) == 0
        if enc == "dq":
            assert len(w.second_level) == 2
    deq = port.dequantize(w)
    assert (bits(deq) == bits(golden[f"{p}_dequant"])).all()
    y = port.linear_forward(w, X)
    dx = port.linear_input_backward(w, dY)
    assert (bits(y) == bits(golden[f"{p}_forward"])).all()
    assert (bits(dx) == bits(golden[f"{p}_backward"])).all()
    # single-thread and OpenMP forms agree bit for bit
    assert (bits(port.linear_forward(w, X, threads=1)) == bits(y)).all()
    # the reference test's own oracle: matmul with the dequantised weight, 3e-5 relative-with-floor
    for got, want in ((y, X @ deq.T), (dx, dY @ deq)):
        assert (np.abs(got - want) <= 3e-5 * np.maximum(1.0, np.maximum(np.abs(got), np.abs(want)))).all()


def test_paged_decode_fixture(port, golden):
    # tests/core/backend/test_nn_backend.cpp:2079-2216: table {3,0,4}, poisoned unused pages
    ctx = port.paged_decode(golden["paged_query"], golden["paged_key_pages"], golden["paged_value_pages"],
                            golden["paged_table"], int(golden["paged_seq_len"][0]))
    assert (bits(ctx) == bits(golden["paged_reference_context"])).all()
    want = golden["paged_expected_causal_last_row"]
    assert (np.abs(ctx - want) <= 2e-6 * np.maximum(1.0, np.maximum(np.abs(ctx), np.abs(want)))).all()


def test_paged_decode_special_values(port):
    # tests/core/backend/test_nn_backend.cpp:2339-2403
    one = np.ones((1, 1, 1, 1), np.float32)
    for bad in (np.nan, np.inf, -np.inf):
        with pytest.raises(FloatingPointError):
            port.paged_decode(np.full((1, 1), bad, np.float32), one, one, [0], 1)


def test_seeded_config1_and_gqa(port, golden):
    c = cases.seeded_cases()
    w = port.quantize_nf4(c["W1"], 64)
    assert int(np.bitwise_xor.reduce(w.codes.view(np.uint32))) == int(golden["c1_codes_xor"][0])
    assert (bits(w.fp32_scales) == bits(golden["c1_scales"])).all()
    assert (bits(port.linear_forward(w, c["X1"])[:8]) == bits(golden["c1_forward_rows0_8"])).all()
    wd = port.quantize_nf4_double_quantized(c["W1"], 64, 256)
    assert (wd.scale_codes == golden["c1_dq_scale_codes"]).all()
    assert (bits(wd.second_level) == bits(golden["c1_dq_second_level"])).all()
    assert np.float32(wd.offset) == golden["c1_dq_offset"][0]
    assert (bits(port.linear_forward(wd, c["X1"])[:8]) == bits(golden["c1_dq_forward_rows0_8"])).all()
    assert (bits(port.linear_input_backward(wd, c["dY1"])) == bits(golden["c1_dq_backward"])).all()
    ctx = port.paged_decode_gqa(c["q"], c["K"], c["V"], c["table"][None, :], np.array([c["seq_len"]], np.uint32))
    assert (bits(ctx) == bits(golden["gqa_context"])).all()


@pytest.mark.skipif(not oracle.ref_available(), reason="reference library not built here")
def test_port_matches_reference_library_on_random_shapes(port):
    ref = oracle.ref()
    rng = np.random.default_rng(7)
    for out_f, in_f, block, sblock in ((5, 96, 32, 32), (17, 64, 64, 256), (9, 130, 32, 64), (3, 4096, 4096, 32)):
        W = (rng.standard_normal((out_f, in_f)) * 0.05).astype(np.float32)
        W[rng.integers(out_f), :] = 0.0
        X = rng.standard_normal((3, in_f)).astype(np.float32)
        dY = rng.standard_normal((2, out_f)).astype(np.float32)
        for dq in (False, True):
            a = port.quantize_nf4_double_quantized(W, block, sblock) if dq else port.quantize_nf4(W, block)
            b = ref.quantize_nf4_double_quantized(W, block, sblock) if dq else ref.quantize_nf4(W, block)
            same_payload(a, b)
            assert (bits(port.dequantize(a)) == bits(ref.dequantize(b))).all()
            assert (bits(port.linear_forward(a, X)) == bits(ref.linear_forward(b, X))).all()
            assert (bits(port.linear_input_backward(a, dY)) == bits(ref.linear_input_backward(b, dY))).all()


# ---- decode-step primitives: the restatements against vectors written by the reference ----------

def test_rms_norm_matches_the_reference_bit_for_bit(port, golden):
    g = cases.decode_glue_inputs()
    got = port.rms_norm(g["rms_x"], g["rms_scale"], 1e-5)
    assert (bits(got) == bits(golden["glue_rms"])).all()


@pytest.mark.parametrize("position", cases.ROPE_POSITIONS)
def test_split_half_rope_matches_the_reference_bit_for_bit(golden, position):
    # the angle is evaluated in double and rounded once to FP32, like rotary_cos_sin
    # (src/model/rotary_embedding.cpp:64-81); numpy's double pow / cos / sin agree with libm here
    from oracle import decode_ref
    g = cases.decode_glue_inputs()
    got = decode_ref.rotate(g["rope_x"][:, :, 0, :], position, 1e4)
    assert (bits(got) == bits(golden[f"glue_rope_{position}"][:, :, 0, :])).all()


def test_silu_and_swiglu_hidden_match_the_reference_bit_for_bit(port, golden):
    g = cases.decode_glue_inputs()
    silu = port.silu_mul(g["silu_gate"])
    assert (bits(silu) == bits(golden["glue_silu"])).all()
    minus_inf = np.flatnonzero(np.isneginf(g["silu_gate"]))
    assert minus_inf.size == 1 and bits(silu[minus_inf])[0] == 0x80000000      # silu(-inf) = -0.0
    hidden = port.silu_mul(g["silu_gate"], g["silu_up"])
    assert (bits(hidden) == bits(golden["glue_swiglu_hidden"])).all()


def test_greedy_choice_takes_the_first_maximum(port, golden):
    g = cases.decode_glue_inputs()
    got = [port.greedy(row) for row in g["greedy_logits"]]
    assert got == golden["glue_greedy"].tolist()
    assert got[1] == 40 and got[2] == 96 and got[3] == 0 and got[4] == 0


def test_rope_page_append_and_paged_attention_match_the_reference_cache(port, golden):
    """One sequence token by token: rotate q and k at the token's position, write k / v into slot
    position % page of page table[position / page], attend over everything appended so far. The
    expected contexts come from the reference's PagedKvCachePool (append_and_attend)."""
    from oracle import decode_ref
    g = cases.decode_glue_inputs()
    steps, heads, width = g["cache_q"].shape
    page, pages = 4, 5
    table = np.array([3, 0, 4, 1, 2], np.uint32)           # any permutation: results do not depend on it
    K = np.full((pages, heads, page, width), 777.0, np.float32)
    V = np.full((pages, heads, page, width), -777.0, np.float32)
    for t in range(steps):
        q = decode_ref.rotate(g["cache_q"][t], t, 1e4)
        K[table[t // page], :, t % page] = decode_ref.rotate(g["cache_k"][t], t, 1e4)
        V[table[t // page], :, t % page] = g["cache_v"][t]
        ctx = port.paged_decode(q, K, V, table, t + 1)
        assert (bits(ctx) == bits(golden["glue_cache_context"][t])).all(), t


def test_lora_branch_matches_the_reference_bit_for_bit(port, golden):
    lo = cases.lora_inputs()
    got = port.lora_forward(lo["x"], lo["a"], lo["b"], float(lo["scale"]))
    assert (bits(got) == bits(golden["lora_branch"])).all()
    base = port.linear_forward(port.quantize_nf4(lo["w"], 32), lo["x"])
    assert (bits(base + got) == bits(golden["lora_adapted_linear"])).all()
