"""RTNF4S1 packed-model-state streams: the C parser's index against streams
written with the layout of packed_model_state_bytes
(src/c_api/model_state.cpp:27-113), and the malformed-stream cases of
parse_packed_model_state (model_state.cpp:165-297) with the reference's
messages. Two streams written by the reference's own serializer for a small
quantised DecoderOnlyTransformer (tests/golden/make_golden.py) pin the layout:
the parser must locate every array of every weight exactly where the
reference's packed_linear_weight_state() says it is, and this repository's
writer must reproduce the reference's bytes."""
import struct

import numpy as np
import pytest


@pytest.fixture(scope="module")
def payloads(port):
    rng = np.random.default_rng(77)
    a = port.quantize_nf4_double_quantized((rng.standard_normal((48, 128)) * 0.02).astype(np.float32), 64, 16)
    b = port.quantize_nf4((rng.standard_normal((10, 96)) * 0.5).astype(np.float32), 32)
    c = port.quantize_nf4_double_quantized((rng.standard_normal((7, 33))).astype(np.float32), 64, 256)
    return [a, b, c]


def test_index_matches_what_was_written(payloads):
    from riftco_transformer_b200 import rtnf4
    stream = rtnf4.dumps(payloads)
    assert stream[:8] == b"RTNF4S1\0"
    entries = rtnf4.index(stream)
    assert len(entries) == len(payloads)
    raw = np.frombuffer(stream, np.uint8)
    for e, p in zip(entries, payloads):
        assert (e.out_features, e.in_features, e.block_size) == (p.out_features, p.in_features, p.block_size)
        assert np.array_equal(raw[e.codes_offset:e.codes_offset + e.n_codes], p.codes)
        if p.fp32_scales is not None:
            assert not e.double_quantized and e.n_scale_codes == 0 and e.n_second == 0 and e.offset == 0.0
            got = raw[e.fp32_scales_offset:e.fp32_scales_offset + 4 * e.n_fp32_scales].view("<f4")
            assert np.array_equal(got.view(np.uint32), np.asarray(p.fp32_scales, np.float32).view(np.uint32))
        else:
            assert e.double_quantized and e.n_fp32_scales == 0
            assert e.scale_block_size == p.scale_block_size and e.offset == np.float32(p.offset)
            assert np.array_equal(raw[e.scale_codes_offset:e.scale_codes_offset + e.n_scale_codes], p.scale_codes)
            got = raw[e.second_offset:e.second_offset + 4 * e.n_second].view("<f4")
            assert np.array_equal(got.view(np.uint32), np.asarray(p.second_level, np.float32).view(np.uint32))
    # entries are laid out back to back and the last one ends the stream
    last = entries[-1]
    end = (last.second_offset + 4 * last.n_second) if last.double_quantized else \
        (last.fp32_scales_offset + 4 * last.n_fp32_scales)
    assert end == len(stream)


def test_accepts_buffers_of_any_kind(payloads):
    from riftco_transformer_b200 import rtnf4
    stream = rtnf4.dumps(payloads[:1])
    for view in (stream, bytearray(stream), memoryview(stream), np.frombuffer(stream, np.uint8)):
        assert len(rtnf4.index(view)) == 1


def _header(rank=2, block=64, n_codes=4, n_fp32=1, n_sc=0, n_second=0, sbs=0, offset_bits=0, flags=0, dims=(1, 8)):
    return struct.pack("<QQQQQQQII", rank, block, n_codes, n_fp32, n_sc, n_second, sbs, offset_bits, flags) + \
        b"".join(struct.pack("<Q", d) for d in dims)


@pytest.mark.parametrize("stream,message", [
    (b"RTNF4S", "truncated packed model state: magic"),
    (b"RTNF4S2\0" + struct.pack("<Q", 1) + bytes(96), "unknown packed model state format"),
    (b"RTNF4S1\0" + struct.pack("<Q", 0), "weight count is inconsistent"),
    (b"RTNF4S1\0" + struct.pack("<Q", 3) + bytes(100), "weight count is inconsistent"),
    (b"RTNF4S1\0" + struct.pack("<Q", 1) + _header(rank=3, dims=(1, 2, 4)) + bytes(8), "must have rank two"),
    (b"RTNF4S1\0" + struct.pack("<Q", 1) + _header(flags=2) + bytes(8), "unknown flags"),
    (b"RTNF4S1\0" + struct.pack("<Q", 1) + _header(offset_bits=1) + bytes(8), "inconsistent NF4 scale metadata"),
    (b"RTNF4S1\0" + struct.pack("<Q", 1) + _header(n_sc=1) + bytes(9), "inconsistent NF4 scale metadata"),
    (b"RTNF4S1\0" + struct.pack("<Q", 1) + _header(flags=1, n_fp32=1, n_sc=1, n_second=1, sbs=4) + bytes(13),
     "inconsistent NF4 scale metadata"),
    (b"RTNF4S1\0" + struct.pack("<Q", 1) + _header(flags=1, n_fp32=0, n_sc=1, n_second=1, sbs=0) + bytes(9),
     "inconsistent NF4 scale metadata"),
    (b"RTNF4S1\0" + struct.pack("<Q", 1) + _header() + bytes(7), "truncated packed model state: weight payload"),
    (b"RTNF4S1\0" + struct.pack("<Q", 1) + _header() + bytes(9), "trailing bytes"),
])
def test_malformed_streams_are_rejected_like_the_reference(stream, message):
    from riftco_transformer_b200 import rtnf4
    with pytest.raises(ValueError, match=message):
        rtnf4.index(stream)


def test_sizes_past_the_address_space_overflow():
    from riftco_transformer_b200 import rtnf4
    stream = b"RTNF4S1\0" + struct.pack("<Q", 1) + _header(n_codes=2 ** 64 - 8, n_fp32=2 ** 62) + bytes(8)
    with pytest.raises(OverflowError, match="exceeds addressable memory"):
        rtnf4.index(stream)


def test_row_shards_are_slices_of_the_stream(payloads):
    """load_weight on the CPU device: a shard's arrays are byte ranges of the stream, the second-level
    scales are shared, and flat_block_base keeps the parent's block numbering."""
    from riftco_transformer_b200 import rtnf4
    stream = rtnf4.dumps(payloads[:1])
    entry = rtnf4.index(stream)[0]
    host = payloads[0]                      # 48 x 128, block 64, 16 blocks per second-level scale
    whole = rtnf4.load_weight(stream, entry, device="cpu")
    assert np.array_equal(whole.codes.numpy(), host.codes)
    assert np.array_equal(whole.primary.numpy(), host.scale_codes)
    assert whole.flat_block_base == 0 and whole.out_features == 48
    blocks_per_row = 128 // 64
    for rank in range(4):
        part = rtnf4.load_weight(stream, entry, device="cpu", rank=rank, world=4)
        rows = slice(12 * rank, 12 * (rank + 1))
        assert part.out_features == 12 and part.in_features == 128
        assert np.array_equal(part.codes.numpy(), host.codes[rows.start * 64:rows.stop * 64])
        assert np.array_equal(part.primary.numpy(),
                              host.scale_codes[rows.start * blocks_per_row:rows.stop * blocks_per_row])
        assert np.array_equal(part.secondary.numpy().view(np.uint32),
                              np.asarray(host.second_level, np.float32).view(np.uint32))
        assert part.flat_block_base == rows.start * blocks_per_row
    with pytest.raises(ValueError):
        rtnf4.load_weight(stream, entry, device="cpu", rank=0, world=5)     # 48 rows do not divide by 5


def _fields(dump: np.ndarray):
    """Weights of the field-by-field dump written beside each reference stream
    (ref_packed_model_fixture, oracle/ref_bridge.cpp)."""
    raw = dump.tobytes()
    count = struct.unpack_from("<Q", raw, 0)[0]
    at, out = 8, []
    for _ in range(count):
        o, i, block, n_codes, n_fp32, n_sc, n_second, sbs, offset_bits = struct.unpack_from("<9Q", raw, at)
        at += 72
        w = {"shape": (o, i), "block": block, "scale_block": sbs,
             "offset": np.array([offset_bits & 0xFFFFFFFF], np.uint32).view(np.float32)[0]}
        w["codes"] = np.frombuffer(raw, np.uint8, n_codes, at)
        at += n_codes
        w["fp32"] = np.frombuffer(raw, "<f4", n_fp32, at)
        at += 4 * n_fp32
        w["scale_codes"] = np.frombuffer(raw, np.uint8, n_sc, at)
        at += n_sc
        w["second"] = np.frombuffer(raw, "<f4", n_second, at)
        at += 4 * n_second
        out.append(w)
    assert at == len(raw)
    return out


@pytest.mark.parametrize("name,double_quantized", [("rtnf4_dq", True), ("rtnf4_f32", False)])
def test_streams_written_by_the_reference(golden, name, double_quantized):
    import oracle
    from riftco_transformer_b200 import rtnf4
    stream = golden[f"{name}_stream"]
    want = _fields(golden[f"{name}_fields"])
    entries = rtnf4.index(stream)
    # two blocks of six projections (q, k, v, o, expand, project) and the LM head
    assert len(entries) == len(want) == 13
    payloads = []
    for e, w in zip(entries, want):
        assert (e.out_features, e.in_features, e.block_size) == (*w["shape"], w["block"])
        assert bool(e.double_quantized) == double_quantized
        assert np.array_equal(stream[e.codes_offset:e.codes_offset + e.n_codes], w["codes"])
        if double_quantized:
            assert e.n_fp32_scales == 0 and e.scale_block_size == w["scale_block"]
            assert np.float32(e.offset).view(np.uint32) == np.float32(w["offset"]).view(np.uint32)
            assert np.array_equal(stream[e.scale_codes_offset:e.scale_codes_offset + e.n_scale_codes], w["scale_codes"])
            second = stream[e.second_offset:e.second_offset + 4 * e.n_second].view("<f4")
            assert np.array_equal(second.view(np.uint32), w["second"].view(np.uint32))
            payloads.append(oracle.Nf4Weight(w["codes"], *w["shape"], w["block"], scale_codes=w["scale_codes"],
                                             second_level=w["second"], scale_block_size=w["scale_block"],
                                             offset=float(w["offset"])))
        else:
            assert e.n_scale_codes == 0 and e.n_second == 0 and e.offset == 0.0
            scales = stream[e.fp32_scales_offset:e.fp32_scales_offset + 4 * e.n_fp32_scales].view("<f4")
            assert np.array_equal(scales.view(np.uint32), w["fp32"].view(np.uint32))
            payloads.append(oracle.Nf4Weight(w["codes"], *w["shape"], w["block"], fp32_scales=w["fp32"]))
        # a weight loaded from the stream is the reference's payload (CPU device, whole and row-sharded)
        whole = rtnf4.load_weight(stream, e, device="cpu")
        assert np.array_equal(whole.codes.numpy(), w["codes"])
        half = rtnf4.load_weight(stream, e, device="cpu", rank=1, world=2)
        rows = e.out_features // 2
        assert np.array_equal(half.codes.numpy(), w["codes"][rows * e.in_features // 2:])
        assert half.flat_block_base == rows * e.in_features // e.block_size
    # the writer of this repository reproduces the reference's stream byte for byte
    assert rtnf4.dumps(payloads) == stream.tobytes()
