"""RTNF4S1 packed-model-state streams: the reference's canonical on-disk / wire
form of packed NF4 linear weights (packed_model_state_bytes and
parse_packed_model_state, src/c_api/model_state.cpp:27-113, 165-297; weights are
stored per block as q, k, v, o, expand, project and then the LM head,
src/model/decoder_only_transformer.cpp:902-932).

``index`` validates a stream with the library's C parser (no GPU needed) and
says where every array lies; ``load_weight`` copies one weight, or a row shard
of it, straight from the stream into device memory as a ``PackedNf4Weight`` -
codes and scales stay packed, nothing is expanded to FP32; ``dumps`` writes a
stream from host payloads (tools and tests).
"""
from __future__ import annotations

import ctypes as C
import struct
from dataclasses import dataclass

import numpy as np

MAGIC = b"RTNF4S1\0"


class _Entry(C.Structure):
    _fields_ = [("block_size", C.c_uint64), ("out_features", C.c_uint64), ("in_features", C.c_uint64),
                ("n_codes", C.c_uint64), ("n_fp32_scales", C.c_uint64), ("n_scale_codes", C.c_uint64),
                ("n_second", C.c_uint64), ("scale_block_size", C.c_uint64), ("offset", C.c_float),
                ("double_quantized", C.c_uint32), ("codes_offset", C.c_uint64),
                ("fp32_scales_offset", C.c_uint64), ("scale_codes_offset", C.c_uint64),
                ("second_offset", C.c_uint64)]


@dataclass(frozen=True)
class Entry:
    block_size: int
    out_features: int
    in_features: int
    n_codes: int
    n_fp32_scales: int
    n_scale_codes: int
    n_second: int
    scale_block_size: int
    offset: float
    double_quantized: bool
    codes_offset: int
    fp32_scales_offset: int
    scale_codes_offset: int
    second_offset: int


def _as_bytes(stream) -> np.ndarray:
    if isinstance(stream, np.ndarray):
        if stream.dtype != np.uint8 or stream.ndim != 1:
            raise TypeError("an RTNF4S1 stream must be a flat uint8 array")
        return np.ascontiguousarray(stream)
    return np.frombuffer(memoryview(stream), dtype=np.uint8)


def index(stream) -> list[Entry]:
    """Validates `stream` (bytes, bytearray, memoryview, mmap or uint8 array) like
    the reference parser and returns one Entry per weight. Raises ValueError /
    OverflowError with the reference's messages on a malformed stream."""
    from ._lib import lib
    from .backend import _check
    buf = _as_bytes(stream)
    base = buf.ctypes.data_as(C.c_void_p)
    count = C.c_uint64(0)
    _check(lib.b2_rtnf4_index(base, buf.size, None, 0, C.byref(count)))
    table = (_Entry * count.value)()
    _check(lib.b2_rtnf4_index(base, buf.size, table, count.value, C.byref(count)))
    return [Entry(e.block_size, e.out_features, e.in_features, e.n_codes, e.n_fp32_scales, e.n_scale_codes,
                  e.n_second, e.scale_block_size, float(e.offset), bool(e.double_quantized), e.codes_offset,
                  e.fp32_scales_offset, e.scale_codes_offset, e.second_offset) for e in table]


def load_weight(stream, entry: Entry, device="cuda", rank: int = 0, world: int = 1):
    """Entry `entry` of `stream` as a device-resident PackedNf4Weight; with
    world > 1 only the rows [rank*out/world, (rank+1)*out/world) are copied (the
    second-level scales are shared by all rows and copied whole, the shard keeps
    the parent's block numbering through ``flat_block_base``)."""
    import torch

    from . import _lib
    from .backend import PackedNf4Weight
    buf = _as_bytes(stream)
    out_f, in_f, block = entry.out_features, entry.in_features, entry.block_size
    numel = out_f * in_f
    if block == 0 or entry.n_codes != (numel + 1) // 2:
        raise ValueError("RTNF4S1 entry: packed code count does not match its dimensions")
    blocks = -(-numel // block)
    if out_f % world != 0:
        raise ValueError("output features must divide evenly over the ranks")
    rows = out_f // world
    first, count = rank * rows * in_f, rows * in_f
    if world > 1 and (first % block != 0 or count % block != 0 or first % 2 != 0):
        raise ValueError("row shards must start and end on NF4 block boundaries")
    b0, nb = (first // block, count // block) if world > 1 else (0, blocks)

    def upload(offset: int, nbytes: int, dtype):
        host = np.ascontiguousarray(buf[offset:offset + nbytes]).view(dtype)
        return torch.from_numpy(host.copy()).to(device)

    codes = upload(entry.codes_offset + first // 2, (count + 1) // 2, np.uint8)
    if not entry.double_quantized:
        if entry.n_fp32_scales != blocks:
            raise ValueError("RTNF4S1 entry: block scale count does not match its dimensions")
        primary = upload(entry.fp32_scales_offset + 4 * b0, 4 * nb, "<f4")
        return PackedNf4Weight(codes, primary, None, _lib.SCALES_FLOAT32, block, 0, 0.0, rows, in_f, b0)
    groups = -(-blocks // entry.scale_block_size)
    if entry.n_scale_codes != blocks or entry.n_second != groups:
        raise ValueError("RTNF4S1 entry: scale code counts do not match its dimensions")
    primary = upload(entry.scale_codes_offset + b0, nb, np.uint8)
    secondary = upload(entry.second_offset, 4 * entry.n_second, "<f4")
    return PackedNf4Weight(codes, primary, secondary, _lib.SCALES_DOUBLE_QUANTIZED_UINT8, block,
                           entry.scale_block_size, entry.offset, rows, in_f, b0)


def dumps(payloads) -> bytes:
    """Stream of the given host payloads (objects with codes, block_size,
    out_features, in_features and either fp32_scales or scale_codes +
    second_level + scale_block_size + offset), byte for byte as
    packed_model_state_bytes lays it out."""
    out = bytearray(MAGIC)
    out += struct.pack("<Q", len(payloads))
    for p in payloads:
        codes = np.ascontiguousarray(p.codes, np.uint8)
        dq = getattr(p, "fp32_scales", None) is None
        fp32 = np.zeros(0, "<f4") if dq else np.ascontiguousarray(p.fp32_scales, "<f4")
        scale_codes = np.ascontiguousarray(p.scale_codes, np.uint8) if dq else np.zeros(0, np.uint8)
        second = np.ascontiguousarray(p.second_level, "<f4") if dq else np.zeros(0, "<f4")
        out += struct.pack("<QQQQQQQ", 2, int(p.block_size), codes.size, fp32.size, scale_codes.size, second.size,
                           int(p.scale_block_size) if dq else 0)
        out += struct.pack("<fI", float(p.offset) if dq else 0.0, 1 if dq else 0)
        out += struct.pack("<QQ", int(p.out_features), int(p.in_features))
        out += codes.tobytes() + fp32.tobytes() + scale_codes.tobytes() + second.tobytes()
    return bytes(out)
