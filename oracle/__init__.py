"""CPU checkers for the NF4-linear / paged-decode path (test infrastructure).

Only the tests, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py`` may import this package. The product package never does.

``port``  - the C restatement (``riftco_oracle.c``), always available.
``ref``   - the reference project's own CPU code behind ``ref_bridge.cpp``,
            available where ``oracle/_ref/libriftco_ref.so`` was built.
Both expose the same numpy-level functions, so a test can run one against the
other.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from pathlib import Path

import numpy as np

from . import build as _build

SCALES_FLOAT32 = 0
SCALES_DOUBLE_QUANTIZED_UINT8 = 1

_u8p = C.POINTER(C.c_uint8)
_f32p = C.POINTER(C.c_float)
_u32p = C.POINTER(C.c_uint32)


@dataclass
class Nf4Weight:
    """Canonical host payload of one packed weight (Nf4Payload in the
    reference, include/riftco_transformer/core/quantized_weight.hpp:40-48)."""

    codes: np.ndarray                 # uint8 [ceil(out*in/2)]
    out_features: int
    in_features: int
    block_size: int
    fp32_scales: np.ndarray | None = None     # float32 [blocks]
    scale_codes: np.ndarray | None = None     # uint8 [blocks]
    second_level: np.ndarray | None = None    # float32 [ceil(blocks/scale_block)]
    scale_block_size: int = 0
    offset: float = 0.0

    @property
    def encoding(self) -> int:
        return SCALES_FLOAT32 if self.fp32_scales is not None else SCALES_DOUBLE_QUANTIZED_UINT8

    @property
    def numel(self) -> int:
        return self.out_features * self.in_features

    @property
    def blocks(self) -> int:
        return -(-self.numel // self.block_size)

    @property
    def scale_bytes(self) -> int:
        """nf4_scale_payload_bytes, quantized_linear/storage.hpp:67-75."""
        if self.encoding == SCALES_FLOAT32:
            return 4 * self.blocks
        return self.blocks + 4 * len(self.second_level) + 4

    @property
    def payload_bytes(self) -> int:
        return len(self.codes) + self.scale_bytes


def _ptr(a: np.ndarray | None, typ):
    if a is None:
        return C.cast(None, typ)
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(typ)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


class _OrcWeight(C.Structure):
    _fields_ = [
        ("codes", _u8p),
        ("fp32_scales", _f32p),
        ("scale_codes", _u8p),
        ("second_level", _f32p),
        ("scale_block_size", C.c_uint64),
        ("offset", C.c_float),
        ("encoding", C.c_uint32),
        ("block_size", C.c_uint64),
        ("out_features", C.c_uint64),
        ("in_features", C.c_uint64),
    ]


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


class Port:
    """ctypes face of riftco_oracle.c."""

    kind = "port"

    def __init__(self) -> None:
        # RIFTCO_ORACLE_SANITIZE=1: the ASan + UBSan build (the process must preload libasan)
        self.lib = C.CDLL(str(_build.build_oracle(sanitize=os.environ.get("RIFTCO_ORACLE_SANITIZE") == "1")))
        L = self.lib
        L.orc_nf4_codebook.restype = _f32p
        L.orc_nearest_nf4_code.restype = C.c_uint8
        L.orc_nearest_nf4_code.argtypes = [C.c_float]
        L.orc_pack_nf4.argtypes = [_f32p, C.c_size_t, C.c_size_t, _u8p, _f32p]
        L.orc_double_quantize_scales.argtypes = [_f32p, C.c_size_t, C.c_size_t, _u8p, _f32p, _f32p]
        L.orc_decode_block_scale.restype = C.c_float
        L.orc_decode_block_scale.argtypes = [C.POINTER(_OrcWeight), C.c_size_t]
        L.orc_nf4_dequantize.argtypes = [C.POINTER(_OrcWeight), _f32p]
        L.orc_nf4_linear_forward.argtypes = [C.POINTER(_OrcWeight), _f32p, _f32p, C.c_size_t, C.c_int]
        L.orc_nf4_linear_input_backward.argtypes = [C.POINTER(_OrcWeight), _f32p, _f32p, C.c_size_t, C.c_int]
        L.orc_paged_decode.argtypes = [_f32p, _f32p, _f32p, _u32p, _f32p] + [C.c_size_t] * 4
        L.orc_paged_decode_gqa.argtypes = (
            [_f32p, _f32p, _f32p, _u32p, _u32p, _f32p] + [C.c_size_t] * 6 + [C.c_int]
        )
        L.orc_rms_norm.argtypes = [_f32p, _f32p, C.c_size_t, C.c_size_t, C.c_float, _f32p]
        L.orc_silu_mul.argtypes = [_f32p, _f32p, C.c_size_t, _f32p]
        L.orc_greedy.restype = C.c_size_t
        L.orc_greedy.argtypes = [_f32p, C.c_size_t]
        L.orc_lora_forward.argtypes = [_f32p, _f32p, _f32p] + [C.c_size_t] * 4 + [C.c_float, _f32p, _f32p]

    # -- format ---------------------------------------------------------
    def codebook(self) -> np.ndarray:
        return np.ctypeslib.as_array(self.lib.orc_nf4_codebook(), shape=(16,)).copy()

    def nearest_code(self, v: float) -> int:
        return int(self.lib.orc_nearest_nf4_code(np.float32(v)))

    def quantize_nf4(self, values, block_size: int = 64) -> Nf4Weight:
        v = _f32(values)
        out_f, in_f = (v.shape if v.ndim == 2 else (1, v.size))
        n = v.size
        codes = np.zeros((n + 1) // 2, np.uint8)
        scales = np.zeros(-(-n // block_size), np.float32)
        rc = self.lib.orc_pack_nf4(_ptr(v, _f32p), n, block_size, _ptr(codes, _u8p), _ptr(scales, _f32p))
        if rc:
            raise ValueError("NF4 source values must be finite")
        return Nf4Weight(codes, out_f, in_f, block_size, fp32_scales=scales)

    def quantize_nf4_double_quantized(self, values, block_size: int = 64,
                                      scale_block_size: int = 256) -> Nf4Weight:
        w = self.quantize_nf4(values, block_size)
        s = w.fp32_scales
        qs = np.zeros(len(s), np.uint8)
        second = np.zeros(-(-len(s) // scale_block_size), np.float32)
        off = C.c_float(0)
        rc = self.lib.orc_double_quantize_scales(
            _ptr(s, _f32p), len(s), scale_block_size, _ptr(qs, _u8p), _ptr(second, _f32p), C.byref(off))
        if rc:
            raise OverflowError("NF4 scale mean exceeds the FP32 double-quantization range")
        return Nf4Weight(w.codes, w.out_features, w.in_features, block_size, scale_codes=qs,
                         second_level=second, scale_block_size=scale_block_size, offset=float(off.value))

    def double_quantize_payload(self, codes, scales, out_features: int, in_features: int, block_size: int = 64,
                                scale_block_size: int = 256) -> Nf4Weight:
        """A double-quantised payload from packed codes and FP32 block scales already in hand (synthetic
        payloads drawn in the packed domain): only the scales go through double_quantize_scales."""
        s = _f32(scales)
        qs = np.zeros(len(s), np.uint8)
        second = np.zeros(-(-len(s) // scale_block_size), np.float32)
        off = C.c_float(0)
        rc = self.lib.orc_double_quantize_scales(
            _ptr(s, _f32p), len(s), scale_block_size, _ptr(qs, _u8p), _ptr(second, _f32p), C.byref(off))
        if rc:
            raise OverflowError("NF4 scale mean exceeds the FP32 double-quantization range")
        return Nf4Weight(np.ascontiguousarray(codes, np.uint8), out_features, in_features, block_size,
                         scale_codes=qs, second_level=second, scale_block_size=scale_block_size,
                         offset=float(off.value))

    def _cw(self, w: Nf4Weight) -> _OrcWeight:
        return _OrcWeight(
            _ptr(w.codes, _u8p), _ptr(w.fp32_scales, _f32p), _ptr(w.scale_codes, _u8p),
            _ptr(w.second_level, _f32p), w.scale_block_size, w.offset, w.encoding,
            w.block_size, w.out_features, w.in_features)

    def decode_scales(self, w: Nf4Weight) -> np.ndarray:
        cw = self._cw(w)
        return np.array([self.lib.orc_decode_block_scale(C.byref(cw), b) for b in range(w.blocks)], np.float32)

    def dequantize(self, w: Nf4Weight) -> np.ndarray:
        out = np.empty((w.out_features, w.in_features), np.float32)
        cw = self._cw(w)
        self.lib.orc_nf4_dequantize(C.byref(cw), _ptr(out, _f32p))
        return out

    # -- operators ------------------------------------------------------
    def linear_forward(self, w: Nf4Weight, x, threads: int = 0) -> np.ndarray:
        x = _f32(x).reshape(-1, w.in_features)
        y = np.empty((x.shape[0], w.out_features), np.float32)
        cw = self._cw(w)
        self.lib.orc_nf4_linear_forward(C.byref(cw), _ptr(x, _f32p), _ptr(y, _f32p), x.shape[0],
                                        threads or host_threads())
        return y

    def linear_input_backward(self, w: Nf4Weight, dy, threads: int = 0) -> np.ndarray:
        dy = _f32(dy).reshape(-1, w.out_features)
        dx = np.empty((dy.shape[0], w.in_features), np.float32)
        cw = self._cw(w)
        self.lib.orc_nf4_linear_input_backward(C.byref(cw), _ptr(dy, _f32p), _ptr(dx, _f32p), dy.shape[0],
                                               threads or host_threads())
        return dx

    def paged_decode(self, q, key_pages, value_pages, block_table, seq_len: int) -> np.ndarray:
        """One sequence, MHA: q [heads, d], pages [P, heads, bs, d]."""
        q = _f32(q)
        k, v = _f32(key_pages), _f32(value_pages)
        _, heads, bs, d = k.shape
        t = np.ascontiguousarray(block_table, np.uint32)
        ctx = np.empty((heads, d), np.float32)
        rc = self.lib.orc_paged_decode(_ptr(q, _f32p), _ptr(k, _f32p), _ptr(v, _f32p), _ptr(t, _u32p),
                                       _ptr(ctx, _f32p), heads, d, bs, seq_len)
        if rc:
            raise FloatingPointError("softmax rejects NaN and positive infinity" if rc == 1
                                     else "softmax requires one finite value per slice")
        return ctx

    def paged_decode_gqa(self, q, key_pages, value_pages, block_tables, seq_lens,
                         threads: int = 0) -> np.ndarray:
        """q [n_seq, Hq, d], pages [P, Hkv, bs, d], tables [n_seq, max_blocks]."""
        q = _f32(q)
        k, v = _f32(key_pages), _f32(value_pages)
        n_seq, hq, d = q.shape
        _, hkv, bs, _ = k.shape
        t = np.ascontiguousarray(block_tables, np.uint32)
        lens = np.ascontiguousarray(seq_lens, np.uint32)
        ctx = np.empty((n_seq, hq, d), np.float32)
        rc = self.lib.orc_paged_decode_gqa(
            _ptr(q, _f32p), _ptr(k, _f32p), _ptr(v, _f32p), _ptr(t, _u32p), _ptr(lens, _u32p),
            _ptr(ctx, _f32p), n_seq, hq, hkv, d, bs, t.shape[1], threads or host_threads())
        if rc:
            raise FloatingPointError("paged decode attention received non-finite scores")
        return ctx


    # -- decode-step primitives --------------------------------------------
    def rms_norm(self, x, scale, eps: float) -> np.ndarray:
        x, scale = _f32(x), _f32(scale)
        out = np.empty_like(x)
        x2 = x.reshape(-1, x.shape[-1])
        self.lib.orc_rms_norm(_ptr(x2, _f32p), _ptr(scale, _f32p), x2.shape[0], x2.shape[1], eps, _ptr(out, _f32p))
        return out

    def silu_mul(self, gate, up=None) -> np.ndarray:
        g = _f32(gate)
        u = None if up is None else _f32(up)
        out = np.empty_like(g)
        self.lib.orc_silu_mul(_ptr(g, _f32p), _ptr(u, _f32p), g.size, _ptr(out, _f32p))
        return out

    def greedy(self, logits) -> int:
        v = _f32(logits).ravel()
        return int(self.lib.orc_greedy(_ptr(v, _f32p), v.size))

    def lora_forward(self, x, a, b, scale: float) -> np.ndarray:
        """((x A^T) B^T) * scale: x [rows, in], a [rank, in], b [out, rank]."""
        x, a, b = _f32(x), _f32(a), _f32(b)
        rows, in_f = x.shape
        rank, out_f = a.shape[0], b.shape[0]
        reduced = np.empty((rows, rank), np.float32)
        out = np.empty((rows, out_f), np.float32)
        self.lib.orc_lora_forward(_ptr(x, _f32p), _ptr(a, _f32p), _ptr(b, _f32p), rows, in_f, out_f, rank, scale,
                                  _ptr(reduced, _f32p), _ptr(out, _f32p))
        return out


class ReferenceError_(RuntimeError):
    def __init__(self, status: int, message: str) -> None:
        super().__init__(f"[status {status}] {message}")
        self.status = status


class Reference:
    """ctypes face of the reference's own CPU code (oracle/_ref)."""

    kind = "reference"

    def __init__(self, path=None) -> None:
        if path is None:
            path = _build.build_reference()
        if path is None or not Path(path).exists():
            raise FileNotFoundError("oracle/_ref/libriftco_ref.so is not built and no reference checkout is present")
        self.lib = C.CDLL(str(path))
        L = self.lib
        L.ref_last_error.restype = C.c_char_p
        L.ref_nearest_nf4_code.restype = C.c_uint8
        L.ref_nearest_nf4_code.argtypes = [C.c_float]
        u64 = C.c_uint64
        wargs = [_u8p, _f32p, _u8p, _f32p, u64, C.c_float, C.c_uint32, u64, u64, u64]
        L.ref_quantize_nf4.argtypes = [_f32p, u64, u64, u64, _u8p, _f32p]
        L.ref_quantize_nf4_double_quantized.argtypes = [_f32p, u64, u64, u64, u64, _u8p, _u8p, _f32p, _f32p]
        L.ref_dequantize.argtypes = wargs + [_f32p]
        L.ref_linear_forward.argtypes = wargs + [_f32p, _f32p, u64, C.POINTER(C.c_double)]
        L.ref_linear_input_backward.argtypes = wargs + [_f32p, _f32p, u64, C.POINTER(C.c_double)]
        L.ref_paged_decode.argtypes = [_f32p, _f32p, _f32p, _u32p, u64, _f32p, u64, u64, u64, u64, u64,
                                       C.POINTER(C.c_double)]
        L.ref_materialized_causal_forward.argtypes = [_f32p, _f32p, _f32p, _f32p, _f32p, u64, u64, u64, u64]
        if hasattr(L, "ref_rms_norm"):   # decode-step primitives and the packed model state
            L.ref_rms_norm.argtypes = [_f32p, _f32p, u64, u64, C.c_float, _f32p]
            L.ref_rope.argtypes = [_f32p, u64, u64, u64, u64, u64, C.c_float, _f32p]
            L.ref_silu_mul.argtypes = [_f32p, _f32p, u64, _f32p]
            L.ref_greedy.argtypes = [_f32p, u64, _u32p]
            L.ref_paged_cache_decode.argtypes = [_f32p, _f32p, _f32p, u64, u64, u64, u64, u64, _f32p]
            L.ref_packed_model_fixture.argtypes = [u64, u64, u64, u64, u64, u64, u64, u64, C.c_uint32,
                                                   _u8p, u64, C.POINTER(u64), _u8p, u64, C.POINTER(u64)]
        if hasattr(L, "ref_lora_forward"):
            L.ref_lora_forward.argtypes = [_f32p, _f32p, _f32p, u64, u64, u64, u64, C.c_float, _f32p]
        self.last_seconds = 0.0

    def _check(self, rc: int) -> None:
        if rc:
            raise ReferenceError_(rc, self.lib.ref_last_error().decode())

    def codebook(self) -> np.ndarray:
        out = np.empty(16, np.float32)
        self.lib.ref_codebook(_ptr(out, _f32p))
        return out

    def nearest_code(self, v: float) -> int:
        return int(self.lib.ref_nearest_nf4_code(np.float32(v)))

    def quantize_nf4(self, values, block_size: int = 64) -> Nf4Weight:
        v = _f32(values)
        out_f, in_f = (v.shape if v.ndim == 2 else (1, v.size))
        codes = np.zeros((v.size + 1) // 2, np.uint8)
        scales = np.zeros(-(-v.size // block_size), np.float32)
        self._check(self.lib.ref_quantize_nf4(_ptr(v, _f32p), out_f, in_f, block_size,
                                              _ptr(codes, _u8p), _ptr(scales, _f32p)))
        return Nf4Weight(codes, out_f, in_f, block_size, fp32_scales=scales)

    def quantize_nf4_double_quantized(self, values, block_size: int = 64,
                                      scale_block_size: int = 256) -> Nf4Weight:
        v = _f32(values)
        out_f, in_f = (v.shape if v.ndim == 2 else (1, v.size))
        blocks = -(-v.size // block_size)
        codes = np.zeros((v.size + 1) // 2, np.uint8)
        qs = np.zeros(blocks, np.uint8)
        second = np.zeros(-(-blocks // scale_block_size), np.float32)
        off = C.c_float(0)
        self._check(self.lib.ref_quantize_nf4_double_quantized(
            _ptr(v, _f32p), out_f, in_f, block_size, scale_block_size, _ptr(codes, _u8p), _ptr(qs, _u8p),
            _ptr(second, _f32p), C.byref(off)))
        return Nf4Weight(codes, out_f, in_f, block_size, scale_codes=qs, second_level=second,
                         scale_block_size=scale_block_size, offset=float(off.value))

    def _wargs(self, w: Nf4Weight):
        return (_ptr(w.codes, _u8p), _ptr(w.fp32_scales, _f32p), _ptr(w.scale_codes, _u8p),
                _ptr(w.second_level, _f32p), w.scale_block_size, w.offset, w.encoding, w.block_size,
                w.out_features, w.in_features)

    def dequantize(self, w: Nf4Weight) -> np.ndarray:
        out = np.empty((w.out_features, w.in_features), np.float32)
        self._check(self.lib.ref_dequantize(*self._wargs(w), _ptr(out, _f32p)))
        return out

    def linear_forward(self, w: Nf4Weight, x, threads: int = 1) -> np.ndarray:
        x = _f32(x).reshape(-1, w.in_features)
        y = np.empty((x.shape[0], w.out_features), np.float32)
        sec = C.c_double(0)
        self._check(self.lib.ref_linear_forward(*self._wargs(w), _ptr(x, _f32p), _ptr(y, _f32p),
                                                x.shape[0], C.byref(sec)))
        self.last_seconds = sec.value
        return y

    def linear_input_backward(self, w: Nf4Weight, dy, threads: int = 1) -> np.ndarray:
        dy = _f32(dy).reshape(-1, w.out_features)
        dx = np.empty((dy.shape[0], w.in_features), np.float32)
        sec = C.c_double(0)
        self._check(self.lib.ref_linear_input_backward(*self._wargs(w), _ptr(dy, _f32p), _ptr(dx, _f32p),
                                                       dy.shape[0], C.byref(sec)))
        self.last_seconds = sec.value
        return dx

    def paged_decode(self, q, key_pages, value_pages, block_table, seq_len: int,
                     physical_blocks: int | None = None) -> np.ndarray:
        q = _f32(q)
        k, v = _f32(key_pages), _f32(value_pages)
        p, heads, bs, d = k.shape
        t = np.ascontiguousarray(block_table, np.uint32)
        ctx = np.empty((heads, d), np.float32)
        sec = C.c_double(0)
        self._check(self.lib.ref_paged_decode(
            _ptr(q, _f32p), _ptr(k, _f32p), _ptr(v, _f32p), _ptr(t, _u32p), len(t), _ptr(ctx, _f32p),
            heads, d, bs, physical_blocks if physical_blocks is not None else p, seq_len, C.byref(sec)))
        self.last_seconds = sec.value
        return ctx

    def paged_decode_gqa(self, q, key_pages, value_pages, block_tables, seq_lens, threads: int = 1) -> np.ndarray:
        """Grouped-query batch through the UNMODIFIED single-sequence operator:
        for j in [0, rep) call it with heads = Hkv and queries Q[:, j::rep]."""
        q = _f32(q)
        n_seq, hq, d = q.shape
        hkv, bs = key_pages.shape[1], key_pages.shape[2]
        rep = hq // hkv
        ctx = np.empty_like(q)
        total = 0.0
        for s in range(n_seq):
            n = int(seq_lens[s])
            table = np.ascontiguousarray(block_tables[s][: -(-n // bs)], np.uint32)
            for j in range(rep):
                sub = np.ascontiguousarray(q[s, j::rep])
                ctx[s, j::rep] = self.paged_decode(sub, key_pages, value_pages, table, n)
                total += self.last_seconds
        self.last_seconds = total
        return ctx

    def materialized_causal_forward(self, q, k, v):
        q, k, v = _f32(q), _f32(k), _f32(v)
        b, h, t, d = q.shape
        probs = np.empty((b, h, t, t), np.float32)
        ctx = np.empty_like(q)
        self._check(self.lib.ref_materialized_causal_forward(
            _ptr(q, _f32p), _ptr(k, _f32p), _ptr(v, _f32p), _ptr(probs, _f32p), _ptr(ctx, _f32p), b, h, t, d))
        return probs, ctx


    # ---- decode-step primitives (reference entry points named in oracle/ref_bridge.cpp) ----

    def rms_norm(self, x, scale, eps: float) -> np.ndarray:
        x, scale = _f32(x), _f32(scale)
        out = np.empty_like(x)
        self._check(self.lib.ref_rms_norm(_ptr(x, _f32p), _ptr(scale, _f32p), x.shape[0], x.shape[1], eps,
                                          _ptr(out, _f32p)))
        return out

    def rope(self, x, position_offset: int, theta: float) -> np.ndarray:
        """x [batch, heads, time, width]; token t of the time axis is at position_offset + t."""
        x = _f32(x)
        out = np.empty_like(x)
        b, h, t, w = x.shape
        self._check(self.lib.ref_rope(_ptr(x, _f32p), b, h, t, w, position_offset, theta, _ptr(out, _f32p)))
        return out

    def silu_mul(self, gate, up=None) -> np.ndarray:
        gate = _f32(gate).ravel()
        up_ = None if up is None else _f32(up).ravel()
        out = np.empty_like(gate)
        self._check(self.lib.ref_silu_mul(_ptr(gate, _f32p), _ptr(up_, _f32p), gate.size, _ptr(out, _f32p)))
        return out

    def greedy(self, logits) -> int:
        logits = _f32(logits).ravel()
        token = np.zeros(1, np.uint32)
        self._check(self.lib.ref_greedy(_ptr(logits, _f32p), logits.size, _ptr(token, _u32p)))
        return int(token[0])

    def paged_cache_decode(self, q, k, v, block_size: int, block_count: int) -> np.ndarray:
        """q, k, v [steps, heads, width] of one sequence fed token by token through the reference's
        paged KV cache; returns the attention context after each append."""
        q, k, v = _f32(q), _f32(k), _f32(v)
        steps, heads, width = q.shape
        ctx = np.empty_like(q)
        self._check(self.lib.ref_paged_cache_decode(_ptr(q, _f32p), _ptr(k, _f32p), _ptr(v, _f32p), steps, heads,
                                                    width, block_size, block_count, _ptr(ctx, _f32p)))
        return ctx

    def lora_forward(self, x, a, b, scale: float) -> np.ndarray:
        x, a, b = _f32(x), _f32(a), _f32(b)
        out = np.empty((x.shape[0], b.shape[0]), np.float32)
        self._check(self.lib.ref_lora_forward(_ptr(x, _f32p), _ptr(a, _f32p), _ptr(b, _f32p), x.shape[0], x.shape[1],
                                              b.shape[0], a.shape[0], scale, _ptr(out, _f32p)))
        return out

    def packed_model_fixture(self, vocabulary, context, width, heads, blocks, feed_forward, block_size,
                             scale_block_size, seed):
        """(RTNF4S1 stream, field-by-field dump) of a small quantised decoder, both as uint8 arrays."""
        n1, n2 = C.c_uint64(0), C.c_uint64(0)
        args = (vocabulary, context, width, heads, blocks, feed_forward, block_size, scale_block_size, seed)
        self._check(self.lib.ref_packed_model_fixture(*args, None, 0, C.byref(n1), None, 0, C.byref(n2)))
        stream, dump = np.empty(n1.value, np.uint8), np.empty(n2.value, np.uint8)
        self._check(self.lib.ref_packed_model_fixture(*args, _ptr(stream, _u8p), stream.size, C.byref(n1),
                                                      _ptr(dump, _u8p), dump.size, C.byref(n2)))
        return stream, dump


_port: Port | None = None
_ref: Reference | None = None


def port() -> Port:
    global _port
    if _port is None:
        _port = Port()
    return _port


def ref() -> Reference:
    global _ref
    if _ref is None:
        _ref = Reference()
    return _ref


def ref_with_b200_adapter() -> Reference:
    """The reference's core linked with the product's CUDA adapter
    (riftco_transformer_b200/adapter/cuda_b200_adapter.cpp) and switched to
    ExecutionBackend::Cuda: the reference's own dispatch layer in front of the
    B200 kernels. Test infrastructure, like everything in this package."""
    path = _build.build_reference_with_b200_adapter()
    if path is None or not Path(path).exists():
        raise FileNotFoundError("oracle/_ref/libriftco_ref_b200.so is not built and no reference checkout is present")
    r = Reference(path)
    r.lib.ref_set_backend.argtypes = [C.c_int]
    if r.lib.ref_set_backend(2) != 0:
        raise RuntimeError("the CUDA backend is not available behind the reference's dispatch layer")
    return r


def ref_available() -> bool:
    try:
        ref()
        return True
    except (FileNotFoundError, OSError):
        return False
