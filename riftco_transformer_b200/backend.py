"""Host-side mirror of the reference's backend operator interface for the hot
path, on top of the C ABI in ``include/riftco_b200.h``.

Names and argument meaning follow the reference's dispatch layer:

* ``dispatch_quantized_linear_forward`` / ``..._input_backward`` -
  src/core/backend/nn/quantized_linear/dispatch.cpp:317-370 with
  ``QuantizedLinearDimensions`` (contracts.hpp:10-15) as a 4-tuple
  ``(rows, input_width, output_width, block_size)``.
* ``dispatch_paged_decode_attention_forward`` -
  src/core/backend/attention/dispatch.cpp:440-509 with
  ``PagedDecodeAttentionDimensions`` (contracts.hpp:91-97) as
  ``(heads, head_width, block_size, physical_block_count, sequence_length)``.
* ``PackedNf4Weight`` plays ``QuantizedWeightStorage`` (storage.hpp:81-108):
  immutable device-resident codes and scales in the reference's packed layout.

C++ exception types map to Python ones: ``std::invalid_argument`` ->
``ValueError``, ``std::out_of_range`` -> ``IndexError``, ``std::overflow_error``
-> ``OverflowError``, ``std::bad_alloc`` -> ``MemoryError``, ``std::logic_error``
/ ``std::runtime_error`` -> ``RuntimeError``, ``std::domain_error`` ->
``DomainError``.

torch is used for device memory and streams only; all arithmetic happens in
the CUDA library.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib
from ._lib import Nf4WeightStruct, lib


class DomainError(ArithmeticError):
    """std::domain_error: attention scores were not finite."""


class BackendUnavailable(RuntimeError):
    """The CUDA backend cannot run here (no sm_100 device)."""


def _raise(status: int) -> None:
    message = lib.b2_last_error().decode()
    if status == _lib.STATUS_INVALID_ARGUMENT:
        raise ValueError(message)
    if status == _lib.STATUS_OUT_OF_RANGE:
        raise IndexError(message)
    if status == _lib.STATUS_OVERFLOW:
        raise OverflowError(message)
    if status == _lib.STATUS_BACKEND_UNAVAILABLE:
        raise BackendUnavailable(message)
    if status == _lib.STATUS_OUT_OF_MEMORY:
        raise MemoryError(message)
    if status == _lib.STATUS_DOMAIN_ERROR:
        raise DomainError(message)
    raise RuntimeError(message)


def _check(status: int) -> None:
    if status != _lib.STATUS_OK:
        _raise(status)


def is_available() -> bool:
    return bool(lib.b2_is_available())


def unavailability_reason() -> str:
    return lib.b2_unavailability_reason().decode()


def check_device_errors() -> None:
    """Synchronises and raises if an earlier asynchronous call flagged a device-side failure."""
    _check(lib.b2_check_device_errors())


ROUTES = ("none", "decode_tmem", "gemv_tma", "gemv_tile", "gemm_tmem", "gemm_smem", "backward_dense",
          "generic", "attention_bulk", "attention_generic")


def last_route() -> str:
    """The kernel family that served this thread's last linear or attention call
    (B2_ROUTE_* of the header, by name)."""
    return ROUTES[lib.b2_last_route()]


def _stream_ptr(stream) -> int:
    if stream is None:
        stream = torch.cuda.current_stream()
    return int(stream.cuda_stream)


def _require_f32_cuda(t: torch.Tensor, what: str) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ValueError(f"{what} storage does not match its backend")
    if t.dtype != torch.float32 or not t.is_contiguous():
        raise ValueError(f"{what} must be contiguous float32")


@dataclass
class PackedNf4Weight:
    """Device-resident packed NF4 weight (QuantizedWeightStorage on CUDA).

    codes: uint8 [ceil(out*in/2)], low nibble = even flat index.
    primary: float32 [blocks] (FP32 scales) or uint8 [blocks] (scale codes).
    secondary: None or float32 [ceil(blocks/scale_block_size)].
    """

    codes: torch.Tensor
    primary: torch.Tensor
    secondary: torch.Tensor | None
    encoding: int
    block_size: int
    scale_block_size: int
    offset: float
    out_features: int
    in_features: int
    flat_block_base: int = 0

    @classmethod
    def from_host(cls, payload, device="cuda") -> "PackedNf4Weight":
        """payload: any object with the fields of the canonical host payload
        (codes, fp32_scales | scale_codes + second_level + scale_block_size +
        offset, block_size, out_features, in_features)."""
        codes = torch.from_numpy(np.ascontiguousarray(payload.codes)).to(device)
        if getattr(payload, "fp32_scales", None) is not None:
            primary = torch.from_numpy(np.ascontiguousarray(payload.fp32_scales, np.float32)).to(device)
            return cls(codes, primary, None, _lib.SCALES_FLOAT32, int(payload.block_size), 0, 0.0,
                       int(payload.out_features), int(payload.in_features))
        primary = torch.from_numpy(np.ascontiguousarray(payload.scale_codes, np.uint8)).to(device)
        secondary = torch.from_numpy(np.ascontiguousarray(payload.second_level, np.float32)).to(device)
        return cls(codes, primary, secondary, _lib.SCALES_DOUBLE_QUANTIZED_UINT8, int(payload.block_size),
                   int(payload.scale_block_size), float(payload.offset), int(payload.out_features),
                   int(payload.in_features))

    @property
    def numel(self) -> int:
        return self.out_features * self.in_features

    @property
    def blocks(self) -> int:
        return -(-self.numel // self.block_size)

    @property
    def device(self):
        return self.codes.device

    def scale_payload_bytes(self) -> int:
        """nf4_scale_payload_bytes, quantized_linear/storage.hpp:67-75."""
        if self.encoding == _lib.SCALES_FLOAT32:
            return 4 * self.blocks
        groups = -(-(self.flat_block_base % max(self.scale_block_size, 1) + self.blocks) // self.scale_block_size)
        return self.blocks + 4 * groups + 4

    def resident_payload_bytes(self) -> int:
        return (self.numel + 1) // 2 + self.scale_payload_bytes()

    def struct(self) -> Nf4WeightStruct:
        return Nf4WeightStruct(
            self.codes.data_ptr(), self.primary.data_ptr(),
            self.secondary.data_ptr() if self.secondary is not None else None,
            self.encoding, self.block_size, self.scale_block_size, self.offset, 0,
            self.out_features, self.in_features, self.flat_block_base)

    def row_shard(self, rank: int, world: int) -> "PackedNf4Weight":
        """Rows [rank*out/world, (rank+1)*out/world) of this weight as a view of
        the same packed bytes (no re-quantisation, so dequantised values are
        bit-identical to the parent's). Needs shard boundaries on whole bytes
        and whole blocks."""
        if self.out_features % world != 0:
            raise ValueError("output features must divide evenly over the ranks")
        rows = self.out_features // world
        first = rank * rows * self.in_features
        count = rows * self.in_features
        if first % self.block_size != 0 or count % self.block_size != 0:
            raise ValueError("row shards must start and end on NF4 block boundaries")
        b0, nb = first // self.block_size, count // self.block_size
        return PackedNf4Weight(
            self.codes[first // 2:(first + count) // 2], self.primary[b0:b0 + nb], self.secondary,
            self.encoding, self.block_size, self.scale_block_size, self.offset, rows, self.in_features,
            self.flat_block_base + b0)


def quantize_nf4(values: torch.Tensor, block_size: int = 64, scale_block_size: int = 0, stream=None) -> PackedNf4Weight:
    """QuantizedWeight::quantize_nf4 (scale_block_size == 0) / quantize_nf4_double_quantized on a
    device tensor [out, in]: the reference's encoder, bit for bit, by the library's own kernels."""
    _require_f32_cuda(values, "NF4 source")
    if values.dim() != 2:
        raise ValueError("NF4 quantization requires a matrix")
    out_f, in_f = values.shape
    n = out_f * in_f
    blocks = -(-n // block_size)
    dev = values.device
    codes = torch.empty((n + 1) // 2, dtype=torch.uint8, device=dev)
    dq = scale_block_size != 0
    primary = torch.empty(blocks, dtype=torch.uint8 if dq else torch.float32, device=dev)
    secondary = torch.empty(-(-blocks // scale_block_size), dtype=torch.float32, device=dev) if dq else None
    need = lib.b2_nf4_quantize_workspace_bytes(out_f, in_f, block_size, scale_block_size)
    workspace = torch.empty(max(need, 256), dtype=torch.uint8, device=dev)
    offset = C.c_float(0.0)
    _check(lib.b2_nf4_quantize(values.data_ptr(), out_f, in_f, block_size, scale_block_size, codes.data_ptr(),
                               primary.data_ptr(), None if secondary is None else secondary.data_ptr(),
                               C.byref(offset), workspace.data_ptr(), workspace.numel(), _stream_ptr(stream)))
    return PackedNf4Weight(codes, primary, secondary,
                           _lib.SCALES_DOUBLE_QUANTIZED_UINT8 if dq else _lib.SCALES_FLOAT32, block_size,
                           scale_block_size, float(offset.value), out_f, in_f)


def validate_payload(weight: PackedNf4Weight, stream=None) -> None:
    """require_canonical_payload of the reference for a device-resident payload; raises ValueError."""
    ws = weight.struct()
    _check(lib.b2_nf4_validate_payload(C.byref(ws), weight.codes.numel(), weight.primary.numel(),
                                       0 if weight.secondary is None else weight.secondary.numel(),
                                       _stream_ptr(stream)))


def dequantize(weight: PackedNf4Weight, stream=None) -> torch.Tensor:
    """QuantizedWeight::dequantize on the device, bit-exact."""
    out = torch.empty((weight.out_features, weight.in_features), dtype=torch.float32, device=weight.device)
    ws = weight.struct()
    _check(lib.b2_nf4_dequantize(C.byref(ws), out.data_ptr(), _stream_ptr(stream)))
    return out


def _check_linear(weight: PackedNf4Weight, dimensions) -> tuple[int, int, int, int]:
    rows, input_width, output_width, block_size = (int(v) for v in dimensions)
    if block_size == 0:
        raise ValueError("NF4 block size must be greater than zero")
    logical = output_width * input_width
    if weight.codes.numel() != (logical + 1) // 2 or output_width != weight.out_features \
            or input_width != weight.in_features:
        raise RuntimeError("NF4 packed-code count does not match weight dimensions")
    if block_size != weight.block_size or weight.primary.numel() != 1 + (logical - 1) // block_size:
        raise ValueError("NF4 scale storage has an invalid representation")
    return rows, input_width, output_width, block_size


def dispatch_quantized_linear_forward(input: torch.Tensor, weight: PackedNf4Weight, output: torch.Tensor,
                                      dimensions, stream=None) -> None:
    """output[rows, out] = input[rows, in] @ W^T (enqueued on the stream)."""
    rows, input_width, output_width, _ = _check_linear(weight, dimensions)
    _require_f32_cuda(input, "quantized linear tensor")
    _require_f32_cuda(output, "quantized linear tensor")
    if input.numel() != rows * input_width or output.numel() != rows * output_width:
        raise RuntimeError("quantized linear tensor storage size does not match dimensions")
    ws = weight.struct()
    _check(lib.b2_nf4_linear_forward(C.byref(ws), input.data_ptr(), output.data_ptr(), rows, None, 0,
                                     _stream_ptr(stream)))


def dispatch_quantized_linear_input_backward(upstream: torch.Tensor, weight: PackedNf4Weight,
                                             input_gradient: torch.Tensor, dimensions, stream=None) -> None:
    """input_gradient[rows, in] = upstream[rows, out] @ W."""
    rows, input_width, output_width, _ = _check_linear(weight, dimensions)
    _require_f32_cuda(upstream, "quantized linear tensor")
    _require_f32_cuda(input_gradient, "quantized linear tensor")
    if upstream.numel() != rows * output_width or input_gradient.numel() != rows * input_width:
        raise RuntimeError("quantized linear tensor storage size does not match dimensions")
    ws = weight.struct()
    _check(lib.b2_nf4_linear_input_backward(C.byref(ws), upstream.data_ptr(), input_gradient.data_ptr(),
                                            rows, None, 0, _stream_ptr(stream)))


@dataclass
class PagedKvPool:
    """One layer's K and V page pools, [physical_blocks, kv_heads, block_size,
    head_width] float32 on the device (PageStorage in the reference,
    src/stages/serving/cache/page_storage.cpp:11-126)."""

    key_pages: torch.Tensor
    value_pages: torch.Tensor

    @property
    def physical_blocks(self) -> int:
        return self.key_pages.shape[0]

    @property
    def kv_heads(self) -> int:
        return self.key_pages.shape[1]

    @property
    def block_size(self) -> int:
        return self.key_pages.shape[2]

    @property
    def head_width(self) -> int:
        return self.key_pages.shape[3]


def paged_decode_attention(queries: torch.Tensor, pool: PagedKvPool, block_tables: torch.Tensor,
                           seq_lens: torch.Tensor, context: torch.Tensor, max_seq_len: int,
                           status: torch.Tensor | None = None, workspace: torch.Tensor | None = None,
                           stream=None) -> None:
    """Batched grouped-query form: queries/context [n_seq, q_heads, d],
    block_tables uint32/int32 [n_seq, max_blocks], seq_lens [n_seq], all on the
    device. Enqueues only; `status` (int32/uint32 [1], zeroed by the caller)
    receives the non-finite-score bits."""
    _require_f32_cuda(queries, "paged decode attention query")
    _require_f32_cuda(context, "paged decode attention context")
    _require_f32_cuda(pool.key_pages, "paged decode attention key pages")
    _require_f32_cuda(pool.value_pages, "paged decode attention value pages")
    n_seq, q_heads, d = queries.shape
    if d != pool.head_width or tuple(context.shape) != tuple(queries.shape):
        raise RuntimeError("paged decode attention storage size does not match dimensions")
    if block_tables.dtype not in (torch.int32, torch.uint32) or seq_lens.dtype not in (torch.int32, torch.uint32):
        raise ValueError("block tables and sequence lengths must be 32-bit integers")
    ws_ptr, ws_bytes = (None, 0) if workspace is None else (workspace.data_ptr(), workspace.numel() * workspace.element_size())
    _check(lib.b2_paged_decode_attention(
        queries.data_ptr(), pool.key_pages.data_ptr(), pool.value_pages.data_ptr(),
        block_tables.data_ptr(), seq_lens.data_ptr(), context.data_ptr(), n_seq, q_heads, pool.kv_heads, d,
        pool.block_size, pool.physical_blocks, block_tables.shape[1], int(max_seq_len), ws_ptr, ws_bytes,
        status.data_ptr() if status is not None else None, _stream_ptr(stream)))


def dispatch_paged_decode_attention_forward(queries: torch.Tensor, key_pages: torch.Tensor,
                                            value_pages: torch.Tensor, block_table, context: torch.Tensor,
                                            dimensions) -> None:
    """The reference operator: one sequence, `heads` heads for both queries and
    pages; `block_table` is a HOST sequence of uint32 borrowed for the call.
    Synchronous, and raises like the reference: ValueError for bad dimensions
    or a short table, IndexError for an out-of-range block, DomainError for
    non-finite scores."""
    heads, head_width, block_size, physical_blocks, seq_len = (int(v) for v in dimensions)
    if min(heads, head_width, block_size, physical_blocks, seq_len) <= 0:
        raise ValueError("paged decode attention dimensions must be positive")
    if physical_blocks - 1 > 0xFFFFFFFF:
        raise OverflowError("paged decode attention physical block IDs exceed uint32_t")
    table = np.ascontiguousarray(block_table, dtype=np.uint32)
    required = (seq_len - 1) // block_size + 1
    if table.size != required:
        raise ValueError("paged decode attention block table size does not match the sequence")
    if required > physical_blocks:
        raise ValueError("paged decode attention has fewer physical than logical blocks")
    if (table >= physical_blocks).any():
        raise IndexError("paged decode attention block table contains an invalid block")
    for t, n, what in ((queries, heads * head_width, "query"), (context, heads * head_width, "context"),
                       (key_pages, physical_blocks * heads * block_size * head_width, "key pages"),
                       (value_pages, physical_blocks * heads * block_size * head_width, "value pages")):
        _require_f32_cuda(t, "paged decode attention " + what)
        if t.numel() != n:
            raise RuntimeError("attention storage size does not match dimensions")
    for t in (queries, key_pages, value_pages):
        if t.data_ptr() == context.data_ptr():
            raise ValueError("attention output must not alias an input")
    device = queries.device
    d_table = torch.from_numpy(table.view(np.int32)).to(device)
    d_len = torch.tensor([seq_len], dtype=torch.int32, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    pool = PagedKvPool(key_pages.view(physical_blocks, heads, block_size, head_width),
                       value_pages.view(physical_blocks, heads, block_size, head_width))
    paged_decode_attention(queries.view(1, heads, head_width), pool, d_table.view(1, -1), d_len,
                           context.view(1, heads, head_width), seq_len, status=status)
    bits = int(status.item())  # synchronises, as the reference adapter contract requires
    # bad block -> IndexError, non-finite scores -> DomainError, a page copy that timed out -> RuntimeError
    _check(lib.b2_attention_status_result(bits))


# ---- host-buffer seam ------------------------------------------------------------

def _host_ptr(a: np.ndarray | torch.Tensor) -> int:
    if isinstance(a, torch.Tensor):
        if a.is_cuda or not a.is_contiguous():
            raise ValueError("host buffer expected")
        return a.data_ptr()
    if not a.flags["C_CONTIGUOUS"]:
        raise ValueError("host buffers must be contiguous")
    return a.ctypes.data


def host_quantized_linear_forward(x_host, weight: PackedNf4Weight, y_host, rows: int, stream=None) -> None:
    """HOST x [rows, in] -> HOST y [rows, out]; copies and kernel inside the call."""
    ws = weight.struct()
    _check(lib.b2_host_nf4_linear_forward(C.byref(ws), _host_ptr(x_host), _host_ptr(y_host), rows,
                                          _stream_ptr(stream)))


def host_quantized_linear_input_backward(dy_host, weight: PackedNf4Weight, dx_host, rows: int, stream=None) -> None:
    ws = weight.struct()
    _check(lib.b2_host_nf4_linear_input_backward(C.byref(ws), _host_ptr(dy_host), _host_ptr(dx_host), rows,
                                                 _stream_ptr(stream)))


def host_paged_decode_attention_forward(q_host, pool: PagedKvPool, block_tables_host, seq_lens_host, ctx_host,
                                        stream=None) -> None:
    """HOST queries/tables/lengths -> HOST context, pages stay on the device."""
    n_seq, q_heads, d = q_host.shape
    tables = np.ascontiguousarray(block_tables_host, np.uint32) if not isinstance(block_tables_host, torch.Tensor) else block_tables_host
    lens = np.ascontiguousarray(seq_lens_host, np.uint32) if not isinstance(seq_lens_host, torch.Tensor) else seq_lens_host
    _check(lib.b2_host_paged_decode_attention(
        _host_ptr(q_host), pool.key_pages.data_ptr(), pool.value_pages.data_ptr(), _host_ptr(tables),
        _host_ptr(lens), _host_ptr(ctx_host), n_seq, q_heads, pool.kv_heads, d, pool.block_size,
        pool.physical_blocks, tables.shape[1], _stream_ptr(stream)))
