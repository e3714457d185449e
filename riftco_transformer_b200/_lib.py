"""ctypes bindings of ``libriftco_b200.so`` (declared in ``include/riftco_b200.h``).

Importing this module only loads the library; it does not touch a GPU. There
is deliberately no fallback: if the shared library is missing the import fails,
and every compute call fails with the library's own status when no sm_100
device is usable.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libriftco_b200.so"

STATUS_OK = 0
STATUS_INVALID_ARGUMENT = 1
STATUS_OUT_OF_RANGE = 2
STATUS_OVERFLOW = 3
STATUS_BACKEND_UNAVAILABLE = 4
STATUS_OUT_OF_MEMORY = 5
STATUS_RUNTIME_ERROR = 6
STATUS_DOMAIN_ERROR = 7

SCALES_FLOAT32 = 0
SCALES_DOUBLE_QUANTIZED_UINT8 = 1

ATTN_STATUS_NAN_OR_POS_INF = 1
ATTN_STATUS_ALL_NEG_INF = 2
ATTN_STATUS_BAD_BLOCK = 4
ATTN_STATUS_TIMEOUT = 8
NOALLOC_SCRATCH_BYTES = 8 * 1024 * 1024


class Nf4WeightStruct(C.Structure):
    """b2_nf4_weight."""

    _fields_ = [
        ("codes", C.c_void_p),
        ("scales_primary", C.c_void_p),
        ("scales_secondary", C.c_void_p),
        ("encoding", C.c_uint32),
        ("block_size", C.c_uint32),
        ("scale_block_size", C.c_uint64),
        ("scale_offset", C.c_float),
        ("reserved", C.c_uint32),
        ("out_features", C.c_uint64),
        ("in_features", C.c_uint64),
        ("flat_block_base", C.c_uint64),
    ]


# name -> (restype, argtypes); every symbol the public header declares.
_W = C.POINTER(Nf4WeightStruct)
_vp, _u32, _u64, _sz, _i32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_size_t, C.c_int32
SIGNATURES = {
    "b2_abi_version": (_i32, []),
    "b2_last_error": (C.c_char_p, []),
    "b2_is_available": (_i32, []),
    "b2_unavailability_reason": (C.c_char_p, []),
    "b2_nf4_dequantize": (_i32, [_W, _vp, _vp]),
    "b2_nf4_quantize_workspace_bytes": (_sz, [_u64, _u64, _u32, _u64]),
    "b2_nf4_quantize": (_i32, [_vp, _u64, _u64, _u32, _u64, _vp, _vp, _vp, C.POINTER(C.c_float), _vp, _sz, _vp]),
    "b2_nf4_validate_payload": (_i32, [_W, _u64, _u64, _u64, _vp]),
    "b2_nf4_linear_forward": (_i32, [_W, _vp, _vp, _u64, _vp, _sz, _vp]),
    "b2_nf4_linear_lora_workspace_bytes": (_sz, [_W, _u64, _u32]),
    "b2_nf4_linear_forward_lora": (_i32, [_W, _vp, _vp, _vp, _u32, C.c_float, _vp, _u64, _vp, _sz, _vp]),
    "b2_nf4_linear_forward_multi": (_i32, [_vp, _u32, _vp, _vp, _u64, _vp, _sz, _vp]),
    "b2_nf4_linear_bf16_supported": (_i32, [_vp, _u32, _u64]),
    "b2_nf4_linear_forward_multi_bf16": (_i32, [_vp, _u32, _vp, _vp, _u64, _vp]),
    "b2_nf4_linear_input_backward": (_i32, [_W, _vp, _vp, _u64, _vp, _sz, _vp]),
    "b2_nf4_linear_workspace_bytes": (_sz, [_W, _u64, _i32]),
    "b2_paged_decode_attention": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32,
                                         _u64, _u32, _u32, _vp, _sz, _vp, _vp]),
    "b2_paged_decode_attention_bf16": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32,
                                              _u64, _u32, _u32, _vp, _sz, _vp, _vp]),
    "b2_paged_decode_workspace_bytes": (_sz, [_u32, _u32, _u32, _u32, _u32]),
    "b2_attention_status_result": (_i32, [_u32]),
    "b2_last_route": (_i32, []),
    "b2_paged_decode_attention_noalloc": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32,
                                                 _u64, _u32, _u32, _vp, _vp]),
    "b2_rmsnorm": (_i32, [_vp, _vp, _vp, _vp, _vp, _u64, _u64, C.c_float, _vp]),
    "b2_rmsnorm_bf16": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _u64, _u64, C.c_float, _vp]),
    "b2_silu_mul_bf16": (_i32, [_vp, _vp, _vp, _vp, _u64, _vp]),
    "b2_rope_append_kv": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _u64, _u32,
                                 C.c_float, _vp, _vp]),
    "b2_rope_append_kv_tokens": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _u64,
                                        _u32, C.c_float, _vp, _vp]),
    "b2_silu_mul": (_i32, [_vp, _vp, _vp, _u64, _vp]),
    "b2_add": (_i32, [_vp, _vp, _vp, _u64, _vp]),
    "b2_gather_rows": (_i32, [_vp, _vp, _vp, _u32, _u32, _u32, _vp, _vp]),
    "b2_rtnf4_index": (_i32, [_vp, _u64, _vp, _u64, _vp]),
    "b2_peer_all_gather_columns": (_i32, [_vp, _u64, _u64, _vp, _vp, _u32, _u32, _vp, _vp, _vp]),
    "b2_peer_all_gather_columns_bf16": (_i32, [_vp, _u64, _u64, _vp, _vp, _vp, _u32, _u32, _vp, _vp, _vp]),
    "b2_argmax": (_i32, [_vp, _vp, _u32, _u32, _vp]),
    "b2_check_device_errors": (_i32, []),
    "b2_host_nf4_linear_forward": (_i32, [_W, _vp, _vp, _u64, _vp]),
    "b2_host_nf4_linear_input_backward": (_i32, [_W, _vp, _vp, _u64, _vp]),
    "b2_host_paged_decode_attention": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32,
                                              _u32, _u64, _u32, _vp]),
}


def load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m riftco_transformer_b200.build` "
            "(there is no CPU fallback)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = load()
