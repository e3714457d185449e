"""B200 (sm_100a) backend for Riftco's packed-NF4 linear and paged-KV decode
attention. The product is the CUDA library behind ``include/riftco_b200.h``;
this package is its host-side face for Python callers, shaped after the
reference's backend operator interface.

Attributes are resolved on first use so that ``python -m
riftco_transformer_b200.build`` can run before the shared library exists.
"""
_EXPORTS = (
    "DomainError",
    "BackendUnavailable",
    "PackedNf4Weight",
    "PagedKvPool",
    "check_device_errors",
    "dequantize",
    "dispatch_paged_decode_attention_forward",
    "dispatch_quantized_linear_forward",
    "dispatch_quantized_linear_input_backward",
    "host_paged_decode_attention_forward",
    "host_quantized_linear_forward",
    "host_quantized_linear_input_backward",
    "is_available",
    "last_route",
    "paged_decode_attention",
    "quantize_nf4",
    "unavailability_reason",
    "validate_payload",
)
__all__ = list(_EXPORTS)


def __getattr__(name):
    if name in _EXPORTS:
        from . import backend
        return getattr(backend, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
