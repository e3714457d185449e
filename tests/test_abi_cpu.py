"""The C-ABI shared library on a machine without a GPU: it loads, exports every
symbol the public header declares, and refuses to compute (no CPU fallback)."""
import ctypes as C
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "riftco_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b2_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from riftco_transformer_b200 import _lib
    names = declared_symbols()
    assert len(names) >= 12
    raw = C.CDLL(str(_lib.LIB_PATH))
    for name in names:
        assert hasattr(raw, name), f"{name} is declared in riftco_b200.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert _lib.lib.b2_abi_version() == 1


def test_weight_struct_layout_matches_header():
    from riftco_transformer_b200._lib import Nf4WeightStruct
    assert C.sizeof(Nf4WeightStruct) == 72
    assert Nf4WeightStruct.flat_block_base.offset == 64
    assert Nf4WeightStruct.scale_offset.offset == 40


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_no_cpu_fallback_without_a_device():
    from riftco_transformer_b200 import _lib
    lib = _lib.lib
    assert lib.b2_is_available() == 0
    assert b"unavailable" in lib.b2_unavailability_reason()
    w = _lib.Nf4WeightStruct()
    status = lib.b2_nf4_dequantize(C.byref(w), None, None)
    assert status == _lib.STATUS_BACKEND_UNAVAILABLE
    assert b"unavailable" in lib.b2_last_error()
    status = lib.b2_nf4_linear_forward(C.byref(w), None, None, 1, None, 0, None)
    assert status == _lib.STATUS_BACKEND_UNAVAILABLE
    status = lib.b2_paged_decode_attention(None, None, None, None, None, None, 1, 1, 1, 1, 1, 1, 1, 1,
                                           None, 0, None, None)
    assert status == _lib.STATUS_BACKEND_UNAVAILABLE


def test_attention_status_word_mapping():
    """b2_attention_status_result: what a synchronous caller reports for the device status word
    (no GPU involved). A page copy whose bounded wait gave up must not pass as success."""
    from riftco_transformer_b200 import _lib
    from riftco_transformer_b200.backend import DomainError, _check
    lib = _lib.lib
    assert lib.b2_attention_status_result(0) == _lib.STATUS_OK
    assert lib.b2_attention_status_result(_lib.ATTN_STATUS_BAD_BLOCK) == _lib.STATUS_OUT_OF_RANGE
    assert b"invalid block" in lib.b2_last_error()
    assert lib.b2_attention_status_result(_lib.ATTN_STATUS_NAN_OR_POS_INF) == _lib.STATUS_DOMAIN_ERROR
    assert lib.b2_attention_status_result(_lib.ATTN_STATUS_ALL_NEG_INF) == _lib.STATUS_DOMAIN_ERROR
    assert lib.b2_attention_status_result(_lib.ATTN_STATUS_TIMEOUT) == _lib.STATUS_RUNTIME_ERROR
    assert b"did not complete" in lib.b2_last_error()
    assert lib.b2_attention_status_result(0x40) == _lib.STATUS_RUNTIME_ERROR          # an unknown bit
    # a bad block outranks the rest, as the host validation of the reference runs first
    assert lib.b2_attention_status_result(_lib.ATTN_STATUS_BAD_BLOCK | _lib.ATTN_STATUS_TIMEOUT) == _lib.STATUS_OUT_OF_RANGE
    with pytest.raises(RuntimeError):
        _check(lib.b2_attention_status_result(_lib.ATTN_STATUS_TIMEOUT))
    with pytest.raises(DomainError):
        _check(lib.b2_attention_status_result(_lib.ATTN_STATUS_ALL_NEG_INF))


def test_route_names_follow_the_header():
    """backend.ROUTES is indexed by the header's B2_ROUTE_* values; a thread that made no call
    reports none."""
    import re
    from pathlib import Path

    from riftco_transformer_b200 import backend
    header = (Path(__file__).resolve().parents[1] / "include" / "riftco_b200.h").read_text()
    routes = dict((name.lower(), int(value)) for name, value in re.findall(r"#define B2_ROUTE_(\w+) (\d+)", header))
    assert sorted(routes.values()) == list(range(len(backend.ROUTES)))
    for name, value in routes.items():
        assert backend.ROUTES[value] == name
    assert backend.last_route() == "none"
