import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests" / "golden"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def golden():
    with np.load(ROOT / "tests" / "golden" / "reference_vectors.npz") as data:
        return {k: data[k] for k in data.files}


@pytest.fixture(scope="session")
def port():
    import oracle
    return oracle.port()


def weight_from_golden(golden, prefix):
    """Rebuilds the canonical host payload stored by make_golden.payload_arrays."""
    import oracle
    out_f, in_f, block, scale_block = (int(v) for v in golden[f"{prefix}_shape"])
    if f"{prefix}_fp32_scales" in golden:
        return oracle.Nf4Weight(golden[f"{prefix}_codes"], out_f, in_f, block,
                                fp32_scales=golden[f"{prefix}_fp32_scales"])
    return oracle.Nf4Weight(golden[f"{prefix}_codes"], out_f, in_f, block,
                            scale_codes=golden[f"{prefix}_scale_codes"],
                            second_level=golden[f"{prefix}_second_level"],
                            scale_block_size=scale_block, offset=float(golden[f"{prefix}_offset"][0]))


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def rel_l2(actual, expected):
    a = np.asarray(actual, np.float64)
    e = np.asarray(expected, np.float64)
    return float(np.linalg.norm(a - e) / max(np.linalg.norm(e), 1e-30))
