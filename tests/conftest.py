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


class Guarded:
    """A float32 CUDA output tensor between two guard bands filled with a bit pattern no kernel
    writes: `check()` fails if a kernel stored a single element outside the tensor it was given."""

    GUARD = 4096          # elements on each side (16 KB)
    PATTERN = 0x7FC0BEEF  # a NaN with a recognisable payload

    def __init__(self, shape, device="cuda"):
        import torch
        n = int(np.prod(shape))
        self.raw = torch.full((n + 2 * self.GUARD,), 0, dtype=torch.int32, device=device)
        self.raw.fill_(self.PATTERN - (1 << 32) if self.PATTERN >= (1 << 31) else self.PATTERN)
        self.tensor = self.raw[self.GUARD:self.GUARD + n].view(torch.float32).view(*shape)

    def check(self):
        import torch
        torch.cuda.synchronize()
        want = self.PATTERN - (1 << 32) if self.PATTERN >= (1 << 31) else self.PATTERN
        lo, hi = self.raw[:self.GUARD], self.raw[-self.GUARD:]
        assert bool((lo == want).all()), "a kernel wrote below its output tensor"
        assert bool((hi == want).all()), "a kernel wrote past its output tensor"
