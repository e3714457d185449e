"""The persistent decode-batch linear kernel (tcgen05, stream-K over weight tiles and 256-wide
rounds) through the C ABI against the FP32 CPU oracle: 17..32 rows in process (bf16 operands,
relative L2 <= 1e-2), 1..16 rows in a worker that forces the kernel for every batch size (fp16
operands, <= 2e-3)."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from decode_linear_cases import CASES, rel_l2, run_case

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def b2():
    import riftco_transformer_b200 as pkg
    assert pkg.is_available(), pkg.unavailability_reason()
    return pkg


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"m{c[0]}_{'+'.join(map(str, c[1]))}x{c[2]}_b{c[3]}_{'dq' if c[4] else 'f32'}")
def test_decode_batches_against_oracle(b2, port, case):
    run_case(b2, port, case, 1e-2)


def test_row_shards_use_the_parent_scale_groups(b2, port):
    """Row shards are views of the parent's bytes with flat_block_base != 0: the kernel must index
    the second-level scales by the PARENT's block numbers (groups of 256 blocks straddle rows when
    a row holds 224 blocks)."""
    rng = np.random.default_rng(77)
    W = (rng.standard_normal((2048, 14336)) * 0.02).astype(np.float32)
    host = port.quantize_nf4_double_quantized(W, 64, 256)
    parent = b2.PackedNf4Weight.from_host(host)
    x = rng.standard_normal((32, 14336)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    want = port.linear_forward(host, x)
    world = 4
    for rank in range(world):
        shard = parent.row_shard(rank, world)
        assert shard.flat_block_base == rank * 512 * 224
        y = torch.empty((32, shard.out_features), device="cuda")
        b2.dispatch_quantized_linear_forward(xd, shard, y, (32, 14336, shard.out_features, 64))
        b2.check_device_errors()
        got = y.cpu().numpy()
        assert rel_l2(got, want[:, rank * 512:(rank + 1) * 512]) <= 1e-2


def test_caller_workspace_and_size_query(b2, port):
    import ctypes as C

    from riftco_transformer_b200._lib import lib
    from riftco_transformer_b200.backend import _check
    rng = np.random.default_rng(5)
    W = (rng.standard_normal((1024, 1024)) * 0.02).astype(np.float32)
    host = port.quantize_nf4_double_quantized(W, 64, 256)
    w = b2.PackedNf4Weight.from_host(host)
    x = rng.standard_normal((32, 1024)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    ws = w.struct()
    need = lib.b2_nf4_linear_workspace_bytes(C.byref(ws), 32, 0)
    assert need > 32 * 1024 * 2
    scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
    y = torch.empty((32, 1024), device="cuda")
    _check(lib.b2_nf4_linear_forward(C.byref(ws), xd.data_ptr(), y.data_ptr(), 32, scratch.data_ptr(), need, None))
    b2.check_device_errors()
    assert rel_l2(y.cpu().numpy(), port.linear_forward(host, x)) <= 1e-2
    with pytest.raises(ValueError):
        _check(lib.b2_nf4_linear_forward(C.byref(ws), xd.data_ptr(), y.data_ptr(), 32, scratch.data_ptr(), need - 1024, None))


def test_small_batches_on_the_fp16_form():
    env = dict(os.environ, B2_DECODE_IMPL="tmem")
    proc = subprocess.run([sys.executable, str(ROOT / "tests" / "decode_linear_worker.py")], env=env,
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "decode linear worker ok" in proc.stdout
