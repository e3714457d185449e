"""The reference's own dispatch layer on ExecutionBackend::Cuda, with its CUDA
seam (cuda_backend_adapter) defined by the product's adapter translation unit:
dispatch_quantized_linear_forward / _input_backward and
dispatch_paged_decode_attention_forward validate the request exactly as the
reference does and then land in the B200 kernels through the C ABI. Results are
compared with the CPU oracle; error behaviour with the reference on its CPU
backend. The adapter library is prebuilt (oracle/_ref, from a checkout of the
reference); without it these tests skip."""
import numpy as np
import pytest

from conftest import rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cuda_ref():
    import oracle
    import riftco_transformer_b200 as pkg
    assert pkg.is_available(), pkg.unavailability_reason()
    try:
        return oracle.ref_with_b200_adapter()
    except FileNotFoundError as e:
        pytest.skip(str(e))


@pytest.mark.parametrize("rows,out_f,in_f,block,dq,tol", [
    (1, 4096, 4096, 64, True, 2e-3),       # decode GEMV
    (8, 1000, 192, 64, False, 2e-3),       # ragged rows, FP32 scales
    (64, 1024, 512, 64, True, 1e-2),       # tensor-memory kernel, small token tile
    (300, 512, 256, 128, True, 1e-2),      # 256 x 256 tensor-core kernel
    (5, 77, 333, 32, True, 2e-3),          # shape only the generic kernel takes
])
def test_linear_forward_through_reference_dispatch(cuda_ref, port, rows, out_f, in_f, block, dq, tol):
    rng = np.random.default_rng(rows * 31 + out_f)
    W = (rng.standard_normal((out_f, in_f)) * 0.02).astype(np.float32)
    host = port.quantize_nf4_double_quantized(W, block, 32) if dq else port.quantize_nf4(W, block)
    x = rng.standard_normal((rows, in_f)).astype(np.float32)
    y = cuda_ref.linear_forward(host, x)
    assert rel_l2(y, port.linear_forward(host, x)) <= tol


@pytest.mark.parametrize("rows,out_f,in_f,tol", [(4, 256, 512, 1e-2), (300, 256, 512, 1e-2)])
def test_linear_input_backward_through_reference_dispatch(cuda_ref, port, rows, out_f, in_f, tol):
    rng = np.random.default_rng(rows + 5)
    W = (rng.standard_normal((out_f, in_f)) * 0.02).astype(np.float32)
    host = port.quantize_nf4_double_quantized(W, 64, 256)
    dy = rng.standard_normal((rows, out_f)).astype(np.float32)
    dx = cuda_ref.linear_input_backward(host, dy)
    assert rel_l2(dx, port.linear_input_backward(host, dy)) <= tol


@pytest.mark.parametrize("heads,width,block,seq_len", [(2, 3, 2, 5), (8, 128, 16, 777)])
def test_paged_decode_through_reference_dispatch(cuda_ref, port, heads, width, block, seq_len):
    rng = np.random.default_rng(seq_len)
    blocks = (seq_len + block - 1) // block
    physical = blocks + 3
    k = rng.standard_normal((physical, heads, block, width)).astype(np.float32)
    v = rng.standard_normal((physical, heads, block, width)).astype(np.float32)
    q = rng.standard_normal((heads, width)).astype(np.float32)
    table = rng.permutation(physical)[:blocks].astype(np.uint32)
    got = cuda_ref.paged_decode(q, k, v, table, seq_len)
    want = port.paged_decode(q, k, v, table, seq_len)
    assert rel_l2(got, want) <= 2e-3


def test_errors_keep_the_reference_types(cuda_ref, port):
    import oracle
    rng = np.random.default_rng(1)
    k = rng.standard_normal((3, 1, 2, 3)).astype(np.float32)
    v = rng.standard_normal((3, 1, 2, 3)).astype(np.float32)
    q = np.full((1, 3), np.nan, np.float32)
    table = np.array([0, 1, 2], np.uint32)
    with pytest.raises(oracle.ReferenceError_) as e:
        cuda_ref.paged_decode(q, k, v, table, 5)     # non-finite scores: std::domain_error
    assert e.value.status == 7
    with pytest.raises(oracle.ReferenceError_) as e:
        cuda_ref.paged_decode(q, k, v, np.array([0, 1, 9], np.uint32), 5)   # block id outside the pool
    assert e.value.status in (1, 2)


def test_reference_conformance_executable():
    """The reference's own accelerator test for the packed-NF4 linear
    (tests/core/backend/test_quantized_linear_backend.cpp, built with
    RIFTCO_TRANSFORMER_TEST_REQUIRE_CUDA=1 against the reference core + this repo's adapter):
    aligned and edge fixtures in both scale encodings, forward and input backward, at the
    reference's accelerator tolerance, plus its storage-size rules."""
    import os
    import subprocess
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    exe = root / "oracle" / "_ref" / "quantized_linear_backend_tests"
    if not exe.exists():
        pytest.skip("the conformance executable is prebuilt from a checkout of the reference (oracle/build.py)")
    proc = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
    log_dir = os.environ.get("B2_TEST_LOG_DIR")   # optional: keep the executable's output as a file
    if log_dir:
        Path(log_dir).mkdir(parents=True, exist_ok=True)
        (Path(log_dir) / "reference_quantized_linear_backend_tests.log").write_text(
            f"$ oracle/_ref/quantized_linear_backend_tests\n{proc.stdout}{proc.stderr}exit code {proc.returncode}\n")
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "quantized-linear backend tests passed" in proc.stdout
