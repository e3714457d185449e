"""The tensor-core (tcgen05) paths of the packed-NF4 linear - every forward with
more than 16 batch rows and the input-backward with more than 32 - against the
FP32 CPU oracle. Tolerance: relative L2 <= 1e-2 (bf16 operands, FP32 accumulate)."""
import numpy as np
import pytest
import torch

from conftest import rel_l2

pytestmark = pytest.mark.gpu

GEMM_TOL = 1e-2


@pytest.fixture(scope="module")
def b2():
    import riftco_transformer_b200 as pkg
    assert pkg.is_available(), pkg.unavailability_reason()
    return pkg


def forward(b2, w, x):
    rows = x.shape[0]
    y = torch.empty((rows, w.out_features), dtype=torch.float32, device="cuda")
    b2.dispatch_quantized_linear_forward(x, w, y, (rows, w.in_features, w.out_features, w.block_size))
    b2.check_device_errors()
    return y.cpu().numpy()


@pytest.mark.parametrize("rows,out_f,in_f,block,dq", [
    (256, 256, 64, 64, False),      # one tile, one k-block
    (300, 512, 256, 64, True),      # ragged M, several k-blocks (ring wraps)
    (257, 300, 1024, 128, True),    # ragged M and N, block 128
    (64, 1000, 4096, 64, False),    # fewer rows than a tile, FP32 scales, long K
    (300, 256, 2048, 64, True),     # full 256-token tiles with the contraction split over a cluster of 4:
                                    # the partial tile fills the whole activation ring
])
def test_gemm_small_shapes(b2, port, rows, out_f, in_f, block, dq):
    rng = np.random.default_rng(rows + out_f)
    W = (rng.standard_normal((out_f, in_f)) * 0.02).astype(np.float32)
    host = port.quantize_nf4_double_quantized(W, block, 32) if dq else port.quantize_nf4(W, block)
    x = rng.standard_normal((rows, in_f)).astype(np.float32)
    y = forward(b2, b2.PackedNf4Weight.from_host(host), torch.from_numpy(x).cuda())
    want = port.linear_forward(host, x)
    assert np.isfinite(y).all()
    assert rel_l2(y, want) <= GEMM_TOL
    for r in (0, rows // 2, rows - 1):
        assert rel_l2(y[r], want[r]) <= GEMM_TOL


@pytest.mark.parametrize("rows,out_f,in_f,block,dq", [
    (17, 4096, 4096, 64, True),      # 32-token tile, contraction split over a cluster of 4
    (32, 14336, 4096, 64, True),     # 112 weight-row tiles, one accumulator per expansion group
    (32, 4096, 14336, 64, True),     # long contraction, split
    (33, 1000, 256, 64, True),       # ragged weight-row tile, 48-token tile (a half-used column chunk)
    (64, 4096, 4096, 128, False),    # FP32 scales, block 128, the largest multi-issuer tile
    (128, 1024, 512, 64, True),      # single issuer, 128-token tile, 8 k-blocks over a cluster of 1
    (100, 32000, 1024, 64, True),    # two waves of tiles, ragged token tile
    (18, 256, 64, 64, True),         # one k-block: three of the four groups have no work
    (24, 128, 192, 64, True),        # three k-blocks
    (100, 512, 4096, 64, True),      # single issuer AND a cluster of 8 over the contraction
])
def test_small_token_tiles(b2, port, rows, out_f, in_f, block, dq):
    """17..128 batch rows on the tensor-memory kernel: up to 64 tokens every expansion group issues
    its own MMAs into its own accumulator; few weight-row tiles split the contraction over a cluster."""
    rng = np.random.default_rng(rows * 11 + out_f)
    W = (rng.standard_normal((out_f, in_f)) * 0.02).astype(np.float32)
    host = port.quantize_nf4_double_quantized(W, block, 256) if dq else port.quantize_nf4(W, block)
    x = rng.standard_normal((rows, in_f)).astype(np.float32)
    w = b2.PackedNf4Weight.from_host(host)
    y = forward(b2, w, torch.from_numpy(x).cuda())
    want = port.linear_forward(host, x)
    assert np.isfinite(y).all()
    assert rel_l2(y, want) <= GEMM_TOL
    for r in range(rows):
        assert rel_l2(y[r], want[r]) <= GEMM_TOL
    # same bits on a second run
    y2 = forward(b2, w, torch.from_numpy(x).cuda())
    assert (y.view(np.uint32) == y2.view(np.uint32)).all()


def test_gemm_config3_sampled_rows(b2, port):
    # baseline configuration 3, forward: M = 4096 tokens through 4096 -> 14336, checked on 24 rows
    rng = np.random.default_rng(1234)
    W = (rng.standard_normal((14336, 4096)) * 0.02).astype(np.float32)
    host = port.quantize_nf4_double_quantized(W, 64, 256)
    x = rng.standard_normal((4096, 4096)).astype(np.float32)
    y = forward(b2, b2.PackedNf4Weight.from_host(host), torch.from_numpy(x).cuda())
    idx = np.r_[0:8, 2000:2008, 4088:4096]
    want = port.linear_forward(host, x[idx])
    assert rel_l2(y[idx], want) <= GEMM_TOL
    assert np.isfinite(y).all()
    # linearity in the activations
    y2 = forward(b2, b2.PackedNf4Weight.from_host(host), torch.from_numpy(2.0 * x[:64]).cuda())
    # (64 tokens run as four partial accumulators, 4096 as one: the FP32 summation order differs)
    assert rel_l2(y2, 2.0 * y[:64]) <= 2e-5


def backward(b2, w, dy):
    rows = dy.shape[0]
    dx = torch.empty((rows, w.in_features), dtype=torch.float32, device="cuda")
    b2.dispatch_quantized_linear_input_backward(dy, w, dx, (rows, w.in_features, w.out_features, w.block_size))
    b2.check_device_errors()
    return dx.cpu().numpy()


@pytest.mark.parametrize("rows,out_f,in_f,block,dq", [
    (256, 64, 256, 64, False),      # one tile, one k-block
    (300, 256, 512, 64, True),      # ragged M, ring wraps
    (100, 1024, 320, 64, True),     # ragged N (320 = 256 + 64), in-blocks past the edge
    (257, 512, 1024, 256, False),   # block 256: four 64-wide column groups share a scale
    (600, 192, 320, 64, True),      # 512+ rows: transposed expansion + plain bf16 GEMM; ragged M and N tiles
    (1000, 128, 64, 64, False),     # same path, one column tile, FP32 scales
    (513, 320, 512, 128, True),     # same path, block 128, five k-blocks (ring wraps)
])
def test_input_backward_tensor_core(b2, port, rows, out_f, in_f, block, dq):
    rng = np.random.default_rng(rows * 3 + in_f)
    W = (rng.standard_normal((out_f, in_f)) * 0.02).astype(np.float32)
    host = port.quantize_nf4_double_quantized(W, block, 32) if dq else port.quantize_nf4(W, block)
    dy = (rng.standard_normal((rows, out_f)) * 0.01).astype(np.float32)
    dx = backward(b2, b2.PackedNf4Weight.from_host(host), torch.from_numpy(dy).cuda())
    want = port.linear_input_backward(host, dy)
    assert np.isfinite(dx).all()
    assert rel_l2(dx, want) <= GEMM_TOL
    for r in (0, rows - 1):
        assert rel_l2(dx[r], want[r]) <= GEMM_TOL


def test_input_backward_config3_sampled_rows(b2, port):
    # baseline configuration 3, backward: dY [4096, 14336] ~ N(0, 1e-4) -> dX [4096, 4096]
    rng = np.random.default_rng(4321)
    W = (rng.standard_normal((14336, 4096)) * 0.02).astype(np.float32)
    host = port.quantize_nf4_double_quantized(W, 64, 256)
    dy = (rng.standard_normal((4096, 14336)) * 0.01).astype(np.float32)
    dx = backward(b2, b2.PackedNf4Weight.from_host(host), torch.from_numpy(dy).cuda())
    idx = np.r_[0:4, 2047:2051, 4092:4096]
    want = port.linear_input_backward(host, dy[idx])
    assert rel_l2(dx[idx], want) <= GEMM_TOL
    assert np.isfinite(dx).all()


@pytest.mark.parametrize("rows", [4, 32, 200])
def test_multi_weight_forward_matches_single_calls(b2, port, rows):
    """b2_nf4_linear_forward_multi: q / k / v style projections of one input. Up to 16 rows it is a
    loop of single calls; above, one conversion and one launch. The products are those of the single
    calls; only the order of the FP32 partial sums may differ (which CTA sums which slice of the
    contraction depends on the tiles of the whole launch)."""
    import ctypes as C

    from riftco_transformer_b200 import _lib
    from riftco_transformer_b200._lib import lib
    from riftco_transformer_b200.backend import _check
    rng = np.random.default_rng(rows)
    in_f = 512
    hosts = [port.quantize_nf4_double_quantized((rng.standard_normal((o, in_f)) * 0.02).astype(np.float32), 64, 256)
             for o in (640, 128, 136)]
    hosts.append(port.quantize_nf4((rng.standard_normal((256, in_f)) * 0.02).astype(np.float32), 128))
    weights = [b2.PackedNf4Weight.from_host(h) for h in hosts]
    x = torch.from_numpy(rng.standard_normal((rows, in_f)).astype(np.float32)).cuda()
    singles = [forward(b2, w, x) for w in weights]
    outs = [torch.empty((rows, w.out_features), device="cuda") for w in weights]
    structs = (_lib.Nf4WeightStruct * len(weights))(*[w.struct() for w in weights])
    ptrs = (C.c_void_p * len(weights))(*[o.data_ptr() for o in outs])
    _check(lib.b2_nf4_linear_forward_multi(structs, len(weights), x.data_ptr(), ptrs, rows, None, 0, None))
    if rows > 16:   # mixed scale encodings: not one launch of the decode kernel, but one of the prefill kernel
        assert b2.last_route() == "gemm_tmem"
    b2.check_device_errors()
    for host, single, out in zip(hosts, singles, outs):
        got = out.cpu().numpy()
        assert rel_l2(got, port.linear_forward(host, x.cpu().numpy())) <= GEMM_TOL
        assert rel_l2(got, single) <= 1e-5
    # an output used twice is a caller error, reported by the single-call path
    ptrs[1] = ptrs[0]
    with pytest.raises(ValueError):
        _check(lib.b2_nf4_linear_forward_multi(structs, len(weights), x.data_ptr(), ptrs, rows, None, 0, None))


def _device_quantized(b2, out_f, in_f, dq, seed):
    """W ~ N(0, 0.02^2) quantised on the device by the torch restatement of the reference encoder
    (held to the oracle bit for bit in test_gpu_parity.py), plus its host payload for the oracle."""
    import oracle
    from riftco_transformer_b200 import synth
    w = synth.quantized_weight(out_f, in_f, seed=seed, double_quantized=dq)
    if dq:
        host = oracle.Nf4Weight(w.codes.cpu().numpy(), out_f, in_f, w.block_size,
                                scale_codes=w.primary.cpu().numpy(), second_level=w.secondary.cpu().numpy(),
                                scale_block_size=w.scale_block_size, offset=w.offset)
    else:
        host = oracle.Nf4Weight(w.codes.cpu().numpy(), out_f, in_f, w.block_size, fp32_scales=w.primary.cpu().numpy())
    return w, host


@pytest.mark.parametrize("out_f,in_f,dq", [
    (14336, 4096, False),   # 4096 -> 14336, FP32 scales
    (4096, 14336, True),    # 14336 -> 4096, double-quantised
    (4096, 14336, False),   # 14336 -> 4096, FP32 scales
])
def test_gemm_config3_remaining_forward_cases(b2, port, out_f, in_f, dq):
    """Baseline configuration 3, forward, the cases test_gemm_config3_sampled_rows does not run:
    M = 4096 tokens, checked on 24 sampled rows against the FP32 oracle."""
    w, host = _device_quantized(b2, out_f, in_f, dq, seed=out_f + 7 * dq)
    g = torch.Generator(device="cuda")
    g.manual_seed(99)
    x = torch.randn((4096, in_f), device="cuda", generator=g)
    y = forward(b2, w, x)
    idx = np.r_[0:8, 2000:2008, 4088:4096]
    want = port.linear_forward(host, x[idx].cpu().numpy())
    assert np.isfinite(y).all()
    assert rel_l2(y[idx], want) <= GEMM_TOL
    for j, r in enumerate(idx):
        assert rel_l2(y[r], want[j]) <= 2 * GEMM_TOL


@pytest.mark.parametrize("out_f,in_f,dq", [
    (14336, 4096, False),   # dY [4096, 14336] -> dX [4096, 4096], FP32 scales
    (4096, 14336, True),    # dY [4096, 4096] -> dX [4096, 14336], double-quantised
    (4096, 14336, False),   # the same with FP32 scales
])
def test_input_backward_config3_remaining_cases(b2, port, out_f, in_f, dq):
    """Baseline configuration 3, input-backward, the cases the sampled-row test above does not run:
    dY ~ N(0, 1e-4), checked on 12 sampled rows."""
    w, host = _device_quantized(b2, out_f, in_f, dq, seed=3 * out_f + dq)
    g = torch.Generator(device="cuda")
    g.manual_seed(98)
    dy = torch.randn((4096, out_f), device="cuda", generator=g) * 0.01
    dx = backward(b2, w, dy)
    idx = np.r_[0:4, 2047:2051, 4092:4096]
    want = port.linear_input_backward(host, dy[idx].cpu().numpy())
    assert np.isfinite(dx).all()
    assert rel_l2(dx[idx], want) <= GEMM_TOL


# ---- low-rank adapter branch --------------------------------------------------------------------

def _lora_forward(b2, w, x, a, b, scale):
    import ctypes as C

    from riftco_transformer_b200._lib import lib
    from riftco_transformer_b200.backend import _check
    rows = x.shape[0]
    y = torch.full((rows, w.out_features), float("nan"), device="cuda")
    ws = w.struct()
    need = lib.b2_nf4_linear_lora_workspace_bytes(C.byref(ws), rows, a.shape[0])
    scratch = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    _check(lib.b2_nf4_linear_forward_lora(C.byref(ws), x.data_ptr(), a.data_ptr(), b.data_ptr(), a.shape[0], scale,
                                          y.data_ptr(), rows, scratch.data_ptr(), scratch.numel(), None))
    b2.check_device_errors()
    return y.cpu().numpy()


def test_lora_reference_vector(b2, golden):
    """The adapted linear of the golden file (written by the reference: base + ((x A^T) B^T) * scale)."""
    import cases
    from conftest import weight_from_golden  # noqa: F401
    import oracle
    lo = cases.lora_inputs()
    host = oracle.port().quantize_nf4(lo["w"], 32)
    w = b2.PackedNf4Weight.from_host(host)
    got = _lora_forward(b2, w, torch.from_numpy(lo["x"]).cuda(), torch.from_numpy(lo["a"]).cuda(),
                        torch.from_numpy(lo["b"]).cuda(), float(lo["scale"]))
    assert rel_l2(got, golden["lora_adapted_linear"]) <= 2e-3


@pytest.mark.parametrize("rows,out_f,in_f,rank,dq", [
    (4, 4096, 4096, 16, True),       # decode rows: FP32-accumulate base kernel, tolerance 2e-3
    (32, 1024, 4096, 8, True),       # decode batch on the tensor cores
    (300, 1000, 1024, 64, False),    # prefill rows, ragged tiles, the largest rank
    (17, 256, 512, 3, True),         # a rank that fills no vector
])
def test_lora_against_oracle(b2, port, rows, out_f, in_f, rank, dq):
    rng = np.random.default_rng(rows + rank)
    W = (rng.standard_normal((out_f, in_f)) * 0.02).astype(np.float32)
    host = port.quantize_nf4_double_quantized(W, 64, 256) if dq else port.quantize_nf4(W, 64)
    x = rng.standard_normal((rows, in_f)).astype(np.float32)
    a = (rng.standard_normal((rank, in_f)) * 0.05).astype(np.float32)
    b = (rng.standard_normal((out_f, rank)) * 0.05).astype(np.float32)
    scale = 16.0 / rank
    w = b2.PackedNf4Weight.from_host(host)
    got = _lora_forward(b2, w, *(torch.from_numpy(t).cuda() for t in (x, a, b)), scale)
    base = port.linear_forward(host, x)
    branch = port.lora_forward(x, a, b, scale)
    assert np.isfinite(got).all()
    tol = 2e-3 if rows <= 16 else GEMM_TOL
    assert rel_l2(got, base + branch) <= tol
    # the branch on its own is FP32: subtracting the library's own base projection leaves it
    assert rel_l2(got - forward(b2, w, torch.from_numpy(x).cuda()), branch) <= 1e-4
    with pytest.raises(ValueError):
        _lora_forward(b2, w, torch.from_numpy(x).cuda(), torch.from_numpy(np.zeros((65, in_f), np.float32)).cuda(),
                      torch.from_numpy(np.zeros((out_f, 65), np.float32)).cuda(), 1.0)


def test_library_arena_under_graph_capture(b2, port):
    """The library's own scratch arena (workspace == NULL): a captured graph keeps working after
    the arena has grown for a later, larger call (memory that was handed out is never freed or
    moved), and a call that would have to grow the arena while its stream is being captured is
    refused instead of allocating inside the capture."""
    rng = np.random.default_rng(7)
    W = (rng.standard_normal((512, 1024)) * 0.02).astype(np.float32)
    host = port.quantize_nf4_double_quantized(W, 64, 256)
    w = b2.PackedNf4Weight.from_host(host)
    # a second call so large (1.2 GB of bf16 scratch) that no earlier test can have grown the arena past it
    big_rows = 600000
    x_small = torch.from_numpy(rng.standard_normal((64, 1024)).astype(np.float32)).cuda()
    x_big = torch.randn((big_rows, 1024), device="cuda")
    y_small = torch.empty((64, 512), device="cuda")
    y_big = torch.empty((big_rows, 512), device="cuda")
    shape_small, shape_big = (64, 1024, 512, 64), (big_rows, 1024, 512, 64)
    b2.dispatch_quantized_linear_forward(x_small, w, y_small, shape_small)   # arena sized outside capture
    torch.cuda.synchronize()
    first = y_small.clone()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    refused = None
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            b2.dispatch_quantized_linear_forward(x_small, w, y_small, shape_small)
            try:
                b2.dispatch_quantized_linear_forward(x_big, w, y_big, shape_big)
            except ValueError as e:   # nothing of the refused call was enqueued: the capture stays valid
                refused = str(e)
    torch.cuda.synchronize()
    assert refused is not None and "stream capture" in refused, refused
    b2.dispatch_quantized_linear_forward(x_big, w, y_big, shape_big)         # grows the arena
    torch.cuda.synchronize()
    y_small.zero_()
    graph.replay()                                                            # still points at the old arena
    torch.cuda.synchronize()
    b2.check_device_errors()
    assert torch.equal(y_small.view(torch.int32), first.view(torch.int32))
    sample = slice(0, 64)
    assert rel_l2(y_big[sample].cpu().numpy(), port.linear_forward(host, x_big[sample].cpu().numpy())) <= GEMM_TOL
