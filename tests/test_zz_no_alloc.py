"""The allocation-free attention entry point (b2_paged_decode_attention_noalloc).

It exists for callers that cannot allocate device memory where they run
attention - an engine whose memory all belongs to its own pool, or a call site
where cudaMalloc / cudaFree are unwelcome because they synchronise the device -
so its split-K scratch is a fixed array inside the library. The test calls it
through the C ABI twice in a row, with different inputs the second time (the
shared scratch still holds the first call's partial results), and checks each
result against b2_paged_decode_attention given an explicit workspace - the two
entry points run the same kernels, so the results must agree bit for bit - and
once against the CPU oracle. It also checks that the call leaves the device's
free memory untouched. It is collected last so that a run stopping at the first
failure has already run every other test, and it passes on its own in a fresh
process as well."""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import rel_l2

pytestmark = pytest.mark.gpu

TOL = 2e-3  # the tolerance of the other attention tests, for the comparison with the oracle


def _case(seed, n_seq, lens):
    from riftco_transformer_b200 import synth
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    pool, tables, dlens = synth.paged_cache(lens, kv_heads=8, seed=seed)
    q = torch.randn((n_seq, 32, 128), device="cuda", generator=g)
    return q, pool, tables, dlens


def _call(lib, noalloc, q, pool, tables, dlens, max_len):
    ctx = torch.full_like(q, float("nan"))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    common = (q.data_ptr(), pool.key_pages.data_ptr(), pool.value_pages.data_ptr(), tables.data_ptr(),
              dlens.data_ptr(), ctx.data_ptr(), q.shape[0], 32, 8, 128, 16, pool.physical_blocks,
              tables.shape[1], max_len)
    if noalloc:
        rc = lib.b2_paged_decode_attention_noalloc(*common, status.data_ptr(), stream)
        ws = None
    else:
        need = lib.b2_paged_decode_workspace_bytes(q.shape[0], 32, 128, 16, max_len)
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
        rc = lib.b2_paged_decode_attention(*common, ws.data_ptr(), ws.numel(), status.data_ptr(), stream)
    torch.cuda.synchronize()
    return rc, ctx.cpu().numpy(), int(status.item())


def test_noalloc_entry_matches_workspace_entry_on_two_calls_in_a_row():
    from riftco_transformer_b200 import _lib
    lib = _lib.lib
    assert lib.b2_is_available() == 1
    first = _case(101, 6, [1, 255, 257, 1024, 2049, 3000])
    second = _case(202, 4, [4096, 17, 600, 2500])
    for q, pool, tables, dlens in (first, second):
        max_len = int(dlens.max().item())
        rc_a, got, st_a = _call(lib, True, q, pool, tables, dlens, max_len)
        rc_b, want, st_b = _call(lib, False, q, pool, tables, dlens, max_len)
        assert rc_a == 0, lib.b2_last_error().decode()
        assert rc_b == 0, lib.b2_last_error().decode()
        assert st_a == 0 and st_b == 0
        assert np.isfinite(got).all()
        assert rel_l2(got, want) <= TOL
        assert (got.view(np.uint32) == want.view(np.uint32)).all()   # same kernels: same bits
    # the second case once more against the CPU oracle
    import oracle
    q, pool, tables, dlens = second
    _, got, _ = _call(lib, True, q, pool, tables, dlens, int(dlens.max().item()))
    want = oracle.port().paged_decode_gqa(q.cpu().numpy(), pool.key_pages.cpu().numpy(), pool.value_pages.cpu().numpy(),
                                          tables.cpu().numpy().astype(np.uint32), dlens.cpu().numpy().astype(np.uint32))
    assert rel_l2(got, want) <= TOL


def test_noalloc_entry_leaves_free_memory_untouched():
    """cudaMemGetInfo before and after a call (after one warm-up call that looks the scratch address
    up): the entry point must not allocate, whatever the shape within its limit."""
    from riftco_transformer_b200 import _lib
    lib = _lib.lib
    q, pool, tables, dlens = _case(404, 5, [300, 4000, 17, 2049, 1024])
    max_len = int(dlens.max().item())
    ctx = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    args = (q.data_ptr(), pool.key_pages.data_ptr(), pool.value_pages.data_ptr(), tables.data_ptr(),
            dlens.data_ptr(), ctx.data_ptr(), 5, 32, 8, 128, 16, pool.physical_blocks, tables.shape[1], max_len,
            status.data_ptr(), stream)
    assert lib.b2_paged_decode_attention_noalloc(*args) == 0, lib.b2_last_error().decode()
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert lib.b2_paged_decode_attention_noalloc(*args) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert int(status.item()) == 0


def test_noalloc_entry_rejects_shapes_beyond_its_fixed_scratch():
    from riftco_transformer_b200 import _lib
    lib = _lib.lib
    # 64 sequences x 32 heads x 32 splits x 520 B = 34 MB > the fixed 8 MiB
    need = lib.b2_paged_decode_workspace_bytes(64, 32, 128, 16, 8192)
    assert need > _lib.NOALLOC_SCRATCH_BYTES
    q, pool, tables, dlens = _case(303, 64, [8192] + [16] * 63)
    rc, _, _ = _call(lib, True, q, pool, tables, dlens, 8192)
    assert rc == _lib.STATUS_INVALID_ARGUMENT
    message = lib.b2_last_error().decode()
    assert "scratch" in message and str(_lib.NOALLOC_SCRATCH_BYTES) in message
