"""The peer-store all-gather kernel (b2_peer_all_gather_columns).

One GPU: the kernel with every "peer" address pointing into this GPU's own
memory (world 1, and a two-rank layout emulated by running rank 0 and rank 1 one
after the other into the same buffers), epochs across calls and CUDA-graph
replays, and the bounded wait: a flag that nothing sets makes the kernel give up
after its time limit with B2_PEER_STATUS_TIMEOUT instead of spinning.
Two or more GPUs: real ranks over symmetric memory, checked against NCCL."""
import os
import socket
import subprocess
import sys
import time

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

PEER_STATUS_TIMEOUT = 16


@pytest.fixture(scope="module")
def b2():
    import riftco_transformer_b200 as pkg
    assert pkg.is_available(), pkg.unavailability_reason()
    return pkg


def _call(local, full_ptrs, flag_ptrs, rank, world, state, status):
    from riftco_transformer_b200._lib import lib
    from riftco_transformer_b200.backend import _check, _stream_ptr
    _check(lib.b2_peer_all_gather_columns(local.data_ptr(), local.shape[0], local.shape[1], full_ptrs.data_ptr(),
                                          flag_ptrs.data_ptr(), rank, world, state.data_ptr(), status.data_ptr(),
                                          _stream_ptr(None)))


def _ptrs(*tensors):
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device="cuda")


def test_world_one_epochs_and_graph_replay(b2):
    rows, cols = 32, 4096
    full = torch.zeros((rows, cols), device="cuda")
    flags = torch.zeros((64,), dtype=torch.int32, device="cuda")
    state = torch.zeros((2,), dtype=torch.int32, device="cuda")
    status = torch.zeros((1,), dtype=torch.int32, device="cuda")
    fp, gp = _ptrs(full), _ptrs(flags)
    local = torch.randn((rows, cols), device="cuda")
    for call in range(3):
        local.normal_()
        _call(local, fp, gp, 0, 1, state, status)
        torch.cuda.synchronize()
        assert torch.equal(full, local)
        assert state.tolist() == [call + 1, 0]
        assert flags[0].item() == call + 1
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        _call(local, fp, gp, 0, 1, state, status)
    for replay in range(3):
        local.normal_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(full, local)
    assert status.item() == 0


def test_two_rank_layout_on_one_gpu(b2):
    # Rank 1 runs first and finds rank 0's flag behind, so it would wait: give it a flag array of
    # its own that rank 0 has already "published" to; then rank 0 runs against the real flags.
    rows, cols = 8, 1024
    full = [torch.zeros((rows, 2 * cols), device="cuda") for _ in range(2)]
    flags = [torch.zeros((64,), dtype=torch.int32, device="cuda") for _ in range(2)]
    state = [torch.zeros((2,), dtype=torch.int32, device="cuda") for _ in range(2)]
    status = torch.zeros((1,), dtype=torch.int32, device="cuda")
    shard = [torch.randn((rows, cols), device="cuda") for _ in range(2)]
    fp, gp = _ptrs(*full), _ptrs(*flags)
    flags[1][0] = 1            # as if rank 0 had already arrived at rank 1
    _call(shard[1], fp, gp, 1, 2, state[1], status)
    torch.cuda.synchronize()
    flags[1][0] = 0
    assert flags[0][1].item() == 1 and flags[1][1].item() == 1
    _call(shard[0], fp, gp, 0, 2, state[0], status)   # rank 1's flag is there: returns at once
    torch.cuda.synchronize()
    want = torch.cat(shard, dim=1)
    assert torch.equal(full[0], want) and torch.equal(full[1], want)
    assert status.item() == 0


def test_two_rank_layout_with_bf16_copies(b2):
    """The same emulation through the entry that also fills every rank's bf16 buffer."""
    from riftco_transformer_b200._lib import lib
    from riftco_transformer_b200.backend import _check, _stream_ptr
    rows, cols = 8, 1024
    full = [torch.zeros((rows, 2 * cols), device="cuda") for _ in range(2)]
    full16 = [torch.zeros((rows, 2 * cols), device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    flags = [torch.zeros((64,), dtype=torch.int32, device="cuda") for _ in range(2)]
    state = [torch.zeros((2,), dtype=torch.int32, device="cuda") for _ in range(2)]
    status = torch.zeros((1,), dtype=torch.int32, device="cuda")
    shard = [torch.randn((rows, cols), device="cuda") for _ in range(2)]
    fp, hp, gp = _ptrs(*full), _ptrs(*full16), _ptrs(*flags)

    def call(rank):
        _check(lib.b2_peer_all_gather_columns_bf16(
            shard[rank].data_ptr(), rows, cols, fp.data_ptr(), hp.data_ptr(), gp.data_ptr(), rank, 2,
            state[rank].data_ptr(), status.data_ptr(), _stream_ptr(None)))

    flags[1][0] = 1            # as if rank 0 had already arrived at rank 1
    call(1)
    torch.cuda.synchronize()
    flags[1][0] = 0
    call(0)
    torch.cuda.synchronize()
    want = torch.cat(shard, dim=1)
    for r in range(2):
        assert torch.equal(full[r], want) and torch.equal(full16[r], want.to(torch.bfloat16))
    assert status.item() == 0


def test_wait_gives_up_with_a_status_bit(b2):
    rows, cols = 4, 256
    full = [torch.zeros((rows, 2 * cols), device="cuda") for _ in range(2)]
    flags = [torch.zeros((64,), dtype=torch.int32, device="cuda") for _ in range(2)]
    state = torch.zeros((2,), dtype=torch.int32, device="cuda")
    status = torch.zeros((1,), dtype=torch.int32, device="cuda")
    local = torch.randn((rows, cols), device="cuda")
    _call(local, _ptrs(*full), _ptrs(*flags), 0, 2, state, status)   # nobody plays rank 1
    torch.cuda.synchronize()
    assert status.item() & PEER_STATUS_TIMEOUT
    assert torch.equal(full[0][:, :cols], local)     # its own part was still delivered
    # the context is still usable
    assert float((local + 1).sum().item()) == pytest.approx(float(local.sum().item()) + rows * cols, rel=1e-4)


def test_rejects_bad_arguments(b2):
    t = torch.zeros((4, 6), device="cuda")
    z = torch.zeros((64,), dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError):
        _call(t, _ptrs(t), _ptrs(z), 0, 1, z, z)          # cols not a multiple of 4
    t = torch.zeros((4, 8), device="cuda")
    with pytest.raises(ValueError):
        _call(t, _ptrs(t), _ptrs(z), 2, 2, z, z)          # rank >= world


def _run_two_ranks(worker_file: str, marker: str) -> None:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    worker = os.path.join(os.path.dirname(__file__), worker_file)
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, worker], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    # A rank that fails leaves the other one waiting in a collective: stop both as soon as one
    # has exited with an error, or after two minutes.
    deadline = time.monotonic() + 120
    while time.monotonic() < deadline and any(p.poll() is None for p in procs):
        if any(p.poll() not in (None, 0) for p in procs):
            break
        time.sleep(0.2)
    for p in procs:
        if p.poll() is None:
            time.sleep(1.0)   # let a rank that is about to finish do so
        if p.poll() is None:
            p.kill()
    outs = [p.communicate()[0] for p in procs]
    report = "\n".join(f"--- rank {r} (exit {p.returncode}) ---\n{o[-2500:]}"
                       for r, (p, o) in enumerate(zip(procs, outs)))
    assert all(p.returncode == 0 for p in procs), report
    assert all(marker in o for o in outs), report


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_match_nccl():
    _run_two_ranks("peer_gather_worker.py", "PEER_GATHER_OK")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_decode_step_variants_agree():
    """Batch-32 decode step on two ranks: bf16 copies delivered by the gather, conversion passes
    instead, and NCCL gathers all give the same logits bit for bit."""
    _run_two_ranks("decode_step_worker.py", "DECODE_STEP_OK")
