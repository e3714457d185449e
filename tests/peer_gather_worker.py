"""One rank of the two-GPU peer all-gather check (started by test_gpu_peer_gather.py):
the library's peer-store gather against NCCL's all-gather on the same shards,
over several rounds, rotating buffers, eagerly and from a replayed CUDA graph."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from riftco_transformer_b200.decode import CudaOps
    ops = CudaOps(dev, dist.group.WORLD)
    assert ops.peer, "peer gather not enabled"
    rows, cols = 32, 2048
    bufs = [ops.gathered_buffer((rows, world * cols), with_bf16=(i == 1)) for i in range(2)]
    assert ops.bf16_of(bufs[0]) is None and ops.bf16_of(bufs[1]).dtype == torch.bfloat16
    gen = torch.Generator(device=dev)
    gen.manual_seed(100 + rank)
    stage = torch.empty((world, rows, cols), device=dev)
    for it in range(12):
        local = torch.randn((rows, cols), device=dev, generator=gen)
        full = bufs[it % 2]
        ops.all_gather_columns(local, None, full)
        dist.all_gather_into_tensor(stage.view(-1, cols), local)
        want = stage.permute(1, 0, 2).reshape(rows, world * cols)
        torch.cuda.synchronize()
        assert torch.equal(full, want), f"round {it}: mismatch on rank {rank}"
        if ops.bf16_of(full) is not None:
            assert torch.equal(ops.bf16_of(full), want.to(torch.bfloat16)), f"round {it}: bf16 copy on rank {rank}"
        dist.barrier()
    # graph: two gathers per replay, one per buffer
    local = torch.randn((rows, cols), device=dev, generator=gen)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            ops.all_gather_columns(local, None, bufs[0])
            ops.all_gather_columns(local, None, bufs[1])
        for _ in range(5):
            local.normal_(generator=gen)
            graph.replay()
            side.synchronize()
            dist.all_gather_into_tensor(stage.view(-1, cols), local)
            want = stage.permute(1, 0, 2).reshape(rows, world * cols)
            torch.cuda.synchronize()
            assert torch.equal(bufs[0], want) and torch.equal(bufs[1], want)
            assert torch.equal(ops.bf16_of(bufs[1]), want.to(torch.bfloat16))
            dist.barrier()   # a replay stores into the peer's buffers at once: wait until it has compared them
    ops.check_peer_status()
    dist.barrier()
    print("PEER_GATHER_OK", flush=True)
    os._exit(0)   # skip process-group teardown (it can block with live CUDA graphs)


if __name__ == "__main__":
    main()
