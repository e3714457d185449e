"""One rank of the two-GPU decode-step check (started by test_gpu_peer_gather.py): a small
batch-32 decoder stepped three ways - peer gathers that also deliver bf16 copies to the
tensor-core linears, peer gathers followed by conversion passes, NCCL gathers - must give
the same logits bit for bit on every rank."""
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
    from riftco_transformer_b200.decode import DecoderConfig, synthetic_step
    cfg = DecoderConfig(layers=2, d_model=512, q_heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2048)
    results = []
    for handoff, peer in (("1", "1"), ("0", "1"), ("1", "0")):
        os.environ["B2_BF16_HANDOFF"], os.environ["B2_PEER_GATHER"] = handoff, peer
        step, inputs = synthetic_step(cfg, 32, 100, rank, world, dev, dist.group.WORLD)
        assert step.ops.peer == (peer == "1")
        assert (step.ctx16 is not None) == (handoff == "1" and peer == "1")
        assert (step.hfull16 is not None) == (handoff == "1" and peer == "1")
        dist.barrier()
        for _ in range(2):   # the second step appends to the same slot again: same result
            nxt, logits = step.step(inputs["tokens"], inputs["positions"], inputs["seq_lens"])
        torch.cuda.synchronize()
        assert int(step.status.item()) == 0
        step.ops.check_peer_status()
        results.append((nxt.clone(), logits.clone()))
        dist.barrier()
    for nxt, logits in results[1:]:
        assert torch.equal(logits, results[0][1]) and torch.equal(nxt, results[0][0])
    assert torch.isfinite(results[0][1]).all()
    print("DECODE_STEP_OK", flush=True)
    os._exit(0)   # skip process-group teardown


if __name__ == "__main__":
    main()
