"""One rank of the multi-GPU decode-step check (started by test_gpu_peer_gather.py). A small
batch-32 decoder - one seeded quantised model, sharded by views - is stepped on `world` GPUs
 * with peer gathers that also deliver bf16 copies to the tensor-core linears, with peer gathers
   followed by conversion passes, and with NCCL gathers: same logits bit for bit on every rank;
 * with the o- and down-projections whole on every rank and with every linear row-sharded
   (flat_block_base != 0 on every rank but the first);
and rank 0 holds every layout to the unsharded step on its own GPU (same tokens; logits up to the
order of FP32 partial sums) and that one to the CPU oracle."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def rel_l2(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm())


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from riftco_transformer_b200.decode import DecoderConfig, synthetic_step
    cfg = DecoderConfig(layers=2, d_model=512, q_heads=8, kv_heads=4, head_dim=128, ffn=2048, vocab=2048)
    results = []
    for handoff, peer, whole in (("1", "1", None), ("0", "1", None), ("1", "0", None), ("1", "1", ())):
        os.environ["B2_BF16_HANDOFF"], os.environ["B2_PEER_GATHER"] = handoff, peer
        step, inputs = synthetic_step(cfg, 32, 100, rank, world, dev, dist.group.WORLD, whole=whole)
        assert step.ops.peer == (peer == "1")
        assert (step.ctx16 is not None) == (handoff == "1" and peer == "1")
        assert step.whole_o == (whole is None) and step.whole_down == (whole is None)
        if rank > 0:
            assert step.w[0]["wq"].flat_block_base != 0 and step.w["lm_head"].flat_block_base != 0
        dist.barrier()
        for _ in range(2):   # the second step appends to the same slot again: same result
            nxt, logits = step.step(inputs["tokens"], inputs["positions"], inputs["seq_lens"])
        torch.cuda.synchronize()
        assert int(step.status.item()) == 0
        step.ops.check_peer_status()
        results.append((nxt.clone(), logits.clone()))
        dist.barrier()
    for nxt, logits in results[1:3]:   # same layout, different plumbing: same bits
        assert torch.equal(logits, results[0][1]) and torch.equal(nxt, results[0][0])
    assert torch.isfinite(results[0][1]).all()
    if rank == 0:
        os.environ["B2_BF16_HANDOFF"] = "1"
        single, inputs = synthetic_step(cfg, 32, 100, 0, 1, dev, None)
        nxt1, logits1 = single.step(inputs["tokens"], inputs["positions"], inputs["seq_lens"])
        torch.cuda.synchronize()
        for nxt, logits in (results[0], results[3]):
            assert torch.equal(nxt, nxt1), "sharded and unsharded steps chose different tokens"
            assert rel_l2(logits, logits1) <= 1e-5, rel_l2(logits, logits1)
        import decode_cases
        single2, inputs2 = synthetic_step(cfg, 32, 100, 0, 1, dev, None)   # fresh pools: the oracle appends too
        checker = decode_cases.checker_step_of(single2)
        want_next, want_logits = checker.step(inputs2["tokens"].cpu(), inputs2["positions"].cpu(), inputs2["seq_lens"].cpu())
        assert rel_l2(logits1.cpu(), want_logits) <= 1e-2, rel_l2(logits1.cpu(), want_logits)   # bf16 linears, two layers
        agree = float((nxt1.cpu() == want_next).float().mean())
        assert agree >= 0.9, agree   # near-ties may flip under bf16 operands
    dist.barrier()
    print("DECODE_STEP_OK", flush=True)
    os._exit(0)   # skip process-group teardown


if __name__ == "__main__":
    main()
