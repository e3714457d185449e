"""The decode step's multi-rank orchestration on CPU: world_size 2 over gloo
with the checker backend must reproduce the single-rank result (row-sharded
linears, KV-head-sharded attention, all-gathers at the layer boundaries)."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import decode_cases


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir, whole=()):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    model = decode_cases.host_model()
    step = decode_cases.checker_step(model, rank, world, dist.group.WORLD, whole)
    nxt, logits = decode_cases.run(step, model)
    np.save(os.path.join(out_dir, f"logits{rank}.npy"), logits)
    np.save(os.path.join(out_dir, f"next{rank}.npy"), nxt)
    dist.destroy_process_group()


import pytest


@pytest.mark.parametrize("whole", [(), ("wo", "w_down")], ids=["all-sharded", "o-and-down-whole"])
def test_two_ranks_match_one_rank(tmp_path, whole):
    """Row / KV-head shards with four gathers per layer, and the variant that keeps the o- and
    down-projections whole on every rank (two gathers per layer)."""
    model = decode_cases.host_model()
    nxt1, logits1 = decode_cases.run(decode_cases.checker_step(model), model)
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), whole), nprocs=2, join=True)
    for rank in range(2):
        logits = np.load(tmp_path / f"logits{rank}.npy")
        nxt = np.load(tmp_path / f"next{rank}.npy")
        # every output element is computed by the same loop on the same inputs: bit-identical
        assert (logits.view(np.uint32) == logits1.view(np.uint32)).all()
        assert (nxt == nxt1).all()


def test_shard_check_rejects_uneven_splits():
    from riftco_transformer_b200.decode import DecoderConfig
    with pytest.raises(ValueError):
        DecoderConfig(kv_heads=8).shard_check(3)
