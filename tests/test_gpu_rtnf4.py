"""Weights loaded straight from an RTNF4S1 stream into device memory: whole and
as row shards, bit-exact against the CPU oracle's dequantisation of the same
payloads, and usable by the linear kernels."""
import numpy as np
import pytest
import torch

from conftest import rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def b2():
    import riftco_transformer_b200 as pkg
    assert pkg.is_available(), pkg.unavailability_reason()
    return pkg


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def test_stream_to_device_whole_and_sharded(b2, port):
    from riftco_transformer_b200 import rtnf4
    rng = np.random.default_rng(11)
    hosts = [
        port.quantize_nf4_double_quantized((rng.standard_normal((256, 512)) * 0.02).astype(np.float32), 64, 256),
        port.quantize_nf4((rng.standard_normal((64, 128)) * 0.3).astype(np.float32), 64),
    ]
    stream = rtnf4.dumps(hosts)
    entries = rtnf4.index(stream)
    for entry, host in zip(entries, hosts):
        want = port.dequantize(host)
        whole = rtnf4.load_weight(stream, entry)
        assert (bits(b2.dequantize(whole).cpu().numpy()) == bits(want)).all()
        parts = [rtnf4.load_weight(stream, entry, rank=r, world=4) for r in range(4)]
        got = np.concatenate([b2.dequantize(p).cpu().numpy() for p in parts], axis=0)
        assert (bits(got) == bits(want)).all()
        # a shard loaded from the stream equals the same shard viewed out of the whole weight
        for r, p in enumerate(parts):
            view = whole.row_shard(r, 4)
            assert torch.equal(p.codes, view.codes) and torch.equal(p.primary, view.primary)
            assert p.flat_block_base == view.flat_block_base
    # and it feeds the decode kernel
    x = rng.standard_normal((4, 512)).astype(np.float32)
    w = rtnf4.load_weight(stream, entries[0])
    y = torch.empty((4, 256), device="cuda")
    b2.dispatch_quantized_linear_forward(torch.from_numpy(x).cuda(), w, y, (4, 512, 256, 64))
    assert rel_l2(y.cpu().numpy(), port.linear_forward(hosts[0], x)) <= 2e-3
