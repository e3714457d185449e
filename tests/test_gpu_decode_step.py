"""The decode step on the GPU (CudaOps, C ABI) against the same step run with
the CPU checker backend, plus the glue operators one by one."""
import numpy as np
import pytest
import torch

import decode_cases
from conftest import rel_l2
from oracle import decode_ref

pytestmark = pytest.mark.gpu


def cuda_step(model):
    import riftco_transformer_b200 as b2
    from riftco_transformer_b200.decode import LAYER_WEIGHTS, CudaOps, DecodeStep
    cfg = decode_cases.CFG
    dev = torch.device("cuda", 0)
    ops = CudaOps(dev)
    weights = {layer: {n: b2.PackedNf4Weight.from_host(model["weights"][layer][n]) for n in LAYER_WEIGHTS}
               for layer in range(cfg.layers)}
    weights["lm_head"] = b2.PackedNf4Weight.from_host(model["weights"]["lm_head"])
    norms = {k: ({a: torch.from_numpy(b).to(dev) for a, b in v.items()} if isinstance(v, dict)
                 else torch.from_numpy(v).to(dev)) for k, v in model["norms"].items()}
    pools = [b2.PagedKvPool(torch.from_numpy(k).to(dev), torch.from_numpy(v).to(dev)) for k, v in model["pools"]]
    return DecodeStep(cfg, ops, weights, norms, torch.from_numpy(model["embedding"]).to(dev), pools,
                      torch.from_numpy(model["tables"]).to(dev), decode_cases.BATCH,
                      int(model["lens"].max()) + 1)


def test_decode_step_matches_checker():
    model = decode_cases.host_model()
    want_next, want_logits = decode_cases.run(decode_cases.checker_step(model), model)
    step = cuda_step(model)
    got_next, got_logits = decode_cases.run(step, model)
    torch.cuda.synchronize()
    assert int(step.status.item()) == 0
    assert np.isfinite(got_logits).all()
    assert rel_l2(got_logits, want_logits) <= 5e-3   # two layers of 2e-3 operators compounded
    assert (got_next == want_next).all()
    # the appended K/V slots hold the rotated key and the value bit for bit (pure copies / exact formulas aside)
    ref = decode_cases.checker_step(model)
    decode_cases.run(ref, model)
    for layer in range(decode_cases.CFG.layers):
        assert rel_l2(step.pools[layer].key_pages.cpu().numpy(), ref.pools[layer].key_pages.numpy()) <= 5e-3
        assert rel_l2(step.pools[layer].value_pages.cpu().numpy(), ref.pools[layer].value_pages.numpy()) <= 5e-3


def test_glue_operators():
    from riftco_transformer_b200.decode import CudaOps
    import riftco_transformer_b200 as b2
    dev = torch.device("cuda", 0)
    ops = CudaOps(dev)
    rng = np.random.default_rng(5)
    x = rng.standard_normal((5, 4096)).astype(np.float32)
    delta = rng.standard_normal((5, 4096)).astype(np.float32)
    scale = (1 + 0.1 * rng.standard_normal(4096)).astype(np.float32)
    tx, td, ts = (torch.from_numpy(a).to(dev) for a in (x, delta, scale))
    y = torch.empty_like(tx)
    ops.rmsnorm(tx, None, None, ts, y, 1e-5)
    assert rel_l2(y.cpu().numpy(), decode_ref.rms_norm(x, scale, 1e-5)) <= 1e-6
    xo = torch.empty_like(tx)
    ops.rmsnorm(tx, td, xo, ts, y, 1e-5)
    assert (xo.cpu().numpy() == x + delta).all()
    assert rel_l2(y.cpu().numpy(), decode_ref.rms_norm(x + delta, scale, 1e-5)) <= 1e-6

    g = rng.standard_normal((7, 1000)).astype(np.float32) * 4
    g[0, 0] = -np.inf
    u = rng.standard_normal((7, 1000)).astype(np.float32)
    out = torch.empty((7, 1000), device=dev)
    ops.silu_mul(torch.from_numpy(g).to(dev), torch.from_numpy(u).to(dev), out)
    want = decode_ref.silu(g) * u
    want[0, 0] = -0.0 * u[0, 0]
    assert np.allclose(out.cpu().numpy(), want, rtol=2e-6, atol=1e-7)

    logits = rng.standard_normal((4, 32000)).astype(np.float32)
    logits[1, 77] = logits[1, 9000] = 50.0   # tie: lowest index wins
    idx = torch.empty(4, dtype=torch.int32, device=dev)
    ops.argmax(torch.from_numpy(logits).to(dev), idx)
    assert (idx.cpu().numpy() == np.argmax(logits, axis=1)).all() and int(idx[1]) == 77

    # RoPE + append at several positions, including position 0 and a page boundary
    hq, hkv, d, bs = 4, 2, 128, 16
    positions = np.array([0, 15, 16, 301], np.int32)
    P = 40
    tables = rng.permutation(P)[:4 * 20].reshape(4, 20).astype(np.int32) if P >= 80 else \
        np.stack([rng.permutation(P)[:20] for _ in range(4)]).astype(np.int32)
    q = rng.standard_normal((4, hq, d)).astype(np.float32)
    k = rng.standard_normal((4, hkv, d)).astype(np.float32)
    v = rng.standard_normal((4, hkv, d)).astype(np.float32)
    pool = b2.PagedKvPool(torch.zeros((P, hkv, bs, d), device=dev), torch.zeros((P, hkv, bs, d), device=dev))
    tq = torch.from_numpy(q).to(dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    # distinct pages per sequence so the slots do not collide
    tables = np.arange(80, dtype=np.int32).reshape(4, 20) % P
    tables[1] = (tables[1] + 7) % P
    ops.rope_append(tq, torch.from_numpy(k).to(dev), torch.from_numpy(v).to(dev), torch.from_numpy(positions).to(dev),
                    torch.from_numpy(tables).to(dev), pool, 1e4, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for s, pos in enumerate(positions):
        assert np.allclose(tq[s].cpu().numpy(), decode_ref.rotate(q[s], int(pos), 1e4), rtol=1e-6, atol=1e-6)
    s = 3
    page, slot = tables[s, positions[s] // bs], positions[s] % bs
    assert np.allclose(pool.key_pages[page, :, slot].cpu().numpy(), decode_ref.rotate(k[s], 301, 1e4), rtol=1e-6, atol=1e-6)
    assert (pool.value_pages[page, :, slot].cpu().numpy() == v[s]).all()


@pytest.mark.parametrize("hq,hkv,d", [(32, 8, 128), (5, 1, 96), (3, 3, 40)])
def test_rope_append_over_several_slices(hq, hkv, d):
    """Head counts that spread one sequence over several CTAs, and head widths whose channel pairs
    do not divide the CTA stride (every thread then evaluates an angle per item)."""
    from riftco_transformer_b200.decode import CudaOps
    import riftco_transformer_b200 as b2
    dev = torch.device("cuda", 0)
    ops = CudaOps(dev)
    rng = np.random.default_rng(11)
    n_seq, bs, P = 6, 16, 60
    positions = np.array([0, 1, 31, 32, 77, 159], np.int32)
    tables = np.stack([(np.arange(10) * n_seq + s) % P for s in range(n_seq)]).astype(np.int32)
    q = rng.standard_normal((n_seq, hq, d)).astype(np.float32)
    k = rng.standard_normal((n_seq, hkv, d)).astype(np.float32)
    v = rng.standard_normal((n_seq, hkv, d)).astype(np.float32)
    pool = b2.PagedKvPool(torch.zeros((P, hkv, bs, d), device=dev), torch.zeros((P, hkv, bs, d), device=dev))
    tq = torch.from_numpy(q).to(dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ops.rope_append(tq, torch.from_numpy(k).to(dev), torch.from_numpy(v).to(dev),
                    torch.from_numpy(positions).to(dev), torch.from_numpy(tables).to(dev), pool, 1e4, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    written = 0
    for s, pos in enumerate(positions):
        assert np.allclose(tq[s].cpu().numpy(), decode_ref.rotate(q[s], int(pos), 1e4), rtol=1e-6, atol=1e-6)
        page, slot = tables[s, pos // bs], pos % bs
        assert np.allclose(pool.key_pages[page, :, slot].cpu().numpy(), decode_ref.rotate(k[s], int(pos), 1e4),
                           rtol=1e-6, atol=1e-6)
        assert (pool.value_pages[page, :, slot].cpu().numpy() == v[s]).all()
        written += hkv * d
    # nothing but the six slots was touched
    assert int((pool.value_pages != 0).sum().item()) <= written
    assert int((pool.key_pages != 0).sum().item()) <= written


def test_argmax_row_shapes():
    """Widths that take the scalar path, rows shorter than the CTA, ties across threads."""
    from riftco_transformer_b200.decode import CudaOps
    dev = torch.device("cuda", 0)
    ops = CudaOps(dev)
    rng = np.random.default_rng(13)
    for width in (1, 3, 257, 1023, 4096, 32003, 128256):
        logits = rng.standard_normal((3, width)).astype(np.float32)
        if width > 2:
            logits[2, width - 1] = logits[2, width // 2] = 9.0
        idx = torch.empty(3, dtype=torch.int32, device=dev)
        ops.argmax(torch.from_numpy(logits).to(dev), idx)
        assert (idx.cpu().numpy() == np.argmax(logits, axis=1)).all(), width


def test_bf16_copies_of_the_glue_outputs():
    """RMSNorm and SiLU*up write, next to their FP32 result, exactly its bf16 rounding."""
    from riftco_transformer_b200.decode import CudaOps
    dev = torch.device("cuda", 0)
    ops = CudaOps(dev)
    g = torch.Generator(device=dev)
    g.manual_seed(3)
    for width in (4096, 1000, 37):   # 16-byte rows, 8-byte rows, the scalar path
        x = torch.randn((19, width), device=dev, generator=g)
        delta = torch.randn((19, width), device=dev, generator=g)
        scale = 1 + 0.1 * torch.randn(width, device=dev, generator=g)
        y, y2, xo = torch.empty_like(x), torch.empty_like(x), torch.empty_like(x)
        y16 = torch.empty((19, width), device=dev, dtype=torch.bfloat16)
        ops.rmsnorm(x, delta, xo, scale, y, 1e-5, y16)
        ops.rmsnorm(x, delta, xo, scale, y2, 1e-5)
        assert torch.equal(y, y2) and torch.equal(y16, y.to(torch.bfloat16))
        out, out16 = torch.empty_like(x), torch.empty((19, width), device=dev, dtype=torch.bfloat16)
        ops.silu_mul(x, delta, out, out16)
        assert torch.equal(out16, out.to(torch.bfloat16))


def test_linear_on_bf16_activations_equals_the_fp32_entry():
    from riftco_transformer_b200 import synth
    from riftco_transformer_b200.decode import CudaOps
    dev = torch.device("cuda", 0)
    ops = CudaOps(dev)
    g = torch.Generator(device=dev)
    g.manual_seed(4)
    ws = [synth.packed_weight(o, 512, seed=60 + i) for i, o in enumerate((512, 256, 384))]
    for rows in (17, 32, 200):
        assert ops.linear_bf16_supported(ws, rows)
        x = torch.randn((rows, 512), device=dev, generator=g)
        want = [torch.empty((rows, w.out_features), device=dev) for w in ws]
        got = [torch.empty_like(t) for t in want]
        ops.linear_multi(x, ws, want)
        ops.linear_multi_bf16(x.to(torch.bfloat16), ws, got)
        for a, b in zip(got, want):
            assert torch.equal(a, b)
        one = torch.empty_like(want[1])
        ops.linear_multi_bf16(x.to(torch.bfloat16), [ws[1]], [one])
        assert torch.equal(one, want[1])
    assert not ops.linear_bf16_supported(ws, 16)          # the GEMV takes FP32 activations
    assert not ops.linear_bf16_supported(ws * 2, 32)      # more than four weights
    with pytest.raises(Exception):
        ops.linear_multi_bf16(torch.zeros((8, 512), device=dev, dtype=torch.bfloat16), ws,
                              [torch.empty((8, w.out_features), device=dev) for w in ws])


def test_decode_step_with_and_without_the_bf16_handoff(monkeypatch):
    """Batch 32 takes the tensor-core linears: the step whose producers hand bf16 copies to them
    gives bit for bit the logits of the step that converts in a pass of its own."""
    from riftco_transformer_b200.decode import DecoderConfig, synthetic_step
    cfg = DecoderConfig(layers=2, d_model=512, q_heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2048)
    results = []
    for flag in ("1", "0"):
        monkeypatch.setenv("B2_BF16_HANDOFF", flag)
        step, inputs = synthetic_step(cfg, 32, 100, device=torch.device("cuda", 0))
        assert (step.n16 is not None) == (flag == "1") and (step.h16 is not None) == (flag == "1")
        step.ops.launches = 0
        nxt, logits = step.step(inputs["tokens"], inputs["positions"], inputs["seq_lens"])
        torch.cuda.synchronize()
        assert int(step.status.item()) == 0
        results.append((nxt.clone(), logits.clone(), step.ops.launches))
    assert torch.equal(results[0][1], results[1][1]) and torch.equal(results[0][0], results[1][0])
    assert results[0][2] == results[1][2] - (4 * cfg.layers + 1)   # one pass less per q/k/v, o, gate/up, down, LM head


def test_rope_append_of_a_prefill_chunk():
    """b2_rope_append_kv_tokens: a chunk of tokens of several sequences in one call writes exactly what
    token-by-token calls write (same q, same K / V pages), and what the CPU restatement - pinned to the
    reference's paged cache - says."""
    from riftco_transformer_b200._lib import lib
    from riftco_transformer_b200.backend import _check
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(21)
    hq, hkv, d, bs, P, max_blocks = 8, 2, 128, 16, 24, 6
    # tokens of three sequences, interleaved and out of order: (sequence, position)
    toks = [(0, 0), (1, 17), (0, 1), (2, 95), (0, 2), (1, 18), (0, 15), (0, 16), (2, 64), (1, 16)]
    tables = np.stack([rng.permutation(P)[:max_blocks] for _ in range(3)]).astype(np.int32)
    # make the three rows disjoint so that no two tokens share a slot
    tables = (np.arange(3 * max_blocks).reshape(3, max_blocks)).astype(np.int32) % P
    q = rng.standard_normal((len(toks), hq, d)).astype(np.float32)
    k = rng.standard_normal((len(toks), hkv, d)).astype(np.float32)
    v = rng.standard_normal((len(toks), hkv, d)).astype(np.float32)
    token_seq = np.array([s for s, _ in toks], np.int32)
    positions = np.array([p for _, p in toks], np.int32)

    def fresh():
        return (torch.full((P, hkv, bs, d), 7.0, device=dev), torch.full((P, hkv, bs, d), -7.0, device=dev))

    K1, V1 = fresh()
    q1 = torch.from_numpy(q).to(dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    tt, tk, tv = torch.from_numpy(tables).to(dev), torch.from_numpy(k).to(dev), torch.from_numpy(v).to(dev)
    d_pos, d_seq = torch.from_numpy(positions).to(dev), torch.from_numpy(token_seq).to(dev)
    _check(lib.b2_rope_append_kv_tokens(q1.data_ptr(), tk.data_ptr(), tv.data_ptr(), d_pos.data_ptr(),
                                        d_seq.data_ptr(), tt.data_ptr(), K1.data_ptr(),
                                        V1.data_ptr(), len(toks), hq, hkv, d, bs, P, max_blocks, 1e4, status.data_ptr(), None))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    # token by token through the single-token entry point (one "sequence" per call)
    K2, V2 = fresh()
    q2 = torch.from_numpy(q).to(dev)
    keep = []   # the calls only enqueue: their arguments must outlive the loop
    for t, (s, pos) in enumerate(toks):
        row = torch.from_numpy(tables[s:s + 1]).to(dev)
        one = torch.tensor([pos], dtype=torch.int32, device=dev)
        keep += [row, one]
        _check(lib.b2_rope_append_kv(q2[t:t + 1].data_ptr(), tk[t:t + 1].data_ptr(), tv[t:t + 1].data_ptr(),
                                     one.data_ptr(), row.data_ptr(), K2.data_ptr(), V2.data_ptr(), 1, hq, hkv, d, bs, P,
                                     max_blocks, 1e4, status.data_ptr(), None))
    torch.cuda.synchronize()
    assert torch.equal(q1, q2) and torch.equal(K1, K2) and torch.equal(V1, V2)
    # against the CPU restatement
    for t, (s, pos) in enumerate(toks):
        page, slot = tables[s, pos // bs], pos % bs
        assert rel_l2(q1[t].cpu().numpy(), decode_ref.rotate(q[t], pos, 1e4)) <= 1e-6
        assert rel_l2(K1[page, :, slot].cpu().numpy(), decode_ref.rotate(k[t], pos, 1e4)) <= 1e-6
        assert np.array_equal(V1[page, :, slot].cpu().numpy(), v[t])
    written = sorted((int(tables[s, p // bs]), p % bs) for s, p in toks)
    mask = torch.ones((P, bs), dtype=torch.bool, device=dev)
    for page, slot in written:
        mask[page, slot] = False
    assert (V1.permute(0, 2, 1, 3)[mask] == -7.0).all() and (K1.permute(0, 2, 1, 3)[mask] == 7.0).all()
