"""A small seeded decoder (real weights quantised by the CPU oracle) shared by
the CPU multi-rank test and the GPU parity test of the decode step."""
import numpy as np
import torch

import oracle
from oracle import decode_ref
from riftco_transformer_b200.decode import LAYER_WEIGHTS, DecoderConfig, weight_shapes

CFG = DecoderConfig(layers=2, d_model=512, q_heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=1024)
BATCH, CONTEXT = 3, 300


def host_model(seed=77):
    """Full (unsharded) host payloads, norms, embedding, KV pools and tables."""
    rng = np.random.default_rng(seed)
    port = oracle.port()
    shapes = weight_shapes(CFG)
    weights = {}
    for layer in range(CFG.layers):
        weights[layer] = {}
        for name in LAYER_WEIGHTS:
            W = (rng.standard_normal(shapes[name]) * 0.05).astype(np.float32)
            weights[layer][name] = port.quantize_nf4_double_quantized(W, 64, 32)
    weights["lm_head"] = port.quantize_nf4_double_quantized(
        (rng.standard_normal(shapes["lm_head"]) * 0.05).astype(np.float32), 64, 32)
    norms = {layer: {"attn": (1 + 0.1 * rng.standard_normal(CFG.d_model)).astype(np.float32),
                     "ffn": (1 + 0.1 * rng.standard_normal(CFG.d_model)).astype(np.float32)}
             for layer in range(CFG.layers)}
    norms["final"] = (1 + 0.1 * rng.standard_normal(CFG.d_model)).astype(np.float32)
    embedding = (rng.standard_normal((CFG.vocab, CFG.d_model)) * 0.5).astype(np.float32)
    lens = np.array([CONTEXT, 17, 256], np.int32)[:BATCH]       # tokens already cached per sequence
    blocks = -(-(lens.astype(np.int64) + 1) // CFG.block_size)
    total = int(blocks.sum())
    perm = rng.permutation(total)
    tables = np.zeros((BATCH, int(blocks.max())), np.int32)
    at = 0
    for s, nb in enumerate(blocks):
        tables[s, :nb] = perm[at:at + nb]
        at += nb
    pools = [(rng.standard_normal((total, CFG.kv_heads, CFG.block_size, CFG.head_dim)).astype(np.float32),
              rng.standard_normal((total, CFG.kv_heads, CFG.block_size, CFG.head_dim)).astype(np.float32))
             for _ in range(CFG.layers)]
    tokens = rng.integers(0, CFG.vocab, BATCH).astype(np.int32)
    return dict(weights=weights, norms=norms, embedding=embedding, lens=lens, tables=tables, pools=pools,
                tokens=tokens)


def checker_step(model, rank=0, world=1, group=None, whole=()):
    """DecodeStep over CheckerOps for one rank (row / KV-head shards of the host model; the
    weights named in `whole` are given to every rank unsharded)."""
    from riftco_transformer_b200.decode import DecodeStep
    ops = decode_ref.CheckerOps(group)
    hkv = CFG.kv_heads // world
    weights = {}
    for layer in range(CFG.layers):
        weights[layer] = {n: (model["weights"][layer][n] if n in whole else
                              decode_ref.shard_rows(model["weights"][layer][n], rank, world)) for n in LAYER_WEIGHTS}
    weights["lm_head"] = decode_ref.shard_rows(model["weights"]["lm_head"], rank, world)
    norms = {k: ({a: torch.from_numpy(b) for a, b in v.items()} if isinstance(v, dict) else torch.from_numpy(v))
             for k, v in model["norms"].items()}
    pools = [decode_ref.HostPool(torch.from_numpy(k[:, rank * hkv:(rank + 1) * hkv].copy()),
                                 torch.from_numpy(v[:, rank * hkv:(rank + 1) * hkv].copy()))
             for k, v in model["pools"]]
    step = DecodeStep(CFG, ops, weights, norms, torch.from_numpy(model["embedding"]), pools,
                      torch.from_numpy(model["tables"]), BATCH, int(model["lens"].max()) + 1, rank, world)
    return step


def run(step, model):
    lens = model["lens"]
    tokens = torch.from_numpy(model["tokens"])
    positions = torch.from_numpy(lens.copy())
    seq_lens = torch.from_numpy((lens + 1).astype(np.int32))
    dev = getattr(step.ops, "device", None)
    if dev is not None:
        tokens, positions, seq_lens = tokens.to(dev), positions.to(dev), seq_lens.to(dev)
    nxt, logits = step.step(tokens, positions, seq_lens)
    return nxt.cpu().numpy().copy(), logits.cpu().numpy().copy()


def oracle_payload(w):
    """The host payload (oracle.Nf4Weight) of a device-resident PackedNf4Weight."""
    codes = w.codes.cpu().numpy()
    if w.secondary is None:
        return oracle.Nf4Weight(codes, w.out_features, w.in_features, w.block_size, fp32_scales=w.primary.cpu().numpy())
    return oracle.Nf4Weight(codes, w.out_features, w.in_features, w.block_size, scale_codes=w.primary.cpu().numpy(),
                            second_level=w.secondary.cpu().numpy(), scale_block_size=w.scale_block_size,
                            offset=w.offset)


def checker_step_of(step):
    """The CPU checker's DecodeStep over the very tensors of an UNSHARDED CUDA DecodeStep (weights as
    host payloads, norms, embedding, KV pools, tables): what the oracle says the step must compute."""
    from riftco_transformer_b200.decode import DecodeStep
    assert step.world == 1
    cfg = step.cfg
    weights = {layer: {n: oracle_payload(step.w[layer][n]) for n in LAYER_WEIGHTS} for layer in range(cfg.layers)}
    weights["lm_head"] = oracle_payload(step.w["lm_head"])
    norms = {k: ({a: b.cpu() for a, b in v.items()} if isinstance(v, dict) else v.cpu()) for k, v in step.norms.items()}
    pools = [decode_ref.HostPool(p.key_pages.cpu().clone(), p.value_pages.cpu().clone()) for p in step.pools]
    return DecodeStep(cfg, decode_ref.CheckerOps(None), weights, norms, step.embedding.cpu(), pools,
                      step.tables.cpu(), step.batch, step.max_seq_len, 0, 1)
