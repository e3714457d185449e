"""numpy restatement of the reference primitives around the hot-path operators
in a decode step (test infrastructure, never imported by the product):

  rms_norm        src/nn/rms_norm.cpp:39-73                  (in riftco_oracle.c)
  rotate_forward  src/model/rotary_embedding.cpp:64-117 (split-half pairs, angle in double)
  silu_forward    src/nn/activations.cpp:38-58 (stable sigmoid) (in riftco_oracle.c)
  SwiGLU          src/model/swiglu.cpp:27-29
  copy_token_to_page  src/stages/serving/cache/page_table_cache.cpp:44-77
  GreedySampler   src/stages/serving/generation.cpp:100-110  (in riftco_oracle.c)

Each of them is held bit for bit to vectors written by the reference's own code
(tests/golden/reference_vectors.npz, tests/test_oracle_golden.py).

and `CheckerOps`, an implementation of the `ops` interface of
riftco_transformer_b200.decode.DecodeStep on CPU tensors, with the packed
linears and the paged attention done by the C oracle. It lets the CPU tests run
the step's orchestration (sharding, buffer flow, all-gathers over gloo) and
gives the GPU test its expected values.
"""
from __future__ import annotations

import numpy as np
import torch

from . import Nf4Weight, port


def rms_norm(x: np.ndarray, scale: np.ndarray, eps: float) -> np.ndarray:
    """The C restatement: sequential FP32 mean like the reference's reduction."""
    return port().rms_norm(x, scale, eps)


def rotary_cos_sin(position: int, half: int, width: int, theta: float):
    c = np.arange(half, dtype=np.float64)
    angle = float(position) * np.power(float(theta), -2.0 * c / float(width))
    return np.cos(angle).astype(np.float32), np.sin(angle).astype(np.float32)


def rotate(v: np.ndarray, position: int, theta: float) -> np.ndarray:
    """v [..., width]; pairs (c, c + width/2)."""
    width = v.shape[-1]
    half = width // 2
    cs, sn = rotary_cos_sin(position, half, width, theta)
    a, b = v[..., :half], v[..., half:]
    return np.concatenate([a * cs - b * sn, b * cs + a * sn], axis=-1).astype(np.float32)


def silu(x: np.ndarray) -> np.ndarray:
    """The C restatement (libm expf, -inf -> -0.0, as the reference)."""
    return port().silu_mul(x)


def shard_rows(w: Nf4Weight, rank: int, world: int) -> Nf4Weight:
    """Rows [rank*out/world, ...) of a host payload; needs block- and
    group-aligned shard boundaries (the checker has no flat_block_base)."""
    rows = w.out_features // world
    first, count = rank * rows * w.in_features, rows * w.in_features
    assert first % w.block_size == 0 and count % w.block_size == 0
    b0, nb = first // w.block_size, count // w.block_size
    if w.fp32_scales is not None:
        return Nf4Weight(w.codes[first // 2:(first + count) // 2].copy(), rows, w.in_features, w.block_size,
                         fp32_scales=w.fp32_scales[b0:b0 + nb].copy())
    assert b0 % w.scale_block_size == 0 and nb % w.scale_block_size == 0
    g0, ng = b0 // w.scale_block_size, nb // w.scale_block_size
    return Nf4Weight(w.codes[first // 2:(first + count) // 2].copy(), rows, w.in_features, w.block_size,
                     scale_codes=w.scale_codes[b0:b0 + nb].copy(), second_level=w.second_level[g0:g0 + ng].copy(),
                     scale_block_size=w.scale_block_size, offset=w.offset)


class HostPool:
    """K/V page pools as CPU tensors, same fields as PagedKvPool."""

    def __init__(self, key_pages: torch.Tensor, value_pages: torch.Tensor) -> None:
        self.key_pages, self.value_pages = key_pages, value_pages

    physical_blocks = property(lambda s: s.key_pages.shape[0])
    kv_heads = property(lambda s: s.key_pages.shape[1])
    block_size = property(lambda s: s.key_pages.shape[2])
    head_width = property(lambda s: s.key_pages.shape[3])


class CheckerOps:
    def __init__(self, group=None) -> None:
        self.group = group
        self.world = 1 if group is None else torch.distributed.get_world_size(group)
        self.oracle = port()
        self.launches = 0

    def empty(self, shape, dtype=torch.float32):
        return torch.zeros(shape, dtype=dtype)

    def linear(self, x, w: Nf4Weight, out) -> None:
        out.copy_(torch.from_numpy(self.oracle.linear_forward(w, x.numpy(), threads=1)))

    def linear_multi(self, x, weights, outs) -> None:
        for w, out in zip(weights, outs):
            self.linear(x, w, out)

    def rmsnorm(self, x, delta, x_out, scale, y, eps) -> None:
        if delta is not None:
            x_out.copy_(x + delta)
            x = x_out
        y.copy_(torch.from_numpy(rms_norm(x.numpy(), scale.numpy(), eps)))

    def rope_append(self, q, k, v, positions, tables, pool, theta, status) -> None:
        bs = pool.block_size
        for s in range(q.shape[0]):
            pos = int(positions[s])
            q[s] = torch.from_numpy(rotate(q[s].numpy(), pos, theta))
            page = int(tables[s, pos // bs])
            pool.key_pages[page, :, pos % bs] = torch.from_numpy(rotate(k[s].numpy(), pos, theta))
            pool.value_pages[page, :, pos % bs] = v[s]

    def attention(self, q, pool, tables, seq_lens, ctx, max_seq_len, status, workspace) -> None:
        out = self.oracle.paged_decode_gqa(q.numpy(), pool.key_pages.numpy(), pool.value_pages.numpy(),
                                           tables.numpy().astype(np.uint32), seq_lens.numpy().astype(np.uint32),
                                           threads=1)
        ctx.copy_(torch.from_numpy(out))

    def attention_workspace(self, *args):
        return None

    def silu_mul(self, gate, up, out) -> None:
        out.copy_(torch.from_numpy(port().silu_mul(gate.numpy(), up.numpy())))

    def gather_rows(self, table, ids, out, status) -> None:
        out.copy_(table[ids.long()])

    def argmax(self, logits, out) -> None:
        rows = logits.numpy()
        out.copy_(torch.tensor([port().greedy(r) for r in rows], dtype=torch.int32))

    def all_gather_columns(self, local, gathered, full) -> None:
        torch.distributed.all_gather_into_tensor(gathered.view(-1, local.shape[1]), local.contiguous(), group=self.group)
        full.view(local.shape[0], self.world, local.shape[1]).copy_(gathered.permute(1, 0, 2))
