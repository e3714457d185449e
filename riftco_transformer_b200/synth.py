"""Seeded synthetic inputs for benchmarks and smoke runs, generated on the
device with torch (no dataset, no checkpoint).

Packed weights are drawn directly in the packed domain with the value
distributions that quantising N(0, 0.02^2) weights in 64-element blocks
produces: NF4 is built so that its 16 codes are (nearly) equally likely for
normal data, and the block absmax of 64 such values concentrates near
0.02 * 2.4. The double-quantised scale encoding is then derived from those
scales with the reference's formulas
(src/core/quantization/quantized_weight.cpp:209-254) evaluated with torch.
"""
from __future__ import annotations

import torch

from . import _lib
from .backend import PackedNf4Weight, PagedKvPool


def packed_weight(out_features: int, in_features: int, *, double_quantized: bool = True, block_size: int = 64,
                  scale_block_size: int = 256, seed: int = 1234, device="cuda") -> PackedNf4Weight:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    n = out_features * in_features
    blocks = -(-n // block_size)
    codes = torch.randint(0, 256, ((n + 1) // 2,), dtype=torch.uint8, device=device, generator=g)
    if n % 2:
        codes[-1] &= 0x0F
    # absmax of 64 draws of N(0, 0.02^2): mean ~0.0479, sd ~0.0066
    scales = (0.0479 + 0.0066 * torch.randn(blocks, device=device, generator=g)).clamp_min(0.02).float()
    if not double_quantized:
        return PackedNf4Weight(codes, scales, None, _lib.SCALES_FLOAT32, block_size, 0, 0.0,
                               out_features, in_features)
    mu = (scales.double().sum() / blocks).float()
    groups = -(-blocks // scale_block_size)
    pad = groups * scale_block_size - blocks
    centered = scales - mu
    padded = torch.cat([centered, torch.zeros(pad, device=device)]) if pad else centered
    second = padded.view(groups, scale_block_size).abs().amax(dim=1)
    denom = second.repeat_interleave(scale_block_size)[:blocks]
    scaled = torch.where(denom > 0, centered / denom, torch.zeros_like(centered)) * 127.0
    rounded = torch.where(scaled >= 0, torch.floor(scaled + 0.5), torch.ceil(scaled - 0.5)).clamp(-127, 127)
    scale_codes = (rounded.to(torch.int32) + 128).to(torch.uint8)
    return PackedNf4Weight(codes, scale_codes, second.float().contiguous(), _lib.SCALES_DOUBLE_QUANTIZED_UINT8,
                           block_size, scale_block_size, float(mu.item()), out_features, in_features)


def host_payload(weight: PackedNf4Weight):
    """Copies a device weight back into the canonical host payload fields (for
    the CPU baseline, which consumes the same bytes)."""
    import types
    p = types.SimpleNamespace(
        codes=weight.codes.cpu().numpy(), out_features=weight.out_features, in_features=weight.in_features,
        block_size=weight.block_size, fp32_scales=None, scale_codes=None, second_level=None,
        scale_block_size=weight.scale_block_size, offset=weight.offset)
    if weight.encoding == _lib.SCALES_FLOAT32:
        p.fp32_scales = weight.primary.cpu().numpy()
    else:
        p.scale_codes = weight.primary.cpu().numpy()
        p.second_level = weight.secondary.cpu().numpy()
    return p


def paged_cache(seq_lens, kv_heads: int, head_width: int = 128, block_size: int = 16, *, seed: int = 91011,
                slack_blocks: int = 0, device="cuda"):
    """K/V pools ~ N(0,1) with one randomly permuted block table per sequence.
    Returns (PagedKvPool, block_tables int32 [n_seq, max_blocks], seq_lens int32)."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    lens = torch.as_tensor(seq_lens, dtype=torch.int64)
    blocks = (lens + block_size - 1) // block_size
    total = int(blocks.sum()) + slack_blocks
    perm = torch.randperm(total, device=device, generator=g).to(torch.int32)
    tables = torch.zeros((len(lens), int(blocks.max())), dtype=torch.int32, device=device)
    at = 0
    for s, nb in enumerate(blocks.tolist()):
        tables[s, :nb] = perm[at:at + nb]
        at += nb
    shape = (total, kv_heads, block_size, head_width)
    k = torch.randn(shape, device=device, generator=g)
    v = torch.randn(shape, device=device, generator=g)
    return PagedKvPool(k, v), tables, lens.to(torch.int32).to(device)
