"""Seeded synthetic inputs for benchmarks and smoke runs, generated on the
device with torch (no dataset, no checkpoint).

``quantized_weight`` draws FP32 weights ~ N(0, sigma^2) and quantises them with
the reference's encoder restated in torch (absmax per block, nearest code with
ties to the lower index, zero blocks -> scale 0 / code 7: pack_nf4,
src/core/quantization/quantized_weight.cpp:176-207 and nf4.cpp:55-68; double
quantisation of the block scales: quantized_weight.cpp:209-254), so benchmark
payloads are those of a quantised model. tests/test_gpu_parity.py holds it to
the CPU oracle bit for bit. ``packed_weight`` draws the payload directly in the
packed domain instead (uniform codes, scales with the distribution the block
absmax of N(0, 0.02^2) weights has); it is cheaper and serves launches whose
arithmetic result is not looked at.
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
    scale_codes, second, mu = double_quantize(scales, scale_block_size)
    return PackedNf4Weight(codes, scale_codes, second, _lib.SCALES_DOUBLE_QUANTIZED_UINT8,
                           block_size, scale_block_size, mu, out_features, in_features)


_CODEBOOK = (-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
             -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
             0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
             0.7229568362236023, 1.0)


def double_quantize(scales: torch.Tensor, scale_block_size: int):
    """double_quantize_scales of the reference on a device tensor: (scale codes u8, second-level f32, offset)."""
    blocks = scales.numel()
    mu = (scales.double().sum() / blocks).float()
    groups = -(-blocks // scale_block_size)
    pad = groups * scale_block_size - blocks
    centered = scales - mu
    padded = torch.cat([centered, torch.zeros(pad, device=scales.device)]) if pad else centered
    second = padded.view(groups, scale_block_size).abs().amax(dim=1)
    denom = second.repeat_interleave(scale_block_size)[:blocks]
    scaled = torch.where(denom > 0, centered / denom, torch.zeros_like(centered)) * 127.0
    rounded = torch.where(scaled >= 0, torch.floor(scaled + 0.5), torch.ceil(scaled - 0.5)).clamp(-127, 127)
    scale_codes = (rounded.to(torch.int32) + 128).to(torch.uint8)
    return scale_codes, second.float().contiguous(), float(mu.item())


def quantize(values: torch.Tensor, *, double_quantized: bool = True, block_size: int = 64,
             scale_block_size: int = 256) -> PackedNf4Weight:
    """The reference's NF4 encoder on a device tensor [out, in] (FP32)."""
    out_features, in_features = values.shape
    n = out_features * in_features
    if n % block_size != 0 or n % 2 != 0:
        raise ValueError("the device encoder takes whole blocks and whole bytes")
    device = values.device
    book = torch.tensor(_CODEBOOK, dtype=torch.float32, device=device)
    flat = values.contiguous().view(-1, block_size)
    scales = flat.abs().amax(dim=1)
    codes = torch.empty(n, dtype=torch.uint8, device=device)
    step = max(1, (1 << 22) // block_size)          # bounds the [rows, block, 16] distance tensor
    for lo in range(0, flat.shape[0], step):
        part, s = flat[lo:lo + step], scales[lo:lo + step]
        normalized = part / torch.where(s > 0, s, torch.ones_like(s)).unsqueeze(1)
        nearest = (normalized.unsqueeze(2) - book).abs().argmin(dim=2)          # first minimum: ties to the lower code
        nearest = torch.where((s > 0).unsqueeze(1), nearest, torch.full_like(nearest, 7))
        codes[lo * block_size:(lo + part.shape[0]) * block_size] = nearest.view(-1).to(torch.uint8)
    packed = (codes[0::2] | (codes[1::2] << 4)).contiguous()
    if not double_quantized:
        return PackedNf4Weight(packed, scales.contiguous(), None, _lib.SCALES_FLOAT32, block_size, 0, 0.0,
                               out_features, in_features)
    scale_codes, second, mu = double_quantize(scales, scale_block_size)
    return PackedNf4Weight(packed, scale_codes, second, _lib.SCALES_DOUBLE_QUANTIZED_UINT8, block_size,
                           scale_block_size, mu, out_features, in_features)


def quantized_weight(out_features: int, in_features: int, *, sigma: float = 0.02, seed: int = 1234,
                     double_quantized: bool = True, block_size: int = 64, scale_block_size: int = 256,
                     device="cuda") -> PackedNf4Weight:
    """W ~ N(0, sigma^2) [out, in], seeded, quantised by `quantize`."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    values = torch.randn((out_features, in_features), device=device, generator=g) * sigma
    return quantize(values, double_quantized=double_quantized, block_size=block_size,
                    scale_block_size=scale_block_size)


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
