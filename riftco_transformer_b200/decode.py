"""One decode step of a Llama-shaped decoder assembled from the hot-path
operators: packed-NF4 linears, RMSNorm, split-half RoPE + KV-page append, paged
grouped-query attention, SwiGLU, greedy argmax.

The reference has no incremental decode for its Llama/Mistral model
(include/riftco_transformer/model/llama_mistral_transformer.hpp:77-79); the
step below strings together the reference's primitives in the order of its
full-sequence forward (src/model/llama_mistral_transformer.cpp) and of
DecoderOnlyTransformer::decode_token (src/model/decoder_only_transformer.cpp:368-460):
per layer  x += Wo·attn(rope(Wq·n1), rope(Wk·n1), Wv·n1),  x += Wdown·(silu(Wgate·n2) * Wup·n2)
with n = RMSNorm(x); bias-free linears; final RMSNorm and LM head.

Multi-GPU (one process per GPU): every linear is sharded by output rows, the
attention by KV head; ranks exchange activations with an all-gather at the four
layer boundaries where the next operator needs the full width. There is no
reduction: no linear is split along its contraction.

The step is written against a small `ops` interface so that the same
orchestration (sharding arithmetic, buffer flow, gathers) is exercised by CPU
tests with a checker backend; the product backend is `CudaOps`, which calls the
C ABI and has no CPU fallback.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import lib
from .backend import PackedNf4Weight, PagedKvPool, _check, _stream_ptr


@dataclass
class DecoderConfig:
    layers: int = 32
    d_model: int = 4096
    q_heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 32000
    eps: float = 1e-5
    theta: float = 1e4
    block_size: int = 16

    def shard_check(self, world: int) -> None:
        for name, v in (("q_heads", self.q_heads), ("kv_heads", self.kv_heads), ("d_model", self.d_model),
                        ("ffn", self.ffn), ("vocab", self.vocab)):
            if v % world != 0:
                raise ValueError(f"{name}={v} does not divide over {world} ranks")


LAYER_WEIGHTS = ("wq", "wk", "wv", "wo", "w_gate", "w_up", "w_down")


def weight_shapes(cfg: DecoderConfig) -> dict[str, tuple[int, int]]:
    """(out, in) of every linear of one layer, plus the LM head."""
    d, hd = cfg.d_model, cfg.head_dim
    return {
        "wq": (cfg.q_heads * hd, d), "wk": (cfg.kv_heads * hd, d), "wv": (cfg.kv_heads * hd, d),
        "wo": (d, cfg.q_heads * hd), "w_gate": (cfg.ffn, d), "w_up": (cfg.ffn, d), "w_down": (d, cfg.ffn),
        "lm_head": (cfg.vocab, d),
    }


class CudaOps:
    """Product backend: torch tensors for memory, the C ABI for arithmetic.

    With more than one rank the activations are joined by the library's own
    peer-store all-gather kernel: the gathered buffers live in symmetric memory
    (torch.distributed._symmetric_memory exchanges the peer mappings, nothing
    else), every rank stores its shard straight into every rank's buffer over
    NVLink and waits, with a time limit, for the others. ``B2_PEER_GATHER=0``
    selects the NCCL all-gather (plus a layout copy) instead."""

    def __init__(self, device, group=None) -> None:
        self.device = device
        self.group = group
        self.world = 1 if group is None else torch.distributed.get_world_size(group)
        self.rank = 0 if group is None else torch.distributed.get_rank(group)
        self.launches = 0
        self.peer = (self.world > 1 and torch.device(device).type == "cuda"
                     and os.environ.get("B2_PEER_GATHER", "1") != "0")
        self._peer_ptrs: dict = {}
        if self.peer:
            import torch.distributed._symmetric_memory as symm
            self._symm = symm
            # flag array (one slot per rank), local epoch / CTA counter, status word
            self._flags = symm.empty((64,), dtype=torch.int32, device=self.device)
            self._flags.zero_()
            handle = symm.rendezvous(self._flags, self.group)
            self._flag_handle = handle
            self._flag_ptrs = torch.tensor([int(p) for p in handle.buffer_ptrs], dtype=torch.int64,
                                           device=self.device)
            self._peer_state = torch.zeros((2,), dtype=torch.int32, device=self.device)
            self.peer_status = torch.zeros((1,), dtype=torch.int32, device=self.device)
            torch.cuda.synchronize(self.device)
            torch.distributed.barrier(group=self.group)

    def empty(self, shape, dtype=torch.float32):
        return torch.empty(shape, dtype=dtype, device=self.device)

    def _peer_mapped(self, shape, dtype):
        t = self._symm.empty(tuple(shape), dtype=dtype, device=self.device)
        handle = self._symm.rendezvous(t, self.group)
        ptrs = torch.tensor([int(p) for p in handle.buffer_ptrs], dtype=torch.int64, device=self.device)
        return t, handle, ptrs

    def gathered_buffer(self, shape, with_bf16: bool = False):
        """Buffer that receives an all-gather: peer-mapped when the peer-store gather is in use.
        With `with_bf16` the gather also fills a bf16 copy of it (`bf16_of`), which every rank must
        then ask for alike."""
        if not self.peer:
            return self.empty(shape)
        t, handle, ptrs = self._peer_mapped(shape, torch.float32)
        t16 = h16 = p16 = None
        if with_bf16:
            t16, h16, p16 = self._peer_mapped(shape, torch.bfloat16)
        self._peer_ptrs[t.data_ptr()] = (handle, ptrs, t16, h16, p16)
        return t

    def bf16_of(self, full):
        """The bf16 copy the peer gather keeps of `full`, or None."""
        entry = self._peer_ptrs.get(full.data_ptr()) if self.peer else None
        return None if entry is None else entry[2]

    def check_peer_status(self) -> None:
        """Raises if a peer-store gather gave up waiting for another rank."""
        if self.peer and int(self.peer_status.item()) != 0:
            raise RuntimeError("peer all-gather timed out waiting for another rank "
                               f"(status {int(self.peer_status.item())})")

    def linear(self, x, w: PackedNf4Weight, out) -> None:
        ws = w.struct()
        _check(lib.b2_nf4_linear_forward(C.byref(ws), x.data_ptr(), out.data_ptr(), x.shape[0], None, 0,
                                         _stream_ptr(None)))
        self.launches += 2 if x.shape[0] > 16 else 1   # above 16 rows: conversion pre-pass + tensor-core kernel

    def linear_multi(self, x, weights, outs) -> None:
        """Several packed linears of the same input (q / k / v, gate / up): one call, and above
        16 rows one conversion and one kernel launch for all of them."""
        n = len(weights)
        structs = (_lib.Nf4WeightStruct * n)(*[w.struct() for w in weights])
        ptrs = (C.c_void_p * n)(*[o.data_ptr() for o in outs])
        _check(lib.b2_nf4_linear_forward_multi(structs, n, x.data_ptr(), ptrs, x.shape[0], None, 0,
                                               _stream_ptr(None)))
        self.launches += 2 if (x.shape[0] > 16 and n <= 4) else n

    def linear_bf16_supported(self, weights, rows: int) -> bool:
        """True when `linear_multi_bf16` takes these weights at this row count."""
        n = len(weights)
        structs = (_lib.Nf4WeightStruct * n)(*[w.struct() for w in weights])
        return bool(lib.b2_nf4_linear_bf16_supported(structs, n, rows))

    def linear_multi_bf16(self, x16, weights, outs) -> None:
        """`linear_multi` on activations already held as bf16 (written by `rmsnorm` / `silu_mul`
        next to their FP32 result): one kernel launch, no conversion pass."""
        n = len(weights)
        structs = (_lib.Nf4WeightStruct * n)(*[w.struct() for w in weights])
        ptrs = (C.c_void_p * n)(*[o.data_ptr() for o in outs])
        _check(lib.b2_nf4_linear_forward_multi_bf16(structs, n, x16.data_ptr(), ptrs, x16.shape[0],
                                                    _stream_ptr(None)))
        self.launches += 1

    def rmsnorm(self, x, delta, x_out, scale, y, eps: float, y16=None) -> None:
        _check(lib.b2_rmsnorm_bf16(x.data_ptr(), None if delta is None else delta.data_ptr(),
                                   None if x_out is None else x_out.data_ptr(), scale.data_ptr(), y.data_ptr(),
                                   None if y16 is None else y16.data_ptr(), x.shape[0], x.shape[1], eps,
                                   _stream_ptr(None)))
        self.launches += 1

    def rope_append(self, q, k, v, positions, tables, pool: PagedKvPool, theta: float, status) -> None:
        n_seq, q_heads, d = q.shape
        _check(lib.b2_rope_append_kv(q.data_ptr(), k.data_ptr(), v.data_ptr(), positions.data_ptr(),
                                     tables.data_ptr(), pool.key_pages.data_ptr(), pool.value_pages.data_ptr(),
                                     n_seq, q_heads, k.shape[1], d, pool.block_size, pool.physical_blocks,
                                     tables.shape[1], theta, status.data_ptr(), _stream_ptr(None)))
        self.launches += 1

    attention_writes_bf16 = True   # `attention` takes `ctx16`: a bf16 copy of the context for the o-projection

    def attention(self, q, pool: PagedKvPool, tables, seq_lens, ctx, max_seq_len: int, status, workspace,
                  ctx16=None) -> None:
        n_seq, q_heads, d = q.shape
        ws = None if workspace is None else workspace.data_ptr()
        ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
        if ctx16 is None:
            _check(lib.b2_paged_decode_attention(
                q.data_ptr(), pool.key_pages.data_ptr(), pool.value_pages.data_ptr(), tables.data_ptr(),
                seq_lens.data_ptr(), ctx.data_ptr(), n_seq, q_heads, pool.kv_heads, d, pool.block_size,
                pool.physical_blocks, tables.shape[1], max_seq_len, ws, ws_bytes, status.data_ptr(),
                _stream_ptr(None)))
        else:
            _check(lib.b2_paged_decode_attention_bf16(
                q.data_ptr(), pool.key_pages.data_ptr(), pool.value_pages.data_ptr(), tables.data_ptr(),
                seq_lens.data_ptr(), ctx.data_ptr(), ctx16.data_ptr(), n_seq, q_heads, pool.kv_heads, d,
                pool.block_size, pool.physical_blocks, tables.shape[1], max_seq_len, ws, ws_bytes,
                status.data_ptr(), _stream_ptr(None)))
        self.launches += 2 if max_seq_len > 256 else 1

    def attention_workspace(self, n_seq, q_heads, d, block_size, max_seq_len):
        need = lib.b2_paged_decode_workspace_bytes(n_seq, q_heads, d, block_size, max_seq_len)
        return torch.empty(max(need, 16), dtype=torch.uint8, device=self.device)

    def silu_mul(self, gate, up, out, out16=None) -> None:
        _check(lib.b2_silu_mul_bf16(gate.data_ptr(), up.data_ptr(), out.data_ptr(),
                                    None if out16 is None else out16.data_ptr(), out.numel(), _stream_ptr(None)))
        self.launches += 1

    def gather_rows(self, table, ids, out, status) -> None:
        _check(lib.b2_gather_rows(table.data_ptr(), ids.data_ptr(), out.data_ptr(), out.shape[0], out.shape[1],
                                  table.shape[0], status.data_ptr(), _stream_ptr(None)))
        self.launches += 1

    def argmax(self, logits, out) -> None:
        _check(lib.b2_argmax(logits.data_ptr(), out.data_ptr(), logits.shape[0], logits.shape[1],
                             _stream_ptr(None)))
        self.launches += 1

    def all_gather_columns(self, local, gathered, full) -> None:
        """local [B, n] on every rank -> full [B, world*n] (rank r's columns at
        r*n). `gathered` is a [world, B, n] staging buffer."""
        if self.world == 1:
            raise RuntimeError("all_gather_columns is only used with more than one rank")
        if self.peer:
            entry = self._peer_ptrs.get(full.data_ptr())
            if entry is None:
                raise RuntimeError("peer all-gather target was not allocated with gathered_buffer()")
            _check(lib.b2_peer_all_gather_columns_bf16(
                local.data_ptr(), local.shape[0], local.shape[1], entry[1].data_ptr(),
                None if entry[4] is None else entry[4].data_ptr(), self._flag_ptrs.data_ptr(), self.rank,
                self.world, self._peer_state.data_ptr(), self.peer_status.data_ptr(), _stream_ptr(None)))
            self.launches += 1
            return
        torch.distributed.all_gather_into_tensor(gathered.view(-1, local.shape[1]), local, group=self.group)
        full.view(local.shape[0], self.world, local.shape[1]).copy_(gathered.permute(1, 0, 2))


class DecodeStep:
    """Holds one rank's weight shards, KV pools and activation buffers and runs
    decode steps for a fixed batch."""

    def __init__(self, cfg: DecoderConfig, ops, weights: dict, norms: dict, embedding, pools: list,
                 tables, batch: int, max_seq_len: int, rank: int = 0, world: int = 1) -> None:
        cfg.shard_check(world)
        self.cfg, self.ops, self.rank, self.world = cfg, ops, rank, world
        self.w, self.norms, self.embedding, self.pools, self.tables = weights, norms, embedding, pools, tables
        self.batch, self.max_seq_len = batch, max_seq_len
        self.active_layers = cfg.layers   # a step may be cut short after this many layers (cross-checks)
        d, hd = cfg.d_model, cfg.head_dim
        self.hq, self.hkv = cfg.q_heads // world, cfg.kv_heads // world
        e = ops.empty
        g = getattr(ops, "gathered_buffer", ops.empty)   # peer-mapped where the backend gathers by peer stores
        B = batch
        # Where the backend's tensor-core linears read bf16 activations, the kernel that produces an
        # activation (RMSNorm, SiLU*up, the peer gather) also writes its bf16 copy and the linear skips
        # its own conversion pass. Values are the same either way: the pass rounds the same FP32
        # numbers the same way.
        takes_bf16 = getattr(ops, "linear_bf16_supported", None)
        if takes_bf16 is None or os.environ.get("B2_BF16_HANDOFF", "1") == "0":
            takes_bf16 = lambda ws, rows: False   # noqa: E731
        w0 = weights[0]
        gather_bf16 = getattr(ops, "bf16_of", None) is not None

        def gathered(shape, consumer):
            if gather_bf16 and takes_bf16([consumer], B):
                return g(shape, True)
            return g(shape)
        self.x = e((B, d))
        self.n = e((B, d))
        self.q = e((B, self.hq, hd))
        self.k = e((B, self.hkv, hd))
        self.v = e((B, self.hkv, hd))
        self.ctx_local = e((B, self.hq, hd))
        self.ctx = gathered((B, cfg.q_heads * hd), w0["wo"]) if world > 1 else None
        # The o- and down-projections may be given whole to every rank instead of row-sharded: their
        # inputs are gathered anyway, a [B, d] output is small, and computing it everywhere costs less
        # than a cross-GPU handshake (two gathers per layer instead of four).
        self.whole_o = world > 1 and weights[0]["wo"].out_features == d
        self.whole_down = world > 1 and weights[0]["w_down"].out_features == d
        self.o_local = e((B, d // world))
        self.o = (e((B, d)) if self.whole_o else g((B, d))) if world > 1 else None
        self.gate = e((B, cfg.ffn // world))
        self.up = e((B, cfg.ffn // world))
        self.h_local = e((B, cfg.ffn // world))
        self.h = gathered((B, cfg.ffn), w0["w_down"]) if world > 1 else None
        self.down_local = e((B, d // world))
        self.down = (e((B, d)) if self.whole_down else g((B, d))) if world > 1 else None
        self.logits_local = e((B, cfg.vocab // world))
        self.logits = g((B, cfg.vocab)) if world > 1 else None
        self.next_tokens = e((B,), dtype=torch.int32)
        self.status = ops.empty((1,), dtype=torch.int32)
        self.status.zero_()   # sticky error bits of the attention / append / gather kernels
        self.workspace = ops.attention_workspace(B, self.hq, hd, cfg.block_size, max_seq_len)
        if world > 1:
            widths = {cfg.q_heads * hd // world, d // world, cfg.ffn // world, cfg.vocab // world}
            self.stage = {n_: e((world, B, n_)) for n_ in widths}
        self.n16 = self.h16 = self.ctx16 = self.hfull16 = None
        if (takes_bf16([w0["wq"], w0["wk"], w0["wv"]], B) and takes_bf16([w0["w_gate"], w0["w_up"]], B)
                and takes_bf16([weights["lm_head"]], B)):
            self.n16 = e((B, d), dtype=torch.bfloat16)
        if world == 1 and takes_bf16([w0["w_down"]], B):
            self.h16 = e((B, cfg.ffn), dtype=torch.bfloat16)
        if world > 1 and gather_bf16:
            self.ctx16, self.hfull16 = ops.bf16_of(self.ctx), ops.bf16_of(self.h)
        # one rank: attention writes the bf16 copy of its context that the o-projection reads
        self.attn16 = None
        if world == 1 and getattr(ops, "attention_writes_bf16", False) and takes_bf16([w0["wo"]], B):
            self.attn16 = e((B, self.hq * hd), dtype=torch.bfloat16)
            self.ctx16 = self.attn16

    def _gather(self, local, full):
        if self.world == 1:
            return local.view(local.shape[0], -1)
        flat = local.view(local.shape[0], -1)
        self.ops.all_gather_columns(flat, self.stage[flat.shape[1]], full)
        return full

    def _norm(self, delta, scale) -> None:
        """x += delta (when given), n = rmsnorm(x) * scale, plus n's bf16 copy where it is used."""
        if self.n16 is not None:
            self.ops.rmsnorm(self.x, delta, self.x, scale, self.n, self.cfg.eps, self.n16)
        else:
            self.ops.rmsnorm(self.x, delta, self.x, scale, self.n, self.cfg.eps)

    def _linears_of_n(self, weights, outs) -> None:
        if self.n16 is not None:
            self.ops.linear_multi_bf16(self.n16, weights, outs)
        elif len(weights) == 1:
            self.ops.linear(self.n, weights[0], outs[0])
        else:
            self.ops.linear_multi(self.n, weights, outs)

    def _linear(self, x, x16, w, out) -> None:
        if x16 is not None:
            self.ops.linear_multi_bf16(x16, [w], [out])
        else:
            self.ops.linear(x, w, out)

    def step(self, tokens, positions, seq_lens):
        """tokens int32 [B]; positions uint32/int32 [B] = index of the new token;
        seq_lens = positions + 1. Returns (next_tokens [B], logits [B, vocab]).
        With B2_NVTX=1 every layer is an NVTX range (for timeline tools; off by default)."""
        cfg, ops = self.cfg, self.ops
        nvtx = os.environ.get("B2_NVTX", "0") == "1"
        ops.gather_rows(self.embedding, tokens, self.x, self.status)
        pending = None  # residual delta not yet added to x
        for layer in range(self.active_layers):
            if nvtx:
                if layer > 0:
                    torch.cuda.nvtx.range_pop()
                torch.cuda.nvtx.range_push(f"decode layer {layer}")
            w, nm = self.w[layer], self.norms[layer]
            self._norm(pending, nm["attn"])
            self._linears_of_n([w["wq"], w["wk"], w["wv"]],
                               [self.q.view(self.batch, -1), self.k.view(self.batch, -1),
                                self.v.view(self.batch, -1)])
            ops.rope_append(self.q, self.k, self.v, positions, self.tables, self.pools[layer], cfg.theta,
                            self.status)
            if self.attn16 is not None:
                ops.attention(self.q, self.pools[layer], self.tables, seq_lens, self.ctx_local, self.max_seq_len,
                              self.status, self.workspace, ctx16=self.attn16)
            else:
                ops.attention(self.q, self.pools[layer], self.tables, seq_lens, self.ctx_local, self.max_seq_len,
                              self.status, self.workspace)
            ctx = self._gather(self.ctx_local, self.ctx)
            if self.whole_o:
                self._linear(ctx, self.ctx16, w["wo"], self.o)
                o = self.o
            else:
                self._linear(ctx, self.ctx16, w["wo"], self.o_local)
                o = self._gather(self.o_local, self.o)
            self._norm(o, nm["ffn"])
            self._linears_of_n([w["w_gate"], w["w_up"]], [self.gate, self.up])
            if self.h16 is not None:   # one rank: the down-projection reads the bf16 copy directly
                ops.silu_mul(self.gate, self.up, self.h_local, self.h16)
                ops.linear_multi_bf16(self.h16, [w["w_down"]], [self.down_local])
                pending = self.down_local
                continue
            ops.silu_mul(self.gate, self.up, self.h_local)
            h = self._gather(self.h_local, self.h)
            if self.whole_down:
                self._linear(h, self.hfull16, w["w_down"], self.down)
                pending = self.down
            else:
                self._linear(h, self.hfull16, w["w_down"], self.down_local)
                pending = self._gather(self.down_local, self.down)
        if nvtx and self.active_layers > 0:
            torch.cuda.nvtx.range_pop()
        self._norm(pending, self.norms["final"])
        self._linears_of_n([self.w["lm_head"]], [self.logits_local])
        logits = self._gather(self.logits_local, self.logits)
        ops.argmax(logits, self.next_tokens)
        return self.next_tokens, logits

    # ---- accounting ---------------------------------------------------------------
    def weight_bytes(self) -> int:
        total = 0
        for layer in range(self.cfg.layers):
            total += sum(self.w[layer][k].resident_payload_bytes() for k in LAYER_WEIGHTS)
        return total + self.w["lm_head"].resident_payload_bytes()


WHOLE_ON_EVERY_RANK = ("wo", "w_down")   # see DecodeStep: replicated rather than row-sharded


def synthetic_step(cfg: DecoderConfig, batch: int, context: int, rank: int = 0, world: int = 1, device="cuda",
                   group=None, seed: int = 1234, whole=None, quantized: bool = True) -> tuple[DecodeStep, dict]:
    """A DecodeStep over a seeded synthetic model for benchmarking and cross-checks.

    Every rank builds the SAME global model from the seed - weights ~ N(0, 0.02^2) quantised to NF4
    (block 64, double-quantised scales) by synth.quantized_weight - and takes its row shards as
    views of the global payload (PackedNf4Weight.row_shard: no re-quantisation, the parent's
    second-level scale groups, flat_block_base != 0). KV pools ~ N(0,1) hold `context` tokens per
    sequence and are seeded per (layer, global KV head), so the heads a rank owns carry the same
    values whatever the world size; block tables are one permutation shared by all layers. The
    step's logits are therefore the same function of the seed at every world size, up to the order
    of FP32 partial sums inside the linears.

    `whole`: names of the layer weights every rank keeps whole (default: WHOLE_ON_EVERY_RANK when
    world > 1). `quantized=False` draws the payloads directly in the packed domain (cheaper)."""
    from . import synth
    cfg.shard_check(world)
    if whole is None:
        whole = WHOLE_ON_EVERY_RANK if world > 1 else ()
    ops = CudaOps(device, group)
    shapes = weight_shapes(cfg)
    make = synth.quantized_weight if quantized else synth.packed_weight

    def shard(name, w):
        return w if (world == 1 or name in whole) else w.row_shard(rank, world)

    weights: dict = {}
    for layer in range(cfg.layers):
        weights[layer] = {}
        for i, name in enumerate(LAYER_WEIGHTS):
            out_f, in_f = shapes[name]
            weights[layer][name] = shard(name, make(out_f, in_f, device=device, seed=seed + 1000 * layer + 10 * i))
    out_f, in_f = shapes["lm_head"]
    weights["lm_head"] = shard("lm_head", make(out_f, in_f, device=device, seed=seed + 999983))
    g = torch.Generator(device=device)
    g.manual_seed(seed + 7)
    norms = {layer: {"attn": 1.0 + 0.1 * torch.randn(cfg.d_model, device=device, generator=g),
                     "ffn": 1.0 + 0.1 * torch.randn(cfg.d_model, device=device, generator=g)}
             for layer in range(cfg.layers)}
    norms["final"] = 1.0 + 0.1 * torch.randn(cfg.d_model, device=device, generator=g)
    embedding = 0.02 * torch.randn((cfg.vocab, cfg.d_model), device=device, generator=g)
    # One spare slot per sequence for the token this step appends.
    lens = [context + 1] * batch
    blocks = -(-(context + 1) // cfg.block_size)
    total = blocks * batch
    perm = torch.randperm(total, device=device, generator=g).to(torch.int32)
    tables = perm.view(batch, blocks).contiguous()
    tokens = torch.randint(0, cfg.vocab, (batch,), device=device, generator=g, dtype=torch.int32)
    pools = []
    hkv = cfg.kv_heads // world
    for layer in range(cfg.layers):
        pages = []
        for which in range(2):   # K, V
            pool = torch.empty((total, hkv, cfg.block_size, cfg.head_dim), device=device)
            for j in range(hkv):
                head = rank * hkv + j
                g.manual_seed(seed + 104729 * (layer + 1) + 31 * head + which)
                pool[:, j] = torch.randn((total, cfg.block_size, cfg.head_dim), device=device, generator=g)
            pages.append(pool)
        pools.append(PagedKvPool(pages[0], pages[1]))
    step = DecodeStep(cfg, ops, weights, norms, embedding, pools, tables, batch, context + 1, rank, world)
    inputs = {
        "tokens": tokens,
        "positions": torch.full((batch,), context, dtype=torch.int32, device=device),
        "seq_lens": torch.full((batch,), context + 1, dtype=torch.int32, device=device),
        "kv_bytes_per_step": cfg.layers * batch * (context + 1) * hkv * cfg.head_dim * 4 * 2,
        "lens": lens,
    }
    return step, inputs
