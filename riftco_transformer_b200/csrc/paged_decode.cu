// Paged-KV single-token decode attention for a batch of sequences with
// grouped-query heads (query head h reads KV head h / rep).
//
// Pages are consumed in the reference's layout, FP32
// [physical_block, kv_head, block_offset, head_width]
// (src/core/backend/attention/contracts.hpp:88-106), through per-sequence block
// tables; the arithmetic restates
// src/core/backend/attention/reference/paged_decode.cpp:37-132 as an online
// softmax split over the sequence (split-K), so each K/V byte is read from HBM
// exactly once for all `rep` query heads that share it. The kernel is bound by
// that read: 8 * head_width bytes per (token, kv head).
//
// Two paths:
//  * paged_decode_bulk_kernel  - head_width 128, block_size 16, rep in {1,2,4,8}.
//  * paged_decode_generic_*    - any shape (the reference's own test uses
//    head_width 3 and block_size 2), scores spilled to workspace.
// Non-finite scores are reported through a device status word, never by
// trapping: bit 0 a NaN or +inf score, bit 1 all scores of a head -inf, bit 2 a
// block id outside the pool (which is then not dereferenced).
#include "b2_common.cuh"
#include "b2_kernels.h"
#include "sm100_ptx.cuh"

#include <cuda_bf16.h>

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace b2 {
namespace {

constexpr int kD = 128;            // head width of the fast path
constexpr int kPage = 16;          // tokens per page of the fast path
constexpr int kFastWarps = 4;
constexpr int kTokensPerCta = 256; // split size: 16 pages, 4 per warp
constexpr int kPartialStride = kD + 2;  // m, l, acc[128]

// One context value, and its bf16 copy when the caller asked for one.
__device__ __forceinline__ void put_ctx(const PagedDecodeArgs& a, uint64_t index, float value) {
    a.ctx[index] = value;
    if (a.ctx16 != nullptr) static_cast<__nv_bfloat16*>(a.ctx16)[index] = __float2bfloat16_rn(value);
}

// Fast path (head_width 128, block_size 16, rep in {1,2,4,8}). The K and V chunks of a page (8 KB
// each, contiguous in the pool) are brought into shared memory by cp.async.bulk: every warp owns a ring
// of two 8 KB slots and has the next chunk in flight while it works on one. 64 KB per CTA lets three
// CTAs share an SM (192 KB outstanding per SM, none of it in registers); three slots per warp and two
// CTAs per SM hold the same bytes in flight but measured slower (96.9 vs 92.3 us per launch inside the
// decode step, 350 vs 333 us on 64 sequences of 512-8192 tokens): with more CTAs per SM a CTA that
// ends and its successor that starts stall a smaller share of the SM's loads.
// The mbarrier waits are bounded; a timeout sets bit 3 of the status word.
// Grids of at most two waves of the three-slot form (which fits two CTAs per SM) are a question of
// wave count instead: 576 CTAs are 1.95 waves of 296 but 1.3 waves of 444, so such launches take
// the three-slot form when it needs fewer CTA-widths of time (see launch_paged_decode).
constexpr int kChunkBytes = kPage * kD * 4;   // 8 KB: one (page, kv head) of K or of V
constexpr int bulk_smem_bytes(int slots) { return kFastWarps * slots * kChunkBytes; }

__device__ __forceinline__ void bulk_load(uint32_t dst32, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst32), "l"(src), "r"(bytes), "r"(sm100::smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ float4 lds_f4(uint32_t a) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a));
    return v;
}

template <int REP, int kBulkSlots>
__global__ void __launch_bounds__(kFastWarps * 32)
paged_decode_bulk_kernel(const PagedDecodeArgs a, float* __restrict__ partials, uint32_t max_splits) {
    sm100::pdl_launch_dependents();   // a following decode GEMV may start its set-up now
    using namespace sm100;
    const uint32_t split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
    const uint32_t len = __ldg(a.seq_lens + seq);
    const uint32_t n_splits = (len + kTokensPerCta - 1) / kTokensPerCta;
    if (split >= n_splits) return;

    extern __shared__ __align__(1024) uint8_t ring_raw[];
    __shared__ __align__(8) uint64_t bars[kFastWarps][kBulkSlots];
    __shared__ uint32_t s_abort;
    __shared__ __align__(16) float s_p[kFastWarps][kPage][REP];
    __shared__ float s_m[kFastWarps][REP], s_l[kFastWarps][REP];

    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t grp = lane >> 3, sub = lane & 7u;
    const float scale = 1.0f / sqrtf(static_cast<float>(kD));
    const uint32_t ring32 = smem_u32(ring_raw) + warp * (kBulkSlots * kChunkBytes);
    volatile uint32_t* abort = &s_abort;

    if (threadIdx.x == 0) s_abort = 0;
    if (lane == 0) {
        for (int i = 0; i < kBulkSlots; ++i) mbar_init(&bars[warp][i], 1);
        mbar_fence_init();
    }
    __syncthreads();

    float4 q[REP][4];
    const float* qbase = a.q + (static_cast<uint64_t>(seq) * a.q_heads + kvh * REP) * kD;
#pragma unroll
    for (int h = 0; h < REP; ++h)
#pragma unroll
        for (int j = 0; j < 4; ++j)
            q[h][j] = __ldg(reinterpret_cast<const float4*>(qbase + h * kD + 4 * sub + 32 * j));

    float m[REP], l[REP];
    float4 acc[REP];
#pragma unroll
    for (int h = 0; h < REP; ++h) {
        m[h] = -INFINITY;
        l[h] = 0.0f;
        acc[h] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    uint32_t flags = 0;

    const uint32_t tok_begin = split * kTokensPerCta;
    const uint32_t tok_end = min(tok_begin + kTokensPerCta, len);
    const uint32_t page_begin = tok_begin / kPage;
    const uint32_t page_end = (tok_end + kPage - 1) / kPage;
    const uint32_t* table = a.block_tables + static_cast<uint64_t>(seq) * a.max_blocks;
    const uint64_t page_stride = static_cast<uint64_t>(a.kv_heads) * kPage * kD;
    // pages of this warp: page_begin + warp, + kFastWarps, ...
    const uint32_t first = page_begin + warp;
    const uint32_t my_pages = first < page_end ? (page_end - first + kFastWarps - 1) / kFastWarps : 0u;
    const uint32_t units = 2u * my_pages;   // unit 2i = K of page i, 2i + 1 = V of page i

    auto issue_unit = [&](uint32_t u) {   // lane 0 only
        const uint32_t pg = first + (u >> 1) * kFastWarps;
        uint64_t phys = __ldg(table + pg);
        if (phys >= a.physical_blocks) phys = 0;   // flagged where the page is consumed
        const float* src = ((u & 1u) ? a.v_pages : a.k_pages) + phys * page_stride +
                           static_cast<uint64_t>(kvh) * kPage * kD;
        const uint32_t slot = u % kBulkSlots;
        fence_proxy_async_smem();
        mbar_expect_tx(&bars[warp][slot], kChunkBytes);
        bulk_load(ring32 + slot * kChunkBytes, src, kChunkBytes, &bars[warp][slot]);
    };
    if (lane == 0) {
        for (uint32_t u = 0; u < kBulkSlots && u < units; ++u) issue_unit(u);
    }

    for (uint32_t i = 0; i < my_pages; ++i) {
        const uint32_t pg = first + i * kFastWarps;
        if (__ldg(table + pg) >= a.physical_blocks) flags |= B2_ATTN_STATUS_BAD_BLOCK;
        const uint32_t valid = min(static_cast<uint32_t>(kPage), len - pg * kPage);
        const uint32_t uk = 2u * i, uv = uk + 1u;

        // ---- scores from the K slot ----
        mbar_wait(&bars[warp][uk % kBulkSlots], (uk / kBulkSlots) & 1u, abort);
        const uint32_t k32 = ring32 + (uk % kBulkSlots) * kChunkBytes;
        float sc[4][REP];
#pragma unroll
        for (int ps = 0; ps < 4; ++ps) {
            float4 kreg[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) kreg[j] = lds_f4(k32 + ((4 * ps + grp) * kD + 4 * sub + 32 * j) * 4u);
#pragma unroll
            for (int h = 0; h < REP; ++h) {
                float d = 0.0f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    d = fmaf(q[h][j].x, kreg[j].x, d);
                    d = fmaf(q[h][j].y, kreg[j].y, d);
                    d = fmaf(q[h][j].z, kreg[j].z, d);
                    d = fmaf(q[h][j].w, kreg[j].w, d);
                }
                d += __shfl_xor_sync(0xFFFFFFFFu, d, 1);
                d += __shfl_xor_sync(0xFFFFFFFFu, d, 2);
                d += __shfl_xor_sync(0xFFFFFFFFu, d, 4);
                d *= scale;
                const bool in_range = static_cast<uint32_t>(4 * ps + grp) < valid;
                if (in_range && (isnan(d) || d == INFINITY)) flags |= B2_ATTN_STATUS_NAN_OR_POS_INF;
                sc[ps][h] = in_range ? d : -INFINITY;
            }
        }
        __syncwarp();   // every lane has read the K slot: refill it with the unit three ahead
        if (lane == 0 && uk + kBulkSlots < units) issue_unit(uk + kBulkSlots);

        // ---- online softmax update (all lanes keep identical m, l) ----
        float rescale[REP];
#pragma unroll
        for (int h = 0; h < REP; ++h) {
            float pm = fmaxf(fmaxf(sc[0][h], sc[1][h]), fmaxf(sc[2][h], sc[3][h]));
            pm = fmaxf(pm, __shfl_xor_sync(0xFFFFFFFFu, pm, 8));
            pm = fmaxf(pm, __shfl_xor_sync(0xFFFFFFFFu, pm, 16));
            const float m_new = fmaxf(m[h], pm);
            const bool dead = (m_new == -INFINITY) || isnan(m_new);
            rescale[h] = dead ? 1.0f : __expf(m[h] - m_new);
            float ps_sum = 0.0f;
#pragma unroll
            for (int ps = 0; ps < 4; ++ps) {
                const float e = dead ? 0.0f : __expf(sc[ps][h] - m_new);
                sc[ps][h] = e;
                ps_sum += e;
            }
            ps_sum += __shfl_xor_sync(0xFFFFFFFFu, ps_sum, 8);
            ps_sum += __shfl_xor_sync(0xFFFFFFFFu, ps_sum, 16);
            l[h] = l[h] * rescale[h] + ps_sum;
            m[h] = dead ? m[h] : m_new;
        }
        __syncwarp();
        if (sub < REP) {
#pragma unroll
            for (int ps = 0; ps < 4; ++ps) {
                float v = sc[ps][0];
#pragma unroll
                for (int h = 1; h < REP; ++h) v = (sub == static_cast<uint32_t>(h)) ? sc[ps][h] : v;
                s_p[warp][4 * ps + grp][sub] = v;
            }
        }
        __syncwarp();

        // ---- values from the V slot: lane owns dims 4*lane .. 4*lane+3 for every head ----
#pragma unroll
        for (int h = 0; h < REP; ++h) {
            acc[h].x *= rescale[h];
            acc[h].y *= rescale[h];
            acc[h].z *= rescale[h];
            acc[h].w *= rescale[h];
        }
        mbar_wait(&bars[warp][uv % kBulkSlots], (uv / kBulkSlots) & 1u, abort);
        const uint32_t v32 = ring32 + (uv % kBulkSlots) * kChunkBytes;
#pragma unroll 4
        for (uint32_t tk = 0; tk < valid; ++tk) {
            const float4 v = lds_f4(v32 + (tk * kD + 4 * lane) * 4u);
#pragma unroll
            for (int h = 0; h < REP; ++h) {
                const float pr = s_p[warp][tk][h];
                acc[h].x = fmaf(pr, v.x, acc[h].x);
                acc[h].y = fmaf(pr, v.y, acc[h].y);
                acc[h].z = fmaf(pr, v.z, acc[h].z);
                acc[h].w = fmaf(pr, v.w, acc[h].w);
            }
        }
        __syncwarp();
        if (lane == 0 && uv + kBulkSlots < units) issue_unit(uv + kBulkSlots);
    }

    // ---- combine the warps of the CTA (the ring is free now: reuse it for the accumulators) ----
    if (lane == 0 && *abort != 0) flags |= 8u;
    if (flags != 0 && a.status != nullptr) atomicOr(a.status, flags);
    __syncthreads();
    float* s_acc = reinterpret_cast<float*>(ring_raw);   // [warp][REP][kD]
#pragma unroll
    for (int h = 0; h < REP; ++h) {
        if (lane == 0) {
            s_m[warp][h] = m[h];
            s_l[warp][h] = l[h];
        }
        *reinterpret_cast<float4*>(&s_acc[(warp * REP + h) * kD + 4 * lane]) = acc[h];
    }
    __syncthreads();

    const uint32_t c = threadIdx.x;
#pragma unroll
    for (int h = 0; h < REP; ++h) {
        float mm = -INFINITY;
#pragma unroll
        for (int wv = 0; wv < kFastWarps; ++wv) mm = fmaxf(mm, s_m[wv][h]);
        float ll = 0.0f, o = 0.0f;
#pragma unroll
        for (int wv = 0; wv < kFastWarps; ++wv) {
            const float f = (s_m[wv][h] == -INFINITY) ? 0.0f : __expf(s_m[wv][h] - mm);
            ll = fmaf(s_l[wv][h], f, ll);
            o = fmaf(s_acc[(wv * REP + h) * kD + c], f, o);
        }
        const uint64_t head = static_cast<uint64_t>(seq) * a.q_heads + kvh * REP + h;
        if (n_splits == 1) {
            if (mm == -INFINITY) {
                if (c == 0 && a.status != nullptr) atomicOr(a.status, B2_ATTN_STATUS_ALL_NEG_INF);
                put_ctx(a, head * kD + c, 0.0f);
            } else {
                put_ctx(a, head * kD + c, o / ll);
            }
        } else {
            float* dst = partials + (head * max_splits + split) * kPartialStride;
            if (c == 0) {
                dst[0] = mm;
                dst[1] = ll;
            }
            dst[2 + c] = o;
        }
    }
}

// Combines the split partials of every (sequence, query head) that was split.
__global__ void __launch_bounds__(kD)
paged_decode_merge_kernel(const PagedDecodeArgs a, const float* __restrict__ partials,
                          uint32_t max_splits) {
    sm100::pdl_launch_dependents();   // a following decode GEMV may start its set-up now
    const uint32_t h = blockIdx.x, seq = blockIdx.y, c = threadIdx.x;
    const uint32_t len = __ldg(a.seq_lens + seq);
    const uint32_t n_splits = (len + kTokensPerCta - 1) / kTokensPerCta;
    if (n_splits <= 1) return;
    const uint64_t head = static_cast<uint64_t>(seq) * a.q_heads + h;
    const float* src = partials + head * max_splits * kPartialStride;
    // Eight splits at a time with all their loads issued before the first use: a loop that uses
    // each value as it arrives pays one L2 round trip per split.
    float mm = -INFINITY;
    for (uint32_t s0 = 0; s0 < n_splits; s0 += 8u) {
        float m8[8];
#pragma unroll
        for (uint32_t u = 0; u < 8u; ++u) m8[u] = s0 + u < n_splits ? __ldg(src + (s0 + u) * kPartialStride) : -INFINITY;
#pragma unroll
        for (uint32_t u = 0; u < 8u; ++u) mm = fmaxf(mm, m8[u]);
    }
    float ll = 0.0f, o = 0.0f;
    for (uint32_t s0 = 0; s0 < n_splits; s0 += 8u) {
        float m8[8], l8[8], o8[8];
#pragma unroll
        for (uint32_t u = 0; u < 8u; ++u) {
            const bool live = s0 + u < n_splits;
            const float* part = src + (s0 + u) * kPartialStride;
            m8[u] = live ? __ldg(part) : -INFINITY;
            l8[u] = live ? __ldg(part + 1) : 0.0f;
            o8[u] = live ? __ldg(part + 2 + c) : 0.0f;
        }
#pragma unroll
        for (uint32_t u = 0; u < 8u; ++u) {   // split order, as before
            const float f = (m8[u] == -INFINITY) ? 0.0f : __expf(m8[u] - mm);
            ll = fmaf(l8[u], f, ll);
            o = fmaf(o8[u], f, o);
        }
    }
    if (mm == -INFINITY) {
        if (c == 0 && a.status != nullptr) atomicOr(a.status, B2_ATTN_STATUS_ALL_NEG_INF);
        put_ctx(a, head * kD + c, 0.0f);
    } else {
        put_ctx(a, head * kD + c, o / ll);
    }
}

// ---- generic path ----------------------------------------------------------------

// One warp per (sequence, query head); scores live in workspace
// [n_seq, q_heads, max_seq_len]. The normaliser is accumulated in double and
// the context in position order, like the reference loop.
__global__ void __launch_bounds__(128)
paged_decode_generic_kernel(const PagedDecodeArgs a, float* __restrict__ scores) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t task = (static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const uint64_t tasks = static_cast<uint64_t>(a.n_seq) * a.q_heads;
    if (task >= tasks) return;
    const uint32_t seq = static_cast<uint32_t>(task / a.q_heads);
    const uint32_t h = static_cast<uint32_t>(task % a.q_heads);
    const uint32_t kvh = h / (a.q_heads / a.kv_heads);
    const uint32_t len = __ldg(a.seq_lens + seq);
    const uint32_t d = a.head_width, bs = a.block_size;
    const float scale = 1.0f / sqrtf(static_cast<float>(d));
    const float* qv = a.q + task * d;
    const uint32_t* table = a.block_tables + static_cast<uint64_t>(seq) * a.max_blocks;
    float* sc = scores + task * a.max_seq_len;
    uint32_t flags = 0;

    auto page_offset = [&](uint32_t pos, uint32_t& flag_out) -> uint64_t {
        uint64_t phys = __ldg(table + pos / bs);
        if (phys >= a.physical_blocks) {
            flag_out |= B2_ATTN_STATUS_BAD_BLOCK;
            phys = 0;
        }
        return ((phys * a.kv_heads + kvh) * bs + pos % bs) * d;
    };

    float mx = -INFINITY;
    for (uint32_t pos = lane; pos < len; pos += 32) {
        const float* kv = a.k_pages + page_offset(pos, flags);
        float s = 0.0f;
        for (uint32_t c = 0; c < d; ++c) s = __fadd_rn(s, __fmul_rn(__ldg(qv + c), __ldg(kv + c)));
        s *= scale;
        if (isnan(s) || s == INFINITY) flags |= B2_ATTN_STATUS_NAN_OR_POS_INF;
        sc[pos] = s;
        mx = fmaxf(mx, s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        flags |= __shfl_xor_sync(0xFFFFFFFFu, flags, o);
    }
    if (mx == -INFINITY && !(flags & B2_ATTN_STATUS_NAN_OR_POS_INF)) flags |= B2_ATTN_STATUS_ALL_NEG_INF;
    if (flags & (B2_ATTN_STATUS_NAN_OR_POS_INF | B2_ATTN_STATUS_ALL_NEG_INF)) {
        for (uint32_t c = lane; c < d; c += 32) put_ctx(a, task * d + c, 0.0f);
        if (lane == 0 && a.status != nullptr) atomicOr(a.status, flags);
        return;
    }
    double denom = 0.0;
    for (uint32_t pos = lane; pos < len; pos += 32) {
        const double e = exp(static_cast<double>(sc[pos] - mx));
        sc[pos] = static_cast<float>(e);
        denom += e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) denom += __shfl_xor_sync(0xFFFFFFFFu, denom, o);
    __syncwarp();
    for (uint32_t c = lane; c < d; c += 32) {
        float total = 0.0f;
        for (uint32_t pos = 0; pos < len; ++pos) {
            const float pr = static_cast<float>(static_cast<double>(sc[pos]) / denom);
            total = __fadd_rn(total, __fmul_rn(pr, __ldg(a.v_pages + page_offset(pos, flags) + c)));
        }
        put_ctx(a, task * d + c, total);
    }
    if (flags != 0 && lane == 0 && a.status != nullptr) atomicOr(a.status, flags);
}

bool fast_path(const PagedDecodeArgs& a) {
    const uint32_t rep = a.q_heads / a.kv_heads;
    return a.head_width == kD && a.block_size == kPage &&
           (rep == 1 || rep == 2 || rep == 4 || rep == 8) &&
           (reinterpret_cast<uintptr_t>(a.q) & 15u) == 0 &&
           (reinterpret_cast<uintptr_t>(a.k_pages) & 15u) == 0 &&
           (reinterpret_cast<uintptr_t>(a.v_pages) & 15u) == 0 && a.kv_heads <= 65535 &&
           a.n_seq <= 65535;
}

uint32_t splits_for(uint32_t max_seq_len) { return (max_seq_len + kTokensPerCta - 1) / kTokensPerCta; }

}  // namespace

size_t paged_decode_workspace_bytes(uint32_t n_seq, uint32_t q_heads, uint32_t head_width,
                                    uint32_t block_size, uint32_t max_seq_len) {
    const size_t heads = static_cast<size_t>(n_seq) * q_heads;
    if (head_width == kD && block_size == kPage) {
        const uint32_t splits = splits_for(max_seq_len);
        return splits > 1 ? heads * splits * kPartialStride * sizeof(float) : 0;
    }
    return heads * max_seq_len * sizeof(float);
}

int32_t launch_paged_decode(const DeviceContext& ctx, const PagedDecodeArgs& a, void* workspace,
                            size_t workspace_bytes, cudaStream_t stream) {
    const size_t need = paged_decode_workspace_bytes(a.n_seq, a.q_heads, a.head_width, a.block_size,
                                                     a.max_seq_len);
    if (need > workspace_bytes) {
        return fail(B2_STATUS_INVALID_ARGUMENT,
                    "paged decode attention workspace too small: need %zu bytes, got %zu", need,
                    workspace_bytes);
    }
    if (fast_path(a)) {
        const uint32_t splits = splits_for(a.max_seq_len);
        if (splits > 65535) return fail(B2_STATUS_OVERFLOW, "paged decode sequence too long");
        const dim3 grid(splits, a.kv_heads, a.n_seq);
        float* partials = static_cast<float*>(workspace);
        note_route(B2_ROUTE_ATTENTION_BULK);
        static PerDeviceOnce configured;
        B2_TRY(once_per_device(configured, ctx.device, []() -> int32_t {
            B2_CUDA_TRY(cudaFuncSetAttribute(paged_decode_bulk_kernel<1, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, bulk_smem_bytes(2)));
            B2_CUDA_TRY(cudaFuncSetAttribute(paged_decode_bulk_kernel<2, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, bulk_smem_bytes(2)));
            B2_CUDA_TRY(cudaFuncSetAttribute(paged_decode_bulk_kernel<4, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, bulk_smem_bytes(2)));
            B2_CUDA_TRY(cudaFuncSetAttribute(paged_decode_bulk_kernel<8, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, bulk_smem_bytes(2)));
            B2_CUDA_TRY(cudaFuncSetAttribute(paged_decode_bulk_kernel<1, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, bulk_smem_bytes(3)));
            B2_CUDA_TRY(cudaFuncSetAttribute(paged_decode_bulk_kernel<2, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, bulk_smem_bytes(3)));
            B2_CUDA_TRY(cudaFuncSetAttribute(paged_decode_bulk_kernel<4, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, bulk_smem_bytes(3)));
            B2_CUDA_TRY(cudaFuncSetAttribute(paged_decode_bulk_kernel<8, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, bulk_smem_bytes(3)));
            return B2_STATUS_OK;
        }));
        // Two slots per warp (three CTAs per SM) by default; three slots (two CTAs per SM) where the
        // grid is between one and two waves of that form and it needs fewer CTA-widths of time
        // (measured on 32 sequences of 2049 tokens: 2 kv heads 33.8 vs 36.7 us, 1 kv head 19.2 vs 18.4 us).
        const uint64_t ctas = static_cast<uint64_t>(splits) * a.kv_heads * a.n_seq;
        const uint64_t sms = ctx.sm_count > 0 ? static_cast<uint64_t>(ctx.sm_count) : 148u;
        const bool three_slots = ctas > 2 * sms && ctas <= 4 * sms &&
                                 ((ctas + 2 * sms - 1) / (2 * sms)) * 2 < ((ctas + 3 * sms - 1) / (3 * sms)) * 3;
        const uint32_t rep = a.q_heads / a.kv_heads;
        const unsigned threads = kFastWarps * 32;
        if (three_slots) {
            constexpr int kBytes = bulk_smem_bytes(3);
            switch (rep) {
            case 1: paged_decode_bulk_kernel<1, 3><<<grid, threads, kBytes, stream>>>(a, partials, splits); break;
            case 2: paged_decode_bulk_kernel<2, 3><<<grid, threads, kBytes, stream>>>(a, partials, splits); break;
            case 4: paged_decode_bulk_kernel<4, 3><<<grid, threads, kBytes, stream>>>(a, partials, splits); break;
            default: paged_decode_bulk_kernel<8, 3><<<grid, threads, kBytes, stream>>>(a, partials, splits); break;
            }
        } else {
            constexpr int kBytes = bulk_smem_bytes(2);
            switch (rep) {
            case 1: paged_decode_bulk_kernel<1, 2><<<grid, threads, kBytes, stream>>>(a, partials, splits); break;
            case 2: paged_decode_bulk_kernel<2, 2><<<grid, threads, kBytes, stream>>>(a, partials, splits); break;
            case 4: paged_decode_bulk_kernel<4, 2><<<grid, threads, kBytes, stream>>>(a, partials, splits); break;
            default: paged_decode_bulk_kernel<8, 2><<<grid, threads, kBytes, stream>>>(a, partials, splits); break;
            }
        }
        B2_CUDA_TRY(cudaGetLastError());
        if (splits > 1) {
            paged_decode_merge_kernel<<<dim3(a.q_heads, a.n_seq), kD, 0, stream>>>(a, partials, splits);
            B2_CUDA_TRY(cudaGetLastError());
        }
        return B2_STATUS_OK;
    }
    const uint64_t tasks = static_cast<uint64_t>(a.n_seq) * a.q_heads;
    const uint64_t blocks = (tasks + 3) / 4;
    if (blocks > 0x7FFFFFFFull) return fail(B2_STATUS_OVERFLOW, "paged decode batch too large");
    note_route(B2_ROUTE_ATTENTION_GENERIC);
    paged_decode_generic_kernel<<<static_cast<unsigned>(blocks), 128, 0, stream>>>(
        a, static_cast<float*>(workspace));
    B2_CUDA_TRY(cudaGetLastError());
    return B2_STATUS_OK;
}

}  // namespace b2

// ---- entry point that allocates nothing ---------------------------------------------
//
// Some callers may not allocate device memory at the point where they run
// attention: an engine that has handed all of its memory to a pool it manages
// itself, or code running inside a region where cudaMalloc / cudaFree are not
// allowed because they synchronise the device. For them the split-K scratch of
// the decode kernel lives in the fixed-size array below, which every GPU that
// loads this library holds from load until exit.
namespace b2 {
namespace {

constexpr size_t kStaticScratchBytes = B2_NOALLOC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxScratchDevices = 64;
std::mutex g_scratch_mutex;
void* g_scratch_address[kMaxScratchDevices];  // device address of g_static_scratch, per device
bool g_scratch_ready[kMaxScratchDevices];

// In host code `g_static_scratch` names a host-side shadow, not device memory;
// the device address has to be asked for once per device, with that device
// current. Nothing here allocates.
int32_t static_scratch_pointer(void** out, int* device_out) {
    int device = -1;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess || device < 0 || device >= kMaxScratchDevices) {
        cudaGetLastError();
        return fail(B2_STATUS_BACKEND_UNAVAILABLE, "CUDA backend unavailable: %s",
                    err != cudaSuccess ? cudaGetErrorString(err) : "device index out of range");
    }
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_ready[device]) {
        int major = 0;
        err = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
        if (err != cudaSuccess || major != 10) {
            cudaGetLastError();
            return fail(B2_STATUS_BACKEND_UNAVAILABLE,
                        "CUDA backend unavailable: this library is built for sm_100a only");
        }
        void* address = nullptr;
        err = cudaGetSymbolAddress(&address, g_static_scratch);
        if (err != cudaSuccess || address == nullptr) {
            return fail_cuda(err != cudaSuccess ? err : cudaErrorInvalidSymbol,
                             "cudaGetSymbolAddress(static attention scratch)");
        }
        g_scratch_address[device] = address;
        g_scratch_ready[device] = true;
    }
    *out = g_scratch_address[device];
    *device_out = device;
    return B2_STATUS_OK;
}

}  // namespace
}  // namespace b2

extern "C" int32_t b2_paged_decode_attention_noalloc(
    const float* q, const float* k_pages, const float* v_pages, const uint32_t* block_tables,
    const uint32_t* seq_lens, float* ctx, uint32_t n_seq, uint32_t q_heads, uint32_t kv_heads,
    uint32_t head_width, uint32_t block_size, uint64_t physical_blocks, uint32_t max_blocks,
    uint32_t max_seq_len, uint32_t* status, void* stream) {
    using namespace b2;
    clear_error();
    // the same dimension rules as b2_paged_decode_attention
    B2_TRY(check_paged_dims(n_seq, q_heads, kv_heads, head_width, block_size, physical_blocks, max_blocks,
                            max_seq_len));
    if (q == nullptr || k_pages == nullptr || v_pages == nullptr || block_tables == nullptr ||
        seq_lens == nullptr || ctx == nullptr) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "paged decode attention pointers must not be null");
    }
    if (ctx == q || ctx == k_pages || ctx == v_pages) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "paged decode attention output must not alias an input");
    }
    const size_t need = paged_decode_workspace_bytes(n_seq, q_heads, head_width, block_size, max_seq_len);
    if (need > kStaticScratchBytes) {
        return fail(B2_STATUS_INVALID_ARGUMENT,
                    "paged decode attention needs %zu bytes of scratch but the allocation-free entry point "
                    "has a fixed %zu: lower n_seq * q_heads * ceil(max_seq_len / 256), or call "
                    "b2_paged_decode_attention with a workspace",
                    need, kStaticScratchBytes);
    }
    void* scratch = nullptr;
    DeviceContext here;   // only the device index is read by the launcher
    B2_TRY(static_scratch_pointer(&scratch, &here.device));
    PagedDecodeArgs args{q, k_pages, v_pages, block_tables, seq_lens, ctx,
                         n_seq, q_heads, kv_heads, head_width, block_size, max_blocks, max_seq_len,
                         physical_blocks, status};
    return launch_paged_decode(here, args, scratch, kStaticScratchBytes, static_cast<cudaStream_t>(stream));
}
