// Decode kernel for the packed-NF4 linear, batch rows <= 32, fed by TMA:
// y[r,o] = sum_i x[r,i] * W[o,i].
//
// Same arithmetic as nf4_gemv_stream.cu (W as the 16-row A operand of
// mma.sync m16n8k16, activations resident in registers as fp16 B fragments,
// one PRMT + one conflict-free table load per packed byte, FP32 block scale
// applied per 64-weight partial sum), but the packed codes no longer travel
// through the L1 load path into registers: one producer thread streams
// [16 rows x 128 byte] boxes into a shared-memory ring with
// cp.async.bulk.tensor (128-byte swizzle, so the 8-byte fragment reads of the
// 16 consumer warps are conflict free), completion is tracked by mbarriers.
// This keeps the L1/shared pipe for the table lookups, needs no load
// registers, and keeps ~96 KB per SM in flight.
// Every mbarrier wait is bounded; a timeout sets an error word and the kernel
// drains, it never spins forever.
// Reference loop: src/core/backend/nn/quantized_linear/reference/operations.cpp:49-81.
#include "b2_common.cuh"
#include "b2_kernels.h"
#include "sm100_ptx.cuh"

#include <cooperative_groups.h>
#include <cuda_fp16.h>

#include <mutex>

namespace cg = cooperative_groups;

namespace b2 {
namespace {

using namespace sm100;

constexpr int kWarps = 16;                       // consumer warps
constexpr int kThreadsProducerWarp = (kWarps + 1) * 32;   // consumer warps + one producer warp
constexpr int kStepK = 64;
constexpr int kTileRows = 16;
constexpr int kRedRow = kTileRows + 4;           // padded row of the [n][row] partial-sum layout
constexpr int kBoxBytes = kTileRows * 128;       // one TMA box: 16 rows x 128 bytes (4 steps)
constexpr int kLutBytes = 256 * 256;

template <int MT>
struct Layout {
    static constexpr int NB = 8 * MT;
    static constexpr int kMaxTiles = MT == 1 ? 48 : 16;
    // 32 batch rows: one partial-sum buffer (two barriers per tile), a 64 KB ring, and the
    // split-K output tiles behind the ring instead of below the table.
    // With 17 warps a scheduler partition holds 5 of them and the register file caps a thread at
    // 96 registers; the 32-row variant needs more, so it runs 16 warps (128 registers) and
    // thread 0 refills a stage itself once the CTA barrier shows every warp has read it.
    static constexpr bool kInlineProducer = MT == 4;
    static constexpr int kThreads = kInlineProducer ? kWarps * 32 : kThreadsProducerWarp;
    static constexpr int kRedParities = MT == 4 ? 1 : 2;
    static constexpr bool kOutBehindRing = MT == 4;
    static constexpr int kRingBytes = MT == 4 ? 64 * 1024 : 96 * 1024;
    // offsets from the first 16-byte aligned address of the dynamic allocation (below the table)
    static constexpr int kBarOff = 0;                                   // full[12], empty[12], abort
    static constexpr int kFactorOff = 256;                              // 256 floats
    static constexpr int kRedOff = kFactorOff + 1024;                   // [parity][16 warps][NB][20]
    static constexpr int kRedBytes = kRedParities * kWarps * (kTileRows + 4) * NB * 4;
    static constexpr int kOutBytes = kMaxTiles * kTileRows * NB * 4;    // [tile][16 rows][NB]
    static constexpr int kOutOff = kRedOff + kRedBytes;                 // when it lives below the table
    static constexpr int kLowBytes = kOutOff + (kOutBehindRing ? 0 : kOutBytes);
    static constexpr int kSmemBytes = 65536 /* bytes below the 64 KB-aligned table */ + kLutBytes + kRingBytes +
                                      (kOutBehindRing ? kOutBytes : 0);
};

struct TmaParams {
    WeightView w;
    const float* x;
    float* y;
    uint32_t rows;            // batch rows M
    uint32_t steps_total;     // in / 64
    uint32_t steps_per_cta;   // multiple of 4, <= 16 * SPW
    uint32_t row_tiles;       // ceil(out / 16)
    uint32_t blocks_per_row;  // in / block_size when rows are block aligned, else 0
    const uint32_t* lut;      // compact [256][32] words of fp16 pairs
    uint32_t* error;
};

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16_16816_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                   uint32_t a3, uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%10,%10,%10,%10};\n"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
// Table read: the table is constant once the kernel's first barrier has passed, so this load is
// not volatile and the compiler may hoist a whole step's lookups ahead of the MMAs.
__device__ __forceinline__ uint32_t lds_u32(uint32_t a) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds_u2(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ void cp_async_16(uint32_t dst32, const void* gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;\n" ::"r"(dst32), "l"(gmem_src));
}

struct RawScale {
    uint32_t bits;
    float second;
};

template <int MT, int SPW>
__global__ void __launch_bounds__(Layout<MT>::kThreads, 1)
nf4_gemv_tma_kernel(const __grid_constant__ CUtensorMap map_w, const TmaParams p) {
    using L = Layout<MT>;
    constexpr int NB = L::NB;
    constexpr uint32_t kThreads = L::kThreads;
    constexpr int NSC = (2 * SPW) / 4;                       // scales decoded per lane per tile
    constexpr int kWarpsPerBox = 4 / SPW;                    // SPW 4: one warp per box, SPW 2: two
    constexpr uint32_t kMaxBoxes = kWarps / kWarpsPerBox;    // boxes per stage at most
    constexpr uint32_t kStageBytes = kMaxBoxes * kBoxBytes;  // 32 KB or 16 KB
    constexpr uint32_t NS = L::kRingBytes / kStageBytes;     // 3, 6 or 4 stages

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t raw32 = smem_u32(smem_raw);
    const uint32_t low32 = (raw32 + 15u) & ~15u;
    const uint32_t lut32 = (raw32 + 65535u) & ~65535u;
    const uint32_t ring32 = lut32 + kLutBytes;
    uint8_t* low = smem_raw + (low32 - raw32);
    uint64_t* full = reinterpret_cast<uint64_t*>(low + L::kBarOff);
    uint64_t* empty = full + 12;
    volatile uint32_t* abort = reinterpret_cast<volatile uint32_t*>(low + L::kBarOff + 200);
    const float* s_factor = reinterpret_cast<const float*>(low + L::kFactorOff);
    float* s_red = reinterpret_cast<float*>(low + L::kRedOff);
    float* s_out = L::kOutBehindRing ? reinterpret_cast<float*>(smem_raw + (ring32 - raw32) + L::kRingBytes)
                                     : reinterpret_cast<float*>(low + L::kOutOff);

    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t ksplit = cluster.num_blocks();
    const uint32_t krank = cluster.block_rank();
    const uint32_t cluster_id = blockIdx.x / ksplit;
    const uint32_t n_clusters = gridDim.x / ksplit;

    const uint32_t tid = threadIdx.x;
    const uint32_t lane = tid & 31u, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t lut_lane = lut32 | (lane * 4u);
    const uint32_t quad_base = lane & ~3u;

    const WeightView& w = p.w;
    const uint64_t in = w.in_features, out = w.out_features;

    // The region below the table must hold barriers, factor table and reduction buffers.
    if (lut32 - low32 < static_cast<uint32_t>(L::kLowBytes)) {
        if (tid == 0 && p.error != nullptr) atomicOr(p.error, 2u);
        return;
    }

    const uint32_t slice_begin = min(krank * p.steps_per_cta, p.steps_total);
    const uint32_t slice_end = min(slice_begin + p.steps_per_cta, p.steps_total);
    const uint32_t n_boxes = (slice_end - slice_begin + 3u) / 4u;      // boxes per stage of this CTA
    const uint32_t my_tiles =
        cluster_id < p.row_tiles ? (p.row_tiles - cluster_id + n_clusters - 1) / n_clusters : 0u;

    if (tid == 0) {
        for (uint32_t s = 0; s < NS; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kWarps);
        }
        *abort = 0;
        mbar_fence_init();
        tma_prefetch_descriptor(&map_w);
    }
    // byte table (used half of each 256-byte row) and scale factor table
    for (uint32_t i = tid; i < 256 * 8; i += kThreads) {
        cp_async_16(lut32 + (i >> 3) * 256u + (i & 7u) * 16u, p.lut + i * 4);
    }
    asm volatile("cp.async.commit_group;\n" ::);
    if (tid < 256) reinterpret_cast<float*>(low + L::kFactorOff)[tid] = dq_factor(tid);
    asm volatile("cp.async.wait_group 0;\n" ::);
    __syncthreads();

    // Streams the boxes of tile `slot` of this CTA into its ring stage (one thread).
    auto issue_tile = [&](uint32_t slot) {
        const uint32_t s = slot % NS;
        mbar_expect_tx(&full[s], n_boxes * kBoxBytes);
        const int x0 = static_cast<int>(slice_begin * 32u);
        const int y = static_cast<int>((cluster_id + slot * n_clusters) * kTileRows);
        for (uint32_t b = 0; b < n_boxes; ++b) {
            tma_load_2d(smem_raw + (ring32 - raw32) + s * kStageBytes + b * kBoxBytes, &map_w,
                        x0 + static_cast<int>(b * 128u), y, &full[s]);
        }
    };

    if (!L::kInlineProducer && warp == kWarps) {
        // ---- producer warp: one thread streams this CTA's boxes of every tile ----
        if (lane == 0) {
            for (uint32_t slot = 0; slot < my_tiles; ++slot) {
                if (slot >= NS) mbar_wait(&empty[slot % NS], ((slot / NS) - 1u) & 1u, abort);
                issue_tile(slot);
            }
        }
    } else {
        if (L::kInlineProducer && tid == 0) {
            for (uint32_t slot = 0; slot < my_tiles && slot < NS; ++slot) issue_tile(slot);
        }
        // ---- consumers ----
        const uint32_t box = warp / kWarpsPerBox;
        const uint32_t sub0 = (warp % kWarpsPerBox) * SPW;           // first step of this warp inside its box
        const uint32_t step0 = slice_begin + warp * SPW;
        const uint32_t my_steps = step0 < slice_end ? min(static_cast<uint32_t>(SPW), slice_end - step0) : 0u;
        const bool warp_active = my_steps > 0;                       // warp-uniform

        const uint32_t scale_step_raw = SPW == 4 ? t : (t & 1u);
        const uint32_t scale_step = warp_active ? min(scale_step_raw, my_steps - 1) : 0u;
        auto scale_row_half = [&](int k) -> uint32_t { return SPW == 4 ? static_cast<uint32_t>(k) : (t >> 1); };
        const bool fp32_scales = w.encoding == B2_SCALES_FLOAT32;
        const uint32_t blocks_per_row = p.blocks_per_row;
        const uint32_t tile_stride_rows = n_clusters * kTileRows;

        RawScale sraw[2][NSC];
        // Hoisted weight-view fields and this lane's running scale-block index: rows are block
        // aligned and tiles are whole (the launcher checks both), so the index of (row, step) is
        // base + slot * stride.
        const float* const fp32_ptr = w.fp32_scales;
        const uint8_t* const code_ptr = w.scale_codes;
        const float* const second_ptr = w.second_level;
        const uint32_t sshift = w.scale_block_shift;
        const uint32_t fbase = static_cast<uint32_t>(w.flat_block_base);
        const float dq_offset = w.offset;
        uint32_t blk0[NSC];
#pragma unroll
        for (int k = 0; k < NSC; ++k) {
            blk0[k] = (cluster_id * kTileRows + g + 8u * scale_row_half(k)) * blocks_per_row +
                      (((step0 + scale_step) * static_cast<uint32_t>(kStepK)) >> w.block_shift);
        }
        const uint32_t blk_stride = tile_stride_rows * blocks_per_row;
        auto fetch_scales = [&](int d, uint32_t slot) {
            if (slot < my_tiles && warp_active) {
#pragma unroll
                for (int k = 0; k < NSC; ++k) {
                    const uint32_t block = blk0[k] + slot * blk_stride;
                    if (fp32_scales) {
                        sraw[d][k].bits = __float_as_uint(__ldg(fp32_ptr + block));
                        sraw[d][k].second = 0.0f;
                    } else {
                        sraw[d][k].bits = __ldg(code_ptr + block);
                        sraw[d][k].second = __ldg(second_ptr + ((fbase + block) >> sshift));
                    }
                }
            }
        };
        (void)tile_stride_rows;
        fetch_scales(0, 0);

        // Activations of this warp's steps as fp16 B fragments (registers for the whole kernel).
        uint4 xf[MT][SPW][2];
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int u = 0; u < SPW; ++u) {
                float4 v[4];
                const uint32_t n = m * 8 + g;
                const bool have = n < p.rows && static_cast<uint32_t>(u) < my_steps;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    v[q4] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (have) {
                        v[q4] = __ldg(reinterpret_cast<const float4*>(
                            p.x + static_cast<uint64_t>(n) * in + static_cast<uint64_t>(step0 + u) * kStepK + 16 * t + 4 * q4));
                    }
                }
                uint32_t h[8];
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    __half2 lo = __floats2half2_rn(v[q4].x, v[q4].y), hi = __floats2half2_rn(v[q4].z, v[q4].w);
                    h[2 * q4] = *reinterpret_cast<uint32_t*>(&lo);
                    h[2 * q4 + 1] = *reinterpret_cast<uint32_t*>(&hi);
                }
                xf[m][u][0] = make_uint4(h[0], h[1], h[2], h[3]);
                xf[m][u][1] = make_uint4(h[4], h[5], h[6], h[7]);
            }

        // byte offset of this lane's 8-byte fragment inside a box, per step: rows g and g+8 share
        // the swizzle term (row & 7) = g
        uint32_t frag_off[SPW];
#pragma unroll
        for (int u = 0; u < SPW; ++u) {
            const uint32_t st = min(sub0 + static_cast<uint32_t>(u), sub0 + (warp_active ? my_steps - 1u : 0u));
            frag_off[u] = g * 128u + (((2u * st + (t >> 1)) ^ g) << 4) + (t & 1u) * 8u;
        }

        // reducing threads (tid < 16 * NB): output element (n = tid / 16, r = tid % 16) of every tile
        const uint32_t red_n = tid / kTileRows, red_r = tid % kTileRows;
        float* y_run = p.y + static_cast<uint64_t>(red_n) * out + static_cast<uint64_t>(cluster_id) * kTileRows + red_r;
        const uint64_t y_stride = static_cast<uint64_t>(tile_stride_rows);
        const bool red_store = tid < kTileRows * NB && red_n < p.rows;

        uint32_t parity = 0;
        for (uint32_t base = 0; base < my_tiles; base += 2) {
#pragma unroll
            for (int d = 0; d < 2; ++d) {
                const uint32_t slot = base + d;
                if (slot < my_tiles) {   // CTA-uniform
                    fetch_scales(d ^ 1, slot + 1);
                    const uint32_t s = slot % NS;
                    float acc[MT][4];
#pragma unroll
                    for (int m = 0; m < MT; ++m)
#pragma unroll
                        for (int e = 0; e < 4; ++e) acc[m][e] = 0.0f;
                    mbar_wait(&full[s], (slot / NS) & 1u, abort);
                    uint2 wa[SPW], wb[SPW];
                    if (warp_active) {
                        const uint32_t box32 = ring32 + s * kStageBytes + box * kBoxBytes;
#pragma unroll
                        for (int u = 0; u < SPW; ++u) {
                            wa[u] = lds_u2(box32 + frag_off[u]);
                            wb[u] = lds_u2(box32 + frag_off[u] + 1024u);
                        }
                    }
                    __syncwarp();
                    // Release the stage once this warp's fragment reads have RETURNED: the arrive
                    // takes the last loaded register as a (dummy) operand, so it cannot issue earlier.
                    if (!L::kInlineProducer && lane == 0) {
                        const uint32_t dep = warp_active ? wb[SPW - 1].y : 0u;
                        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0]; // %1" ::"r"(smem_u32(&empty[s])), "r"(dep)
                                     : "memory");
                    }
                    if (warp_active) {
                        float sc[NSC];
#pragma unroll
                        for (int k = 0; k < NSC; ++k) {
                            sc[k] = fp32_scales ? __uint_as_float(sraw[d][k].bits)
                                                : dq_finish(s_factor[sraw[d][k].bits], sraw[d][k].second, dq_offset);
                        }
#pragma unroll
                        for (int u = 0; u < SPW; ++u) {
                            const float sA = __shfl_sync(0xFFFFFFFFu, sc[0], quad_base + u);
                            const float sB = SPW == 4 ? __shfl_sync(0xFFFFFFFFu, sc[NSC - 1], quad_base + u)
                                                      : __shfl_sync(0xFFFFFFFFu, sc[0], quad_base + 2 + u);
                            float part[MT][4];
                            const uint32_t wwa[2] = {wa[u].x, wa[u].y};
                            const uint32_t wwb[2] = {wb[u].x, wb[u].y};
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const uint32_t word_a = wwa[i >> 1], word_b = wwb[i >> 1];
                                const uint32_t sel0 = (i & 1) ? 0x7624u : 0x7604u;
                                const uint32_t sel1 = (i & 1) ? 0x7634u : 0x7614u;
                                const uint32_t a0 = lds_u32(__byte_perm(word_a, lut_lane, sel0));
                                const uint32_t a2 = lds_u32(__byte_perm(word_a, lut_lane, sel1));
                                const uint32_t a1 = lds_u32(__byte_perm(word_b, lut_lane, sel0));
                                const uint32_t a3 = lds_u32(__byte_perm(word_b, lut_lane, sel1));
#pragma unroll
                                for (int m = 0; m < MT; ++m) {
                                    const uint4& xv = xf[m][u][i >> 1];
                                    const uint32_t b0 = (i & 1) ? xv.z : xv.x;
                                    const uint32_t b1 = (i & 1) ? xv.w : xv.y;
                                    if (i == 0) {
                                        mma_f16_16816_zero(part[m], a0, a1, a2, a3, b0, b1);
                                    } else {
                                        mma_f16_16816(part[m], a0, a1, a2, a3, b0, b1);
                                    }
                                }
                            }
#pragma unroll
                            for (int m = 0; m < MT; ++m) {
                                acc[m][0] = fmaf(sA, part[m][0], acc[m][0]);
                                acc[m][1] = fmaf(sA, part[m][1], acc[m][1]);
                                acc[m][2] = fmaf(sB, part[m][2], acc[m][2]);
                                acc[m][3] = fmaf(sB, part[m][3], acc[m][3]);
                            }
                        }
                    }
                    // partial tile as [n][row] with rows padded to 20 words: conflict-free scalar stores
                    // here, contiguous reads by the reducing threads below
                    if (L::kRedParities == 1) {
                        // every warp has read its fragments of this stage and the reducers of the
                        // previous tile are done
                        asm volatile("bar.sync 1, 512;" ::: "memory");
                        if (L::kInlineProducer && tid == 0 && slot + NS < my_tiles) issue_tile(slot + NS);
                    }
                    float* red = s_red + (parity * kWarps + warp) * (NB * kRedRow);
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        float* q = red + (m * 8 + 2 * t) * kRedRow;
                        q[g] = acc[m][0];
                        q[kRedRow + g] = acc[m][1];
                        q[g + 8] = acc[m][2];
                        q[kRedRow + g + 8] = acc[m][3];
                    }
                    asm volatile("bar.sync 1, 512;" ::: "memory");
                    if (tid < kTileRows * NB) {
                        const float* src = s_red + parity * kWarps * (NB * kRedRow) + red_n * kRedRow + red_r;
                        float v = 0.0f;
#pragma unroll
                        for (int k = 0; k < kWarps; ++k) v += src[k * (NB * kRedRow)];
                        if (ksplit == 1) {
                            if (red_store) y_run[slot * y_stride] = v;
                        } else {
                            s_out[slot * kTileRows * NB + red_r * NB + red_n] = v;
                        }
                    }
                    if (L::kRedParities == 2) parity ^= 1u;
                }
            }
        }
    }

    if (ksplit > 1) {
        // ---- combine the cluster ranks (fixed order) and store ----
        cluster.sync();
        const uint32_t total = my_tiles * kTileRows * NB;
        for (uint32_t e = tid + krank * kThreads; e < total; e += kThreads * ksplit) {
            const uint32_t slot = e / (kTileRows * NB), rem = e % (kTileRows * NB);
            const uint32_t n = rem / kTileRows, r = rem % kTileRows;
            float v = 0.0f;
            for (uint32_t k = 0; k < ksplit; ++k) v += cluster.map_shared_rank(s_out, k)[slot * kTileRows * NB + r * NB + n];
            const uint64_t row = static_cast<uint64_t>(cluster_id + slot * n_clusters) * kTileRows + r;
            if (n < p.rows && row < out) p.y[static_cast<uint64_t>(n) * out + row] = v;
        }
        cluster.sync();
    }
    if (tid == 0 && *abort != 0 && p.error != nullptr) atomicOr(p.error, 4u);
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
        }
    });
    return fn;
}

// Clusters of `ksplit` CTAs of this kernel the device can hold at once (GPC packing), cached.
template <int MT, int SPW>
int32_t max_active_clusters(const DeviceContext& ctx, uint32_t ksplit, uint32_t* out) {
    auto kernel = nf4_gemv_tma_kernel<MT, SPW>;
    static bool configured = false;
    static int cached[9] = {0};
    if (!configured) {
        B2_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Layout<MT>::kSmemBytes));
        configured = true;
    }
    if (cached[ksplit] == 0) {
        cudaLaunchConfig_t config = {};
        config.blockDim = dim3(Layout<MT>::kThreads);
        config.dynamicSmemBytes = Layout<MT>::kSmemBytes;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = ksplit;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        config.attrs = attr;
        config.numAttrs = 1;
        config.gridDim = dim3(static_cast<unsigned>(ctx.sm_count / ksplit) * ksplit);
        int n = 0;
        B2_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, kernel, &config));
        cached[ksplit] = n > 0 ? n : 1;
    }
    uint32_t clusters = static_cast<uint32_t>(cached[ksplit]);
    const uint32_t by_sm = static_cast<uint32_t>(ctx.sm_count) / ksplit;
    *out = clusters < by_sm ? clusters : by_sm;
    return B2_STATUS_OK;
}

template <int MT, int SPW>
int32_t launch_tma(const DeviceContext& ctx, const CUtensorMap& map, TmaParams p, uint32_t ksplit,
                   cudaStream_t stream) {
    auto kernel = nf4_gemv_tma_kernel<MT, SPW>;
    uint32_t clusters = 0;
    B2_TRY((max_active_clusters<MT, SPW>(ctx, ksplit, &clusters)));
    if (clusters > p.row_tiles) clusters = p.row_tiles;
    if (clusters == 0) clusters = 1;
    if ((p.row_tiles + clusters - 1) / clusters > static_cast<uint32_t>(Layout<MT>::kMaxTiles)) {
        return fail(B2_STATUS_RUNTIME_ERROR, "internal: NF4 TMA decode kernel tile budget exceeded");
    }
    cudaLaunchConfig_t config = {};
    config.blockDim = dim3(Layout<MT>::kThreads);
    config.dynamicSmemBytes = Layout<MT>::kSmemBytes;
    config.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ksplit;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    config.gridDim = dim3(clusters * ksplit);
    B2_CUDA_TRY(cudaLaunchKernelEx(&config, kernel, map, p));
    return B2_STATUS_OK;
}

}  // namespace

// Shapes the TMA decode kernel takes: whole 128-byte boxes per CTA slice, 16-byte aligned rows.
bool nf4_gemv_tma_plan(const DeviceContext& ctx, const WeightView& w, const float* x, uint64_t rows,
                       uint32_t* ksplit_out, uint32_t* steps_per_cta_out) {
    if (rows < 1 || rows > 32 || w.in_features % kStepK != 0 || w.block_size < kStepK) return false;
    if ((reinterpret_cast<uintptr_t>(w.codes) & 15u) != 0 || (reinterpret_cast<uintptr_t>(x) & 15u) != 0) return false;
    if (encode_tiled() == nullptr) return false;
    if (w.in_features % w.block_size != 0 || w.out_features % kTileRows != 0) return false;
    const uint64_t steps = w.in_features / kStepK;
    const uint64_t row_tiles = (w.out_features + kTileRows - 1) / kTileRows;
    if (steps > 0xFFFFFFull || row_tiles > 0x7FFFFFFull || w.out_features > 0x7FFFFFFFull) return false;
    if ((w.out_features + 2048) * (w.in_features / w.block_size + 1) + w.flat_block_base > 0xFFFFFFFFull) return false;
    const uint64_t cap = rows <= 8 ? 64 : 32;   // steps one CTA covers (16 warps x 4 or 2)
    uint64_t ks = (steps + cap - 1) / cap;
    if (ks > 8) return false;
    uint64_t per = (steps + ks - 1) / ks;
    per = (per + 3) / 4 * 4;
    if (per > cap) return false;
    uint32_t active = 0;
    const int32_t st = rows <= 8    ? max_active_clusters<1, 4>(ctx, static_cast<uint32_t>(ks), &active)
                       : rows <= 16 ? max_active_clusters<2, 2>(ctx, static_cast<uint32_t>(ks), &active)
                                    : max_active_clusters<4, 2>(ctx, static_cast<uint32_t>(ks), &active);
    if (st != B2_STATUS_OK) {
        clear_error();
        return false;
    }
    const uint64_t clusters = active;
    if (clusters == 0) return false;
    const uint64_t max_tiles = rows <= 8 ? 48 : 16;
    if ((row_tiles + clusters - 1) / clusters > max_tiles) return false;
    *ksplit_out = static_cast<uint32_t>(ks);
    *steps_per_cta_out = static_cast<uint32_t>(per);
    return true;
}

int32_t launch_nf4_gemv_tma(const DeviceContext& ctx, const WeightView& w, const float* x, float* y,
                            uint64_t rows, uint32_t ksplit, uint32_t steps_per_cta, cudaStream_t stream) {
    CUtensorMap map;
    const cuuint64_t dims[2] = {w.in_features / 2, w.out_features};
    const cuuint64_t strides[1] = {w.in_features / 2};
    const cuuint32_t box[2] = {128, kTileRows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode_tiled()(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(w.codes), dims,
                                      strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B2_STATUS_RUNTIME_ERROR, "cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
    TmaParams p;
    p.w = w;
    p.x = x;
    p.y = y;
    p.rows = static_cast<uint32_t>(rows);
    p.steps_total = static_cast<uint32_t>(w.in_features / kStepK);
    p.steps_per_cta = steps_per_cta;
    p.row_tiles = static_cast<uint32_t>((w.out_features + kTileRows - 1) / kTileRows);
    p.blocks_per_row = w.in_features % w.block_size == 0 ? static_cast<uint32_t>(w.in_features / w.block_size) : 0u;
    p.lut = ctx.gemv_lut;
    p.error = ctx.gemm_error;
    if (rows <= 8) return launch_tma<1, 4>(ctx, map, p, ksplit, stream);
    if (rows <= 16) return launch_tma<2, 2>(ctx, map, p, ksplit, stream);
    return launch_tma<4, 2>(ctx, map, p, ksplit, stream);
}

}  // namespace b2
