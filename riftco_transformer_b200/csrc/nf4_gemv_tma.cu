// Decode kernel for the packed-NF4 linear, batch rows <= 16, fed by TMA:
// y[r,o] = sum_i x[r,i] * W[o,i].
//
// Same arithmetic as nf4_gemv.cu (W as the 16-row A operand of
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

#include <cstdlib>
#include <mutex>

namespace cg = cooperative_groups;

namespace b2 {
namespace {

using namespace sm100;

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kStepK = 64;
constexpr int kTileRows = 16;
constexpr int kRedRow = kTileRows + 4;           // padded row of the [n][row] partial-sum layout
constexpr int kBoxBytes = kTileRows * 128;       // one TMA box: 16 rows x 128 bytes (4 steps)
constexpr int kLutBytes = 256 * 256;
// Per ring stage, the tile's raw scales: a [16 rows x kScaleBoxU8 bytes] box of scale codes
// (or [16 x kScaleBoxF32] floats) and 32 second-level values.
constexpr int kScaleBoxU8 = 64 + 16;             // blocks of the widest CTA slice + alignment slack
constexpr int kScaleBoxF32 = 64 + 4;
constexpr int kScaleBoxBytesU8 = kTileRows * kScaleBoxU8;          // 1280
constexpr int kScaleBoxBytesF32 = kTileRows * kScaleBoxF32 * 4;    // 4352
constexpr int kSecondOff = kScaleBoxBytesF32;
constexpr int kSecondBox = 32;                   // floats
constexpr int kScaleStageBytes = 4608;           // 4352 + 128, rounded to 128

// MT = batch rows / 8. Sixteen warps share the contraction range of the CTA, SPW steps of 64
// each; thread 0 is also the producer: it refills a ring stage once a CTA barrier has shown that
// every warp is done with it. (A seventeenth, dedicated producer warp would put five warps on
// one scheduler partition and cap every thread at 96 registers.)
template <int MT>
struct Layout {
    static constexpr int NB = 8 * MT;
    static constexpr int SPW = MT == 4 ? 2 : 4;
    static constexpr int kWarpsPerBox = 4 / SPW;
    static constexpr int kBoxesPerStage = kWarps / kWarpsPerBox;
    static constexpr int kStageBytes = kBoxesPerStage * kBoxBytes;      // 32 KB or 16 KB
    static constexpr int kRingBytes = MT == 4 ? 64 * 1024 : 96 * 1024;
    static constexpr int NS = kRingBytes / kStageBytes;                 // 3 or 4 stages
    static constexpr int kMaxTiles = MT == 1 ? 48 : 16;
    // One partial-sum buffer costs a second CTA barrier per tile; 8 batch rows can afford two.
    static constexpr int kRedParities = MT == 1 ? 2 : 1;
    static constexpr bool kOutBehindRing = MT == 4;
    // offsets from the first 128-byte aligned address of the dynamic allocation (below the table)
    static constexpr int kBarOff = 0;                                   // full[8], abort
    static constexpr int kFactorOff = 256;                              // 256 floats
    static constexpr int kScaleOff = 1280;                              // [stage] raw scales
    static constexpr int kRedOff = kScaleOff + NS * kScaleStageBytes;   // [parity][16 warps][NB][20]
    static constexpr int kRedBytes = kRedParities * kWarps * kRedRow * NB * 4;
    static constexpr int kOutBytes = kMaxTiles * kTileRows * NB * 4;    // [tile][16 rows][NB]
    static constexpr int kOutOff = kRedOff + kRedBytes;                 // when it lives below the table
    static constexpr int kLowBytes = kOutOff + (kOutBehindRing ? 0 : kOutBytes);
    static constexpr int kSmemBytes = 65536 /* bytes below the 64 KB-aligned table */ + kLutBytes + kRingBytes +
                                      (kOutBehindRing ? kOutBytes : 0);
    static_assert(kLowBytes <= 65536 - 2048, "region below the table too large");
};

struct TmaParams {
    WeightView w;
    const float* x;
    float* y;
    uint32_t rows;            // batch rows M
    uint32_t steps_total;     // in / 64
    uint32_t steps_per_cta;   // multiple of 4, <= 16 * SPW
    uint32_t row_tiles;       // out / 16
    uint32_t blocks_per_row;  // in / block_size
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
__device__ __forceinline__ float lds_f32(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds_u8(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];\n" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void tma_load_1d(uint32_t dst32, const CUtensorMap* map, int x, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.1d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2}], [%3];"
                 ::"r"(dst32), "l"(map), "r"(x), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tma_load_2d_at(uint32_t dst32, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst32), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void cp_async_16(uint32_t dst32, const void* gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;\n" ::"r"(dst32), "l"(gmem_src));
}

template <int MT>
__global__ void __launch_bounds__(kThreads, 1)
nf4_gemv_tma_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_s,
                    const __grid_constant__ CUtensorMap map_2, const TmaParams p) {
    using L = Layout<MT>;
    constexpr int NB = L::NB;
    constexpr int SPW = L::SPW;
    constexpr int NSC = (2 * SPW) / 4;                       // scales decoded per lane per tile
    constexpr uint32_t kWarpsPerBox = L::kWarpsPerBox;
    constexpr uint32_t kStageBytes = L::kStageBytes;
    constexpr uint32_t NS = L::NS;

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t raw32 = smem_u32(smem_raw);
    const uint32_t low32 = (raw32 + 127u) & ~127u;
    const uint32_t lut32 = (raw32 + 65535u) & ~65535u;
    const uint32_t ring32 = lut32 + kLutBytes;
    const uint32_t scale32 = low32 + L::kScaleOff;
    uint8_t* low = smem_raw + (low32 - raw32);
    uint64_t* full = reinterpret_cast<uint64_t*>(low + L::kBarOff);
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

    // The region below the table must hold barriers, factor table, scales and reduction buffers.
    if (lut32 - low32 < static_cast<uint32_t>(L::kLowBytes)) {
        if (tid == 0 && p.error != nullptr) atomicOr(p.error, 2u);
        return;
    }

    const uint32_t slice_begin = min(krank * p.steps_per_cta, p.steps_total);
    const uint32_t slice_end = min(slice_begin + p.steps_per_cta, p.steps_total);
    const uint32_t n_boxes = (slice_end - slice_begin + 3u) / 4u;      // boxes per stage of this CTA
    const uint32_t my_tiles =
        cluster_id < p.row_tiles ? (p.row_tiles - cluster_id + n_clusters - 1) / n_clusters : 0u;

    // Scale blocks of this CTA's slice: first block column, rounded down to the 16-byte
    // granularity a TMA coordinate needs; running block index of the first tile's first row.
    const bool fp32_scales = w.encoding == B2_SCALES_FLOAT32;
    const uint32_t blocks_per_row = p.blocks_per_row;
    const uint32_t b_begin = (slice_begin * static_cast<uint32_t>(kStepK)) >> w.block_shift;
    const uint32_t scale_x0 = fp32_scales ? (b_begin & ~3u) : (b_begin & ~15u);
    const uint32_t sshift = w.scale_block_shift;
    const uint32_t fbase = static_cast<uint32_t>(w.flat_block_base);
    const uint32_t tile_stride_rows = n_clusters * kTileRows;
    const uint32_t blk_stride = tile_stride_rows * blocks_per_row;
    const uint32_t tile_blk0 = cluster_id * kTileRows * blocks_per_row + b_begin;   // + slot * blk_stride
    const uint32_t tx_bytes = n_boxes * kBoxBytes +
                              (fp32_scales ? kScaleBoxBytesF32 : kScaleBoxBytesU8 + kSecondBox * 4);

    // Streams tile `slot` of this CTA into its ring stage: packed codes, raw scales and, for
    // double-quantised weights, the second-level values the tile's blocks refer to (one thread).
    auto issue_tile = [&](uint32_t slot) {
        const uint32_t s = slot % NS;
        mbar_expect_tx(&full[s], tx_bytes);
        const int x0 = static_cast<int>(slice_begin * 32u);
        const int y = static_cast<int>((cluster_id + slot * n_clusters) * kTileRows);
        for (uint32_t b = 0; b < n_boxes; ++b) {
            tma_load_2d_at(ring32 + s * kStageBytes + b * kBoxBytes, &map_w, x0 + static_cast<int>(b * 128u), y,
                           &full[s]);
        }
        const uint32_t sdst = scale32 + s * kScaleStageBytes;
        tma_load_2d_at(sdst, &map_s, static_cast<int>(scale_x0), y, &full[s]);
        if (!fp32_scales) {
            const uint32_t first = (fbase + tile_blk0 + slot * blk_stride) >> sshift;
            tma_load_1d(sdst + kSecondOff, &map_2, static_cast<int>(first & ~3u), &full[s]);
        }
    };

    // Set-up that touches no tensor of the caller (barriers, the byte table, the factor table)
    // runs before the dependency wait, so it overlaps the tail of the previous kernel in the
    // stream; weights, scales and activations are only read after it.
    if (tid == 0) {
        for (uint32_t s = 0; s < NS; ++s) mbar_init(&full[s], 1);
        *abort = 0;
        mbar_fence_init();
    }
    for (uint32_t i = tid; i < 256 * 8; i += kThreads) {
        cp_async_16(lut32 + (i >> 3) * 256u + (i & 7u) * 16u, p.lut + i * 4);
    }
    asm volatile("cp.async.commit_group;\n" ::);
    if (tid < 256) reinterpret_cast<float*>(low + L::kFactorOff)[tid] = dq_factor(tid);
    // The first ring fill reads only the immutable weights and writes only this CTA's shared memory,
    // so it too goes out before the dependency wait: the loads are in flight while the previous
    // kernel drains. Activations and outputs are touched after the wait.
    if (tid == 0) {
        for (uint32_t slot = 0; slot < my_tiles && slot < NS; ++slot) issue_tile(slot);
    }
    pdl_launch_dependents();
    pdl_wait();

    {
        const uint32_t box = warp / kWarpsPerBox;
        const uint32_t sub0 = (warp % kWarpsPerBox) * SPW;           // first step of this warp inside its box
        const uint32_t step0 = slice_begin + warp * SPW;
        const uint32_t my_steps = step0 < slice_end ? min(static_cast<uint32_t>(SPW), slice_end - step0) : 0u;
        const bool warp_active = my_steps > 0;                       // warp-uniform

        // This lane decodes NSC scales per tile: SPW 4 -> (row g, step t) and (row g+8, step t);
        // SPW 2 -> (row g + 8*(t/2), step t%2). Quad shuffles hand them to the lanes that use them.
        const uint32_t scale_step_raw = SPW == 4 ? t : (t & 1u);
        const uint32_t scale_step = warp_active ? min(scale_step_raw, my_steps - 1) : 0u;
        const float dq_offset = w.offset;
        const uint32_t lane_block = ((step0 + scale_step) * static_cast<uint32_t>(kStepK)) >> w.block_shift;
        uint32_t scale_addr[NSC];   // shared-memory byte offset of this lane's raw scale inside a stage
        uint32_t blk0[NSC];         // its block index relative to the tile's first block
#pragma unroll
        for (int k = 0; k < NSC; ++k) {
            const uint32_t row = g + 8u * (SPW == 4 ? static_cast<uint32_t>(k) : (t >> 1));
            scale_addr[k] = fp32_scales ? (row * kScaleBoxF32 + (lane_block - scale_x0)) * 4u
                                        : row * kScaleBoxU8 + (lane_block - scale_x0);
            blk0[k] = row * blocks_per_row + (lane_block - b_begin);
        }

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
            frag_off[u] = box * kBoxBytes + g * 128u + (((2u * st + (t >> 1)) ^ g) << 4) + (t & 1u) * 8u;
        }

        // reducing threads (tid < 16 * NB): output element (n = tid / 16, r = tid % 16) of every tile
        const uint32_t red_n = tid / kTileRows, red_r = tid % kTileRows;
        float* y_run = p.y + static_cast<uint64_t>(red_n) * out + static_cast<uint64_t>(cluster_id) * kTileRows + red_r;
        const bool red_thread = tid < kTileRows * NB;
        const bool red_store = red_thread && red_n < p.rows;
        float* const my_red = s_red + warp * (NB * kRedRow);
        const float* const red_src = s_red + red_n * kRedRow + red_r;
        float* out_run = s_out + red_r * NB + red_n;

        asm volatile("cp.async.wait_group 0;\n" ::);
        __syncthreads();   // tables and barrier initialisation visible to every thread

        uint32_t parity_off = 0;          // float offset of the partial-sum buffer in use
        uint32_t stage = 0, phase = 0;    // ring position of the current tile
        uint32_t tile_first = fbase + tile_blk0;   // flat index of the tile's first scale block
        for (uint32_t slot = 0; slot < my_tiles; ++slot) {
            const uint32_t stage_ring = ring32 + stage * kStageBytes;
            const uint32_t stage_scale = scale32 + stage * kScaleStageBytes;
            mbar_wait(&full[stage], phase, abort);
            float acc[MT][4];
#pragma unroll
            for (int m = 0; m < MT; ++m)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[m][e] = 0.0f;
            if (warp_active) {
                uint2 wa[SPW], wb[SPW];
#pragma unroll
                for (int u = 0; u < SPW; ++u) {
                    wa[u] = lds_u2(stage_ring + frag_off[u]);
                    wb[u] = lds_u2(stage_ring + frag_off[u] + 1024u);
                }
                float sc[NSC];
#pragma unroll
                for (int k = 0; k < NSC; ++k) {
                    if (fp32_scales) {
                        sc[k] = lds_f32(stage_scale + scale_addr[k]);
                    } else {
                        const uint32_t code = lds_u8(stage_scale + scale_addr[k]);
                        const uint32_t idx = ((tile_first + blk0[k]) >> sshift) - ((tile_first >> sshift) & ~3u);
                        const float second = lds_f32(stage_scale + kSecondOff + idx * 4u);
                        sc[k] = dq_finish(s_factor[code], second, dq_offset);
                    }
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
            if (L::kRedParities == 1) {
                // every warp is done with this ring stage, and the reducers of the previous tile
                // are done with the partial-sum buffer
                __syncthreads();
                if (tid == 0 && slot + NS < my_tiles) issue_tile(slot + NS);
            }
            // partial tile as [n][row] with rows padded to 20 words: conflict-free scalar stores
            // here, contiguous reads by the reducing threads below
            {
                float* red = my_red + parity_off;
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    float* q = red + (m * 8 + 2 * t) * kRedRow;
                    q[g] = acc[m][0];
                    q[kRedRow + g] = acc[m][1];
                    q[g + 8] = acc[m][2];
                    q[kRedRow + g + 8] = acc[m][3];
                }
            }
            __syncthreads();
            if (L::kRedParities == 2) {
                if (tid == 0 && slot + NS < my_tiles) issue_tile(slot + NS);
            }
            if (red_thread) {
                const float* src = red_src + parity_off;
                float v = 0.0f;
#pragma unroll
                for (int k = 0; k < kWarps; ++k) v += src[k * (NB * kRedRow)];
                if (ksplit == 1) {
                    if (red_store) *y_run = v;
                } else {
                    *out_run = v;
                }
            }
            y_run += tile_stride_rows;
            out_run += kTileRows * NB;
            tile_first += blk_stride;
            if (L::kRedParities == 2) parity_off ^= static_cast<uint32_t>(kWarps * NB * kRedRow);
            if (++stage == NS) {
                stage = 0;
                phase ^= 1u;
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
template <int MT>
int32_t max_active_clusters(const DeviceContext& ctx, uint32_t ksplit, uint32_t* out) {
    auto kernel = nf4_gemv_tma_kernel<MT>;
    static PerDeviceOnce configured;                 // per template instance
    static int cached_all[kMaxDevices][9] = {};      // clusters per cluster size, per device
    static std::mutex cache_mutex;
    B2_TRY(once_per_device(configured, ctx.device, [kernel]() -> int32_t {
        B2_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Layout<MT>::kSmemBytes));
        return B2_STATUS_OK;
    }));
    std::lock_guard<std::mutex> lock(cache_mutex);
    int* cached = cached_all[ctx.device];
    if (cached[ksplit] == 0) {
        cudaLaunchConfig_t config = {};
        config.blockDim = dim3(kThreads);
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

int32_t active_clusters_for(const DeviceContext& ctx, uint64_t rows, uint32_t ksplit, uint32_t* out) {
    if (rows <= 8) return max_active_clusters<1>(ctx, ksplit, out);
    return max_active_clusters<2>(ctx, ksplit, out);
}

template <int MT>
int32_t launch_tma(const DeviceContext& ctx, const CUtensorMap& map_w, const CUtensorMap& map_s,
                   const CUtensorMap& map_2, TmaParams p, uint32_t ksplit, cudaStream_t stream) {
    auto kernel = nf4_gemv_tma_kernel<MT>;
    uint32_t clusters = 0;
    B2_TRY((max_active_clusters<MT>(ctx, ksplit, &clusters)));
    if (clusters > p.row_tiles) clusters = p.row_tiles;
    if (clusters == 0) clusters = 1;
    if ((p.row_tiles + clusters - 1) / clusters > static_cast<uint32_t>(Layout<MT>::kMaxTiles)) {
        return fail(B2_STATUS_RUNTIME_ERROR, "internal: NF4 TMA decode kernel tile budget exceeded");
    }
    cudaLaunchConfig_t config = {};
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = Layout<MT>::kSmemBytes;
    config.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ksplit;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // Programmatic stream serialisation: the kernel may start while its predecessor drains; it
    // calls griddepcontrol.wait before it reads or writes any caller tensor.
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = 2;
    config.gridDim = dim3(clusters * ksplit);
    B2_CUDA_TRY(cudaLaunchKernelEx(&config, kernel, map_w, map_s, map_2, p));
    return B2_STATUS_OK;
}

int32_t encode(const char* what, CUtensorMap* map, CUtensorMapDataType type, uint32_t rank, const void* base,
               const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box, CUtensorMapSwizzle swizzle) {
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode_tiled()(map, type, rank, const_cast<void*>(base), dims, strides, box, elem,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        return fail(B2_STATUS_RUNTIME_ERROR, "cuTensorMapEncodeTiled failed (%d) for the %s map", static_cast<int>(r), what);
    }
    return B2_STATUS_OK;
}

}  // namespace

// Shapes the TMA decode kernel takes: whole 16-row tiles, rows made of whole scale blocks, every
// array 16-byte aligned with 16-byte aligned row pitches (what a TMA descriptor needs), and few
// enough second-level values per tile to fit the 32-float box.
bool nf4_gemv_tma_plan(const DeviceContext& ctx, const WeightView& w, const float* x, uint64_t rows,
                       uint32_t* ksplit_out, uint32_t* steps_per_cta_out) {
    if (rows < 1 || rows > 16 || w.in_features % kStepK != 0 || w.block_size < kStepK) return false;
    if ((reinterpret_cast<uintptr_t>(w.codes) & 15u) != 0 || (reinterpret_cast<uintptr_t>(x) & 15u) != 0) return false;
    if (encode_tiled() == nullptr) return false;
    if (w.in_features % w.block_size != 0 || w.out_features % kTileRows != 0) return false;
    const uint64_t blocks_per_row = w.in_features / w.block_size;
    if (w.encoding == B2_SCALES_FLOAT32) {
        if ((reinterpret_cast<uintptr_t>(w.fp32_scales) & 15u) != 0 || blocks_per_row % 4 != 0) return false;
    } else {
        if ((reinterpret_cast<uintptr_t>(w.scale_codes) & 15u) != 0 || blocks_per_row % 16 != 0) return false;
        if ((reinterpret_cast<uintptr_t>(w.second_level) & 15u) != 0) return false;
        if (((kTileRows * blocks_per_row) >> w.scale_block_shift) + 5 > static_cast<uint64_t>(kSecondBox)) return false;
    }
    const uint64_t steps = w.in_features / kStepK;
    const uint64_t row_tiles = w.out_features / kTileRows;
    if (steps > 0xFFFFFFull || row_tiles > 0x7FFFFFFull || w.out_features > 0x7FFFFFFFull) return false;
    if ((w.out_features + 2048) * (blocks_per_row + 1) + w.flat_block_base > 0xFFFFFFFFull) return false;
    const uint64_t cap = 64;   // steps one CTA covers (16 warps x 4)
    uint64_t ks = (steps + cap - 1) / cap;
    if (ks > 8) return false;
    uint64_t per = (steps + ks - 1) / ks;
    per = (per + 3) / 4 * 4;
    if (per > cap) return false;
    uint32_t active = 0;
    if (active_clusters_for(ctx, rows, static_cast<uint32_t>(ks), &active) != B2_STATUS_OK) {
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
    const uint64_t blocks_per_row = w.in_features / w.block_size;
    CUtensorMap map_w, map_s, map_2;
    {
        const cuuint64_t dims[2] = {w.in_features / 2, w.out_features};
        const cuuint64_t strides[1] = {w.in_features / 2};
        const cuuint32_t box[2] = {128, kTileRows};
        B2_TRY(encode("codes", &map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w.codes, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B));
    }
    if (w.encoding == B2_SCALES_FLOAT32) {
        const cuuint64_t dims[2] = {blocks_per_row, w.out_features};
        const cuuint64_t strides[1] = {blocks_per_row * 4};
        const cuuint32_t box[2] = {kScaleBoxF32, kTileRows};
        B2_TRY(encode("fp32 scales", &map_s, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, w.fp32_scales, dims, strides, box,
                      CU_TENSOR_MAP_SWIZZLE_NONE));
        map_2 = map_s;   // never used for this encoding
    } else {
        const cuuint64_t dims[2] = {blocks_per_row, w.out_features};
        const cuuint64_t strides[1] = {blocks_per_row};
        const cuuint32_t box[2] = {kScaleBoxU8, kTileRows};
        B2_TRY(encode("scale codes", &map_s, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w.scale_codes, dims, strides, box,
                      CU_TENSOR_MAP_SWIZZLE_NONE));
        // second-level values this view's blocks refer to: indices [0, last] of the shared array
        const uint64_t last = (w.flat_block_base + w.out_features * blocks_per_row - 1) >> w.scale_block_shift;
        const cuuint64_t dims2[1] = {last + 1};
        const cuuint64_t strides2[1] = {0};   // rank 1 has no strides; the pointer must still be valid
        const cuuint32_t box2[1] = {kSecondBox};
        B2_TRY(encode("second-level", &map_2, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 1, w.second_level, dims2, strides2, box2,
                      CU_TENSOR_MAP_SWIZZLE_NONE));
    }
    TmaParams p;
    p.w = w;
    p.x = x;
    p.y = y;
    p.rows = static_cast<uint32_t>(rows);
    p.steps_total = static_cast<uint32_t>(w.in_features / kStepK);
    p.steps_per_cta = steps_per_cta;
    p.row_tiles = static_cast<uint32_t>(w.out_features / kTileRows);
    p.blocks_per_row = static_cast<uint32_t>(blocks_per_row);
    p.lut = ctx.gemv_lut;
    p.error = ctx.gemm_error;
    if (rows <= 8) return launch_tma<1>(ctx, map_w, map_s, map_2, p, ksplit, stream);
    return launch_tma<2>(ctx, map_w, map_s, map_2, p, ksplit, stream);
}

}  // namespace b2
