// Streaming decode kernel for the packed-NF4 linear, batch rows <= 16:
// y[r,o] = sum_i x[r,i] * W[o,i].
//
// Bound by the HBM read of the packed weight (0.5 B per weight + scales). A
// decode GEMV lasts a few microseconds, i.e. a handful of DRAM round trips, so
// the kernel is organised to expose exactly one of them:
//  * one persistent 16-warp CTA per SM; a cluster of `ksplit` CTAs shares a row
//    range and splits the contraction, each CTA keeping a fixed slice of it;
//  * warp w owns SPW consecutive 64-weight steps of that slice for the whole
//    kernel, so its activations are converted to fp16 once and stay in
//    REGISTERS as mma.sync B fragments;
//  * the CTA walks 16-row weight tiles; the packed codes and raw scale bytes of
//    the next D tiles are already in flight in registers while a tile is
//    multiplied (software pipeline, 64 KB in flight per SM);
//  * a packed byte becomes two fp16 codebook values with one conflict-free
//    shared-memory load (table replicated per lane, address formed by one
//    PRMT); the FP32 block scale is applied to the 64-weight partial sum;
//  * the 16 warps' partial sums meet in shared memory once per tile (one
//    barrier, double-buffered), the cluster ranks' sums meet once per kernel
//    through distributed shared memory, both in a fixed order (deterministic).
// Reference loop: src/core/backend/nn/quantized_linear/reference/operations.cpp:49-81.
#include "b2_common.cuh"
#include "b2_kernels.h"

#include <cooperative_groups.h>
#include <cuda_fp16.h>

#include <cstdlib>

namespace cg = cooperative_groups;

namespace b2 {
namespace {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kStepK = 64;
constexpr int kTileRows = 16;
constexpr int kLutBytes = 256 * 256;   // 256-byte row stride, bytes [0,128) used
constexpr int kMaxTilesPerCluster = 48;

struct StreamParams {
    WeightView w;
    const float* x;
    float* y;
    uint32_t rows;            // batch rows M
    uint32_t steps_total;     // in / 64
    uint32_t steps_per_cta;   // <= 16 * SPW
    uint32_t row_tiles;       // ceil(out / 16)
    uint32_t tiles_per_cluster;
    const uint32_t* lut;      // compact [256][32] words
    uint32_t blocks_per_row;  // in / block_size when the rows are block aligned, else 0
};

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// First MMA of a chain: D = A*B with a zero C operand, so no register has to be cleared.
__device__ __forceinline__ void mma_f16_16816_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                   uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%10,%10,%10,%10};\n"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

__device__ __forceinline__ uint2 ldg_stream_u2(const uint8_t* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];\n"
                 : "=r"(v.x), "=r"(v.y)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(gmem_src));
}

// Dynamic shared memory: the byte table sits at the first 64 KB-aligned shared
// address (so that a lookup address is assembled by one PRMT: byte 0 = 4*lane,
// byte 1 = packed byte, bytes 2-3 = table base), everything else follows it.
template <int MT>
struct Smem {
    static constexpr int NB = 8 * MT;
    static constexpr int kRedBytes = 2 * kWarps * kTileRows * NB * 4;           // two parities
    static constexpr int kOutBytes = kMaxTilesPerCluster * kTileRows * NB * 4;  // per-tile sums
    // offsets from the table base
    static constexpr int kFactorOff = kLutBytes;                                // 256 floats
    static constexpr int kRedOff = kFactorOff + 1024;
    static constexpr int kOutOff = kRedOff + kRedBytes;
    static constexpr int kTotal = 65536 /* alignment slack */ + kOutOff + kOutBytes;
};

// Raw (undecoded) scale data of one (row, step) pair.
struct RawScale {
    uint32_t bits;   // FP32 scale bits, or the 8-bit scale code
    float second;    // second-level scale (double-quantised only)
};

__device__ __forceinline__ uint32_t lds_u32(uint32_t shared_addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(shared_addr));
    return v;
}

template <int MT, int SPW>
__global__ void __launch_bounds__(kThreads, 1) nf4_gemv_stream_kernel(const StreamParams p) {
    using S = Smem<MT>;
    constexpr int NB = S::NB;
    constexpr int D = 8 / SPW;            // tiles in flight
    constexpr int NSC = (2 * SPW) / 4;    // scales decoded per lane per tile (2 rows x SPW steps over 4 lanes)
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t raw32 = static_cast<uint32_t>(__cvta_generic_to_shared(smem_raw));
    const uint32_t lut32 = (raw32 + 65535u) & ~65535u;
    uint8_t* smem = smem_raw + (lut32 - raw32);                       // table base, generic pointer
    const float* s_factor = reinterpret_cast<const float*>(smem + S::kFactorOff);
    float* s_red = reinterpret_cast<float*>(smem + S::kRedOff);      // [2][16 warps][16 rows][NB]
    float* s_out = reinterpret_cast<float*>(smem + S::kOutOff);      // [tile][16 rows][NB]

    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t ksplit = cluster.num_blocks();
    const uint32_t krank = cluster.block_rank();
    const uint32_t cluster_id = blockIdx.x / ksplit;
    const uint32_t n_clusters = gridDim.x / ksplit;

    const uint32_t tid = threadIdx.x;
    const uint32_t lane = tid & 31u, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t lut_lane = lut32 | (lane * 4u);   // bytes 2-3: table base, byte 0: 4*lane
    const uint32_t quad_base = lane & ~3u;

    const WeightView& w = p.w;
    const uint64_t in = w.in_features, out = w.out_features;
    const uint64_t row_bytes = in >> 1;

    // Steps of this warp: SPW consecutive steps of the CTA's slice. A warp whose
    // range is cut by the end of the slice re-reads its last valid step with zero
    // activations instead of branching per step.
    const uint32_t slice_begin = min(krank * p.steps_per_cta, p.steps_total);
    const uint32_t slice_end = min(slice_begin + p.steps_per_cta, p.steps_total);
    const uint32_t step0 = slice_begin + warp * SPW;
    const uint32_t my_steps = step0 < slice_end ? min(static_cast<uint32_t>(SPW), slice_end - step0) : 0u;
    const bool warp_active = my_steps > 0;   // warp-uniform
    const uint32_t my_tiles =
        cluster_id < p.row_tiles ? (p.row_tiles - cluster_id + n_clusters - 1) / n_clusters : 0u;

    // (row half, step) whose scale this lane decodes, NSC per tile:
    //   SPW == 4: lane t decodes step t of rows g and g+8 (NSC = 2, k = row half)
    //   SPW == 2: lane t decodes step t&1 of row half t>>1   (NSC = 1)
    const uint32_t scale_step_raw = SPW == 4 ? t : (t & 1u);
    const uint32_t scale_step = warp_active ? min(scale_step_raw, my_steps - 1) : 0u;
    auto scale_row_half = [&](int k) -> uint32_t { return SPW == 4 ? static_cast<uint32_t>(k) : (t >> 1); };

    uint2 wbuf[D][SPW][2];
    RawScale sraw[D][NSC];

    // Running addresses of the next tile to issue (tiles are issued in slot order).
    const uint32_t tile_stride_rows = n_clusters * kTileRows;
    uint32_t next_row = cluster_id * kTileRows;
    const uint8_t* next_code = w.codes + (static_cast<uint64_t>(next_row) + g) * row_bytes +
                               static_cast<uint64_t>(step0) * 32 + t * 8;
    const uint64_t code_stride = static_cast<uint64_t>(tile_stride_rows) * row_bytes;
    const uint64_t half_rows = 8 * row_bytes;
    uint32_t step_off[SPW];   // byte offset of step u (clamped to the warp's last valid step)
#pragma unroll
    for (int u = 0; u < SPW; ++u) step_off[u] = (warp_active ? min(static_cast<uint32_t>(u), my_steps - 1) : 0u) * 32u;
    uint32_t next_block = 0, block_stride = 0;
    const uint32_t blocks_per_row = p.blocks_per_row;
    if (blocks_per_row != 0) {
        next_block = (next_row + g) * blocks_per_row +
                     (((step0 + scale_step) * static_cast<uint32_t>(kStepK)) >> w.block_shift);
        block_stride = tile_stride_rows * blocks_per_row;
    }
    const bool fp32_scales = w.encoding == B2_SCALES_FLOAT32;

    auto issue_tile = [&](int d, uint32_t tile_slot) {
        if (tile_slot < my_tiles && warp_active) {
            const bool whole = next_row + kTileRows <= out;  // all 16 rows exist
            const uint8_t* pa = next_code;
            const uint8_t* pb = next_code + half_rows;
            if (!whole) {
                const uint64_t rA = min(static_cast<uint64_t>(next_row) + g, out - 1);
                const uint64_t rB = min(static_cast<uint64_t>(next_row) + g + 8, out - 1);
                pa = w.codes + rA * row_bytes + static_cast<uint64_t>(step0) * 32 + t * 8;
                pb = w.codes + rB * row_bytes + static_cast<uint64_t>(step0) * 32 + t * 8;
            }
#pragma unroll
            for (int u = 0; u < SPW; ++u) {
                wbuf[d][u][0] = ldg_stream_u2(pa + step_off[u]);
                wbuf[d][u][1] = ldg_stream_u2(pb + step_off[u]);
            }
#pragma unroll
            for (int k = 0; k < NSC; ++k) {
                uint64_t block;
                if (whole && blocks_per_row != 0) {
                    block = next_block + (scale_row_half(k) ? 8u * blocks_per_row : 0u);
                } else {
                    const uint64_t row = min(static_cast<uint64_t>(next_row) + g + 8 * scale_row_half(k), out - 1);
                    block = (row * in + static_cast<uint64_t>(step0 + scale_step) * kStepK) >> w.block_shift;
                }
                if (fp32_scales) {
                    sraw[d][k].bits = __float_as_uint(__ldg(w.fp32_scales + block));
                    sraw[d][k].second = 0.0f;
                } else {
                    sraw[d][k].bits = __ldg(w.scale_codes + block);
                    sraw[d][k].second = __ldg(w.second_level + ((w.flat_block_base + block) >> w.scale_block_shift));
                }
            }
        }
        next_row += tile_stride_rows;
        next_code += code_stride;
        next_block += block_stride;
    };

    // ---- prologue: get everything in flight at once ----
#pragma unroll
    for (int d = 0; d < D; ++d) issue_tile(d, d);

    for (uint32_t i = tid; i < 256 * 8; i += kThreads) {
        cp_async_16(smem + (i >> 3) * 256 + (i & 7u) * 16, p.lut + i * 4);
    }
    asm volatile("cp.async.commit_group;\n" ::);
    if (tid < 256) reinterpret_cast<float*>(smem + S::kFactorOff)[tid] = dq_factor(tid);

    // Activations of this warp's steps as fp16 B fragments: batch row g (+8 per
    // tile m), weights 16t .. 16t+15 of each step; zero for steps past the slice.
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

    asm volatile("cp.async.wait_group 0;\n" ::);
    __syncthreads();

    // ---- main loop over this cluster's tiles, D at a time (static buffer indices) ----
    uint32_t parity = 0;
    for (uint32_t base = 0; base < my_tiles; base += D) {
#pragma unroll
        for (int d = 0; d < D; ++d) {
            const uint32_t slot = base + d;
            if (slot < my_tiles) {  // CTA-uniform
                float acc[MT][4];
#pragma unroll
                for (int m = 0; m < MT; ++m)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[m][e] = 0.0f;
                if (warp_active) {
                    float sc[NSC];
#pragma unroll
                    for (int k = 0; k < NSC; ++k) {
                        sc[k] = fp32_scales ? __uint_as_float(sraw[d][k].bits)
                                            : dq_finish(s_factor[sraw[d][k].bits], sraw[d][k].second, w.offset);
                    }
#pragma unroll
                    for (int u = 0; u < SPW; ++u) {
                        // scale of rows g / g+8 at step u, from the lane that decoded it
                        const float sA = __shfl_sync(0xFFFFFFFFu, sc[0], quad_base + u);
                        const float sB = SPW == 4 ? __shfl_sync(0xFFFFFFFFu, sc[NSC - 1], quad_base + u)
                                                  : __shfl_sync(0xFFFFFFFFu, sc[0], quad_base + 2 + u);
                        float part[MT][4];
                        const uint32_t wa[2] = {wbuf[d][u][0].x, wbuf[d][u][0].y};
                        const uint32_t wb[2] = {wbuf[d][u][1].x, wbuf[d][u][1].y};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const uint32_t word_a = wa[i >> 1], word_b = wb[i >> 1];
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
                // refill this buffer with the tile D slots ahead
                issue_tile(d, slot + D);

                // publish this warp's partial tile
                float* red = s_red + (parity * kWarps + warp) * kTileRows * NB;
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    *reinterpret_cast<float2*>(red + g * NB + m * 8 + 2 * t) = make_float2(acc[m][0], acc[m][1]);
                    *reinterpret_cast<float2*>(red + (g + 8) * NB + m * 8 + 2 * t) = make_float2(acc[m][2], acc[m][3]);
                }
                __syncthreads();
                if (tid < kTileRows * NB) {
                    const float* src = s_red + parity * kWarps * kTileRows * NB + tid;
                    float v = 0.0f;
#pragma unroll
                    for (int k = 0; k < kWarps; ++k) v += src[k * kTileRows * NB];
                    s_out[slot * kTileRows * NB + tid] = v;
                }
                parity ^= 1u;
            }
        }
    }

    // ---- combine the cluster ranks (fixed order) and store ----
    if (ksplit > 1) {
        cluster.sync();
    } else {
        __syncthreads();
    }
    const uint32_t total = my_tiles * kTileRows * NB;
    // element e = (slot, n, r): consecutive threads write consecutive output columns
    for (uint32_t e = tid + krank * kThreads; e < total; e += kThreads * ksplit) {
        const uint32_t slot = e / (kTileRows * NB), rem = e % (kTileRows * NB);
        const uint32_t n = rem / kTileRows, r = rem % kTileRows;
        float v = 0.0f;
        for (uint32_t k = 0; k < ksplit; ++k) {
            const float* remote = ksplit > 1 ? cluster.map_shared_rank(s_out, k) : s_out;
            v += remote[slot * kTileRows * NB + r * NB + n];
        }
        const uint64_t row = static_cast<uint64_t>(cluster_id + slot * n_clusters) * kTileRows + r;
        if (n < p.rows && row < out) p.y[static_cast<uint64_t>(n) * out + row] = v;
    }
    if (ksplit > 1) cluster.sync();  // peers may still be reading this CTA's s_out
}

template <int MT, int SPW>
int32_t launch_stream(const DeviceContext& ctx, StreamParams p, uint32_t ksplit, cudaStream_t stream) {
    using S = Smem<MT>;
    auto kernel = nf4_gemv_stream_kernel<MT, SPW>;
    static bool configured = false;
    static int max_clusters[9] = {0};
    if (!configured) {
        B2_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
        configured = true;
    }
    cudaLaunchConfig_t config = {};
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = S::kTotal;
    config.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ksplit;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    if (max_clusters[ksplit] == 0) {
        // How many clusters of this size the device can hold at once (GPC packing).
        config.gridDim = dim3(static_cast<unsigned>(ctx.sm_count / ksplit) * ksplit);
        int n = 0;
        B2_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, kernel, &config));
        max_clusters[ksplit] = n > 0 ? n : 1;
    }
    uint32_t clusters = static_cast<uint32_t>(max_clusters[ksplit]);
    const uint32_t by_sm = static_cast<uint32_t>(ctx.sm_count) / ksplit;
    if (clusters > by_sm) clusters = by_sm;
    if (clusters > p.row_tiles) clusters = p.row_tiles;
    if (clusters == 0) clusters = 1;
    p.tiles_per_cluster = (p.row_tiles + clusters - 1) / clusters;
    if (p.tiles_per_cluster > kMaxTilesPerCluster) {
        return fail(B2_STATUS_RUNTIME_ERROR, "internal: NF4 stream kernel tile budget exceeded");
    }
    config.gridDim = dim3(clusters * ksplit);
    B2_CUDA_TRY(cudaLaunchKernelEx(&config, kernel, p));
    return B2_STATUS_OK;
}

}  // namespace

// Chooses (steps per warp, cluster size) or reports that the shape does not fit.
bool nf4_gemv_stream_plan(const DeviceContext& ctx, const WeightView& w, uint64_t rows, uint32_t* spw_out,
                          uint32_t* ksplit_out) {
    if (rows < 1 || rows > 16 || w.in_features % kStepK != 0 || w.block_size < kStepK) return false;
    const uint64_t steps = w.in_features / kStepK;
    const uint64_t row_tiles = (w.out_features + kTileRows - 1) / kTileRows;
    if (steps > 0xFFFFFFFFull || row_tiles > 0x7FFFFFFull) return false;
    if ((w.out_features + 2048) * (w.in_features / w.block_size + 1) > 0xFFFFFFFFull) return false;  // 32-bit block index
    double best = 0.0;
    uint32_t best_spw = 0, best_ks = 0;
    // Prefer 4 steps per warp: longer contiguous row segments per CTA (DRAM page
    // locality) and half the per-tile bookkeeping per byte; 2 steps per warp
    // only when 4 do not fit (two batch tiles) or waste the machine.
    for (uint32_t spw = 4; spw >= 2; spw -= 2) {
        if (rows > 8 && spw == 4) continue;  // two batch tiles keep activations for 2 steps only
        const uint64_t cap = 16ull * spw;    // steps one CTA covers
        const uint32_t ks = static_cast<uint32_t>((steps + cap - 1) / cap);
        if (ks > 8) continue;
        const uint64_t clusters = static_cast<uint64_t>(ctx.sm_count) / ks;
        if (clusters == 0) continue;
        const uint64_t rounds = (row_tiles + clusters - 1) / clusters;
        if (rounds > static_cast<uint64_t>(kMaxTilesPerCluster)) continue;
        const double balance = static_cast<double>(row_tiles) / static_cast<double>(rounds * clusters);
        const double fill = static_cast<double>(steps) / static_cast<double>(ks * cap);
        const double sm_use = static_cast<double>(clusters * ks) / ctx.sm_count;
        const double score = balance * fill * sm_use * (spw == 4 ? 1.25 : 1.0);
        if (score > best) {
            best = score;
            best_spw = spw;
            best_ks = ks;
        }
    }
    if (best_spw == 0) return false;
    static const char* env_spw = getenv("B2_GEMV_SPW");
    if (env_spw != nullptr) {
        const uint32_t v = static_cast<uint32_t>(atoi(env_spw));
        const uint64_t cap = 16ull * v;
        if ((v == 2 || (v == 4 && rows <= 8)) && (steps + cap - 1) / cap <= 8) {
            best_spw = v;
            best_ks = static_cast<uint32_t>((steps + cap - 1) / cap);
        }
    }
    *spw_out = best_spw;
    *ksplit_out = best_ks;
    return true;
}

int32_t launch_nf4_gemv_stream(const DeviceContext& ctx, const WeightView& w, const float* x, float* y,
                               uint64_t rows, uint32_t spw, uint32_t ksplit, cudaStream_t stream) {
    StreamParams p;
    p.w = w;
    p.x = x;
    p.y = y;
    p.rows = static_cast<uint32_t>(rows);
    p.steps_total = static_cast<uint32_t>(w.in_features / kStepK);
    p.steps_per_cta = (p.steps_total + ksplit - 1) / ksplit;
    p.row_tiles = static_cast<uint32_t>((w.out_features + kTileRows - 1) / kTileRows);
    p.tiles_per_cluster = 0;
    p.lut = ctx.gemv_lut;
    p.blocks_per_row = w.in_features % w.block_size == 0 ? static_cast<uint32_t>(w.in_features / w.block_size) : 0u;
    if (rows <= 8) {
        return spw == 4 ? launch_stream<1, 4>(ctx, p, ksplit, stream) : launch_stream<1, 2>(ctx, p, ksplit, stream);
    }
    return launch_stream<2, 2>(ctx, p, ksplit, stream);
}

}  // namespace b2
