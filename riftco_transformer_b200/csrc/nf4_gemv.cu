// Decode-path packed-NF4 linear (rows <= 32): y[r,o] = sum_i x[r,i] * W[o,i].
//
// The kernel is bound by the HBM read of the packed codes and scales
// (0.5 B + scale bytes per weight); activations and outputs are a few hundred
// KB and stay in L2. Design:
//  * W is the 16-row A operand of mma.sync m16n8k16 (fp16 in, FP32 accumulate),
//    the batch rows are the 8-wide N operand, so one tensor instruction covers
//    256 weights for up to 8 batch rows and the CUDA cores only decode.
//  * Each thread loads 8 packed bytes (16 consecutive weights) of two weight
//    rows per 64-weight step: a warp request is eight full 32-byte sectors.
//  * A packed byte becomes two fp16 codebook values with ONE shared-memory
//    load: the 256-entry byte table is replicated for the 32 lanes (entry v of
//    lane l at byte v*256 + 4*l), which makes every lookup conflict-free, and
//    its address is formed by a single PRMT from the packed word and 4*lane.
//  * The 64 weights of a step share one block scale, so the four MMAs of a
//    step accumulate unscaled codebook products and the FP32 block scale is
//    applied once to the partial sum (acc += scale * partial).
//  * The contraction is split over warps of a CTA and over the CTAs of a
//    thread-block cluster; partial sums are combined through (distributed)
//    shared memory in a fixed order, so results are deterministic.
// Reference loop: src/core/backend/nn/quantized_linear/reference/operations.cpp:49-81.
#include "b2_common.cuh"
#include "b2_kernels.h"

#include <cooperative_groups.h>
#include <cuda_fp16.h>

#include <cstdlib>

namespace cg = cooperative_groups;

namespace b2 {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kStepK = 64;            // weights per step (one scale block or a part of one)
// Steps of activations staged in shared memory at once (per batch-tile count).
template <int MT> constexpr int chunk_steps_for() { return MT >= 4 ? 16 : 32; }
constexpr int kXRowHalves = 72;       // 64 fp16 + 8 of padding: conflict-free 128-bit reads
constexpr int kLutBytes = 256 * 256;  // byte table, 256-byte stride, 128 bytes used per row
constexpr int kUnit = 4;              // steps whose loads are in flight together per warp

struct GemvParams {
    WeightView w;
    const float* x;
    float* y;
    uint32_t rows;           // batch rows M
    uint32_t steps_total;    // in_features / 64
    uint32_t steps_per_cta;  // contraction slice of one cluster rank
    uint32_t row_tiles;      // ceil(out / (16 * WR))
    const uint32_t* lut;
};

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint2 ldg_stream_u2(const uint8_t* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];\n"
                 : "=r"(v.x), "=r"(v.y)
                 : "l"(p));
    return v;
}

// Shared memory carve-up (dynamic): [lut 64 KB][x chunk][scales][reduction].
template <int MT, int WR>
struct Smem {
    static constexpr int kChunkSteps = chunk_steps_for<MT>();
    static constexpr int kRowsTile = 16 * WR;
    static constexpr int kWK = kWarps / WR;
    static constexpr int kXBytes = kChunkSteps * 8 * MT * kXRowHalves * 2;
    static constexpr int kScaleBytes = kRowsTile * kChunkSteps * 4;
    static constexpr int kRedBytes = kWK * kRowsTile * 8 * MT * 4;
    static constexpr int kOutBytes = kRowsTile * 8 * MT * 4;
    static constexpr int kXOff = kLutBytes;
    static constexpr int kScaleOff = kXOff + kXBytes;
    static constexpr int kRedOff = kScaleOff + kScaleBytes;
    static constexpr int kOutOff = kRedOff + kRedBytes;
    static constexpr int kTotal = kOutOff + kOutBytes;
};

template <int MT, int WR>
__global__ void __launch_bounds__(kThreads, 1) nf4_gemv_kernel(const GemvParams p) {
    using S = Smem<MT, WR>;
    constexpr int WK = S::kWK;
    constexpr int NB = 8 * MT;  // padded batch rows
    constexpr int kChunkSteps = S::kChunkSteps;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint8_t* s_lut = smem;
    __half* s_x = reinterpret_cast<__half*>(smem + S::kXOff);
    float* s_scale = reinterpret_cast<float*>(smem + S::kScaleOff);
    float* s_red = reinterpret_cast<float*>(smem + S::kRedOff);
    float* s_out = reinterpret_cast<float*>(smem + S::kOutOff);

    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t ksplit = cluster.num_blocks();
    const uint32_t krank = cluster.block_rank();

    const uint32_t tid = threadIdx.x;
    const uint32_t lane = tid & 31u, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t wr = warp % WR, wk = warp / WR;
    const uint32_t lane4 = lane * 4u;

    const WeightView& w = p.w;
    const uint64_t in = w.in_features, out = w.out_features;
    const uint64_t row_bytes = in >> 1;

    // Contraction slice of this cluster rank.
    const uint32_t step_begin = min(krank * p.steps_per_cta, p.steps_total);
    const uint32_t step_end = min(step_begin + p.steps_per_cta, p.steps_total);

    // ---- prologue: byte table into shared memory (used 128 B of each row) ----
    for (uint32_t i = tid; i < 256 * 8; i += kThreads) {
        const uint32_t row = i >> 3, part = i & 7u;
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(p.lut) + row * 16 + part);
        *reinterpret_cast<uint4*>(smem + row * 256 + part * 16) = v;
    }

    // Row tiles are handed out round-robin over the clusters of the grid.
    const uint32_t cluster_id = blockIdx.x / ksplit;
    const uint32_t n_clusters = gridDim.x / ksplit;

    for (uint32_t tile = cluster_id; tile < p.row_tiles; tile += n_clusters) {
        const uint64_t row0 = static_cast<uint64_t>(tile) * S::kRowsTile;
        // Rows of this warp's two 8-row halves, clamped for loads.
        const uint64_t rA = min(row0 + wr * 16 + g, out - 1);
        const uint64_t rB = min(row0 + wr * 16 + g + 8, out - 1);
        const uint8_t* codeA = w.codes + rA * row_bytes + t * 8;
        const uint8_t* codeB = w.codes + rB * row_bytes + t * 8;

        float acc[MT][4];
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[m][e] = 0.0f;

        for (uint32_t chunk0 = step_begin; chunk0 < step_end; chunk0 += kChunkSteps) {
            const uint32_t chunk_steps = min(static_cast<uint32_t>(kChunkSteps), step_end - chunk0);
            // Steps of this warp inside the chunk: wk, wk + WK, ...
            const uint32_t my_steps = chunk_steps > wk ? (chunk_steps - wk + WK - 1) / WK : 0;

            // Issue the first unit's code loads before the staging work.
            uint2 curA[kUnit], curB[kUnit];
#pragma unroll
            for (int u = 0; u < kUnit; ++u) {
                const uint32_t s = wk + u * WK;
                if (static_cast<uint32_t>(u) < my_steps) {
                    const uint64_t off = static_cast<uint64_t>(chunk0 + s) * 32;
                    curA[u] = ldg_stream_u2(codeA + off);
                    curB[u] = ldg_stream_u2(codeB + off);
                } else {
                    curA[u] = make_uint2(0x77777777u, 0x77777777u);
                    curB[u] = curA[u];
                }
            }

            __syncthreads();  // previous chunk / tile finished with s_x and s_scale
            // Activations of the chunk -> fp16 [step][batch row][64 (+8 pad)].
            {
                const uint32_t quads = chunk_steps * 16;  // float4 per batch row
                for (uint32_t i = tid; i < quads * NB; i += kThreads) {
                    const uint32_t n = i / quads, q4 = i % quads;
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (n < p.rows) {
                        v = __ldg(reinterpret_cast<const float4*>(
                            p.x + static_cast<uint64_t>(n) * in +
                            static_cast<uint64_t>(chunk0) * kStepK + q4 * 4));
                    }
                    const uint32_t s = q4 >> 4, c = (q4 & 15u) * 4;
                    __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
                    uint2 packed;
                    packed.x = *reinterpret_cast<uint32_t*>(&lo);
                    packed.y = *reinterpret_cast<uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(s_x + (s * NB + n) * kXRowHalves + c) = packed;
                }
            }
            // Decoded block scales of the tile's rows for the chunk.
            for (uint32_t i = tid; i < S::kRowsTile * chunk_steps; i += kThreads) {
                const uint32_t r = i / chunk_steps, s = i % chunk_steps;
                const uint64_t row = min(row0 + r, out - 1);
                const uint64_t flat = row * in + static_cast<uint64_t>(chunk0 + s) * kStepK;
                s_scale[r * kChunkSteps + s] = decode_block_scale(w, flat >> w.block_shift);
            }
            __syncthreads();

            for (uint32_t u0 = 0; u0 < my_steps; u0 += kUnit) {
                // Prefetch the next unit while this one is consumed.
                uint2 nxtA[kUnit], nxtB[kUnit];
#pragma unroll
                for (int u = 0; u < kUnit; ++u) {
                    const uint32_t idx = u0 + kUnit + u;
                    if (idx < my_steps) {
                        const uint64_t off = static_cast<uint64_t>(chunk0 + wk + idx * WK) * 32;
                        nxtA[u] = ldg_stream_u2(codeA + off);
                        nxtB[u] = ldg_stream_u2(codeB + off);
                    } else {
                        nxtA[u] = make_uint2(0x77777777u, 0x77777777u);
                        nxtB[u] = nxtA[u];
                    }
                }
#pragma unroll
                for (int u = 0; u < kUnit; ++u) {
                    const uint32_t idx = u0 + u;
                    if (idx < my_steps) {
                        const uint32_t s = wk + idx * WK;
                        const uint32_t wa[2] = {curA[u].x, curA[u].y};
                        const uint32_t wb[2] = {curB[u].x, curB[u].y};
                        float part[MT][4];
#pragma unroll
                        for (int m = 0; m < MT; ++m)
#pragma unroll
                            for (int e = 0; e < 4; ++e) part[m][e] = 0.0f;
                        uint4 xf[MT][2];
#pragma unroll
                        for (int m = 0; m < MT; ++m) {
                            const __half* xp = s_x + (s * NB + m * 8 + g) * kXRowHalves + t * 16;
                            xf[m][0] = *reinterpret_cast<const uint4*>(xp);
                            xf[m][1] = *reinterpret_cast<const uint4*>(xp + 8);
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const uint32_t word_a = wa[i >> 1], word_b = wb[i >> 1];
                            const uint32_t sel0 = (i & 1) ? 0x5524u : 0x5504u;
                            const uint32_t sel1 = (i & 1) ? 0x5534u : 0x5514u;
                            const uint32_t a0 = *reinterpret_cast<const uint32_t*>(
                                s_lut + __byte_perm(word_a, lane4, sel0));
                            const uint32_t a2 = *reinterpret_cast<const uint32_t*>(
                                s_lut + __byte_perm(word_a, lane4, sel1));
                            const uint32_t a1 = *reinterpret_cast<const uint32_t*>(
                                s_lut + __byte_perm(word_b, lane4, sel0));
                            const uint32_t a3 = *reinterpret_cast<const uint32_t*>(
                                s_lut + __byte_perm(word_b, lane4, sel1));
#pragma unroll
                            for (int m = 0; m < MT; ++m) {
                                const uint4& xv = xf[m][i >> 1];
                                const uint32_t b0 = (i & 1) ? xv.z : xv.x;
                                const uint32_t b1 = (i & 1) ? xv.w : xv.y;
                                mma_f16_16816(part[m], a0, a1, a2, a3, b0, b1);
                            }
                        }
                        const float sA = s_scale[(wr * 16 + g) * kChunkSteps + s];
                        const float sB = s_scale[(wr * 16 + g + 8) * kChunkSteps + s];
#pragma unroll
                        for (int m = 0; m < MT; ++m) {
                            acc[m][0] = fmaf(sA, part[m][0], acc[m][0]);
                            acc[m][1] = fmaf(sA, part[m][1], acc[m][1]);
                            acc[m][2] = fmaf(sB, part[m][2], acc[m][2]);
                            acc[m][3] = fmaf(sB, part[m][3], acc[m][3]);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < kUnit; ++u) {
                    curA[u] = nxtA[u];
                    curB[u] = nxtB[u];
                }
            }
        }

        // ---- combine the WK warps of the CTA (fixed order) ----
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float* dst = s_red + (wk * S::kRowsTile + wr * 16) * NB + m * 8;
            dst[g * NB + 2 * t] = acc[m][0];
            dst[g * NB + 2 * t + 1] = acc[m][1];
            dst[(g + 8) * NB + 2 * t] = acc[m][2];
            dst[(g + 8) * NB + 2 * t + 1] = acc[m][3];
        }
        __syncthreads();
        for (uint32_t i = tid; i < S::kRowsTile * NB; i += kThreads) {
            float v = 0.0f;
#pragma unroll
            for (int k = 0; k < WK; ++k) v += s_red[k * S::kRowsTile * NB + i];
            s_out[i] = v;
        }

        // ---- combine the ranks of the cluster through distributed shared memory ----
        if (ksplit > 1) {
            cluster.sync();
        } else {
            __syncthreads();
        }
        // Element i = n * rows_tile + r so that consecutive threads write
        // consecutive output columns of one batch row.
        for (uint32_t i = tid + krank * kThreads; i < S::kRowsTile * NB; i += kThreads * ksplit) {
            const uint32_t n = i / S::kRowsTile, r = i % S::kRowsTile;
            float v = 0.0f;
            for (uint32_t k = 0; k < ksplit; ++k) {
                const float* remote = ksplit > 1 ? cluster.map_shared_rank(s_out, k) : s_out;
                v += remote[r * NB + n];
            }
            if (n < p.rows && row0 + r < out) p.y[static_cast<uint64_t>(n) * out + row0 + r] = v;
        }
        if (ksplit > 1) cluster.sync();  // peers may still be reading this CTA's s_out
    }
}

__global__ void gemv_lut_init_kernel(uint32_t* lut) {
    // 256 rows x 64 words; words 0..31 of row v hold the fp16 pair of byte v.
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= 256 * 64) return;
    const uint32_t v = i >> 6, word = i & 63u;
    uint32_t value = 0;
    if (word < 32) {
        const __half lo = __float2half_rn(kNf4Codebook[v & 15u]);
        const __half hi = __float2half_rn(kNf4Codebook[v >> 4]);
        value = static_cast<uint32_t>(__half_as_ushort(lo)) |
                (static_cast<uint32_t>(__half_as_ushort(hi)) << 16);
    }
    lut[i] = value;
}

template <int MT, int WR>
int32_t launch_config(const DeviceContext& ctx, GemvParams p, uint32_t ksplit, cudaStream_t stream) {
    using S = Smem<MT, WR>;
    auto kernel = nf4_gemv_kernel<MT, WR>;
    B2_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
    p.row_tiles = static_cast<uint32_t>((p.w.out_features + S::kRowsTile - 1) / S::kRowsTile);
    uint32_t clusters = static_cast<uint32_t>(ctx.sm_count) / ksplit;
    if (clusters > p.row_tiles) clusters = p.row_tiles;
    if (clusters == 0) clusters = 1;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(clusters * ksplit);
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
    B2_CUDA_TRY(cudaLaunchKernelEx(&config, kernel, p));
    return B2_STATUS_OK;
}

template <int MT>
int32_t launch_mt(const DeviceContext& ctx, const GemvParams& p, uint32_t wr, uint32_t ksplit,
                  cudaStream_t stream) {
    switch (wr) {
    case 1: return launch_config<MT, 1>(ctx, p, ksplit, stream);
    case 2: return launch_config<MT, 2>(ctx, p, ksplit, stream);
    case 4: return launch_config<MT, 4>(ctx, p, ksplit, stream);
    default: return launch_config<MT, 8>(ctx, p, ksplit, stream);
    }
}

}  // namespace

int32_t init_gemv_lut(DeviceContext* ctx) {
    B2_CUDA_TRY(cudaMalloc(&ctx->gemv_lut, kLutBytes));
    gemv_lut_init_kernel<<<64, 256>>>(ctx->gemv_lut);
    B2_CUDA_TRY(cudaGetLastError());
    B2_CUDA_TRY(cudaDeviceSynchronize());
    return B2_STATUS_OK;
}

bool nf4_gemv_supported(const WeightView& w, const float* x, const float* y, uint64_t rows) {
    (void)y;
    return rows >= 1 && rows <= 32 && w.in_features % kStepK == 0 && w.block_size >= kStepK &&
           (reinterpret_cast<uintptr_t>(w.codes) & 7u) == 0 &&
           (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && w.in_features / kStepK <= 0xFFFFFFFFull &&
           w.out_features <= 0x7FFFFFFFull;
}

// Tunable through the environment for experiments: B2_GEMV_WR (rows per CTA /
// 16) and B2_GEMV_KSPLIT (cluster size along the contraction).
int32_t launch_nf4_gemv(const DeviceContext& ctx, const WeightView& w, const float* x, float* y,
                        uint64_t rows, cudaStream_t stream) {
    GemvParams p;
    p.w = w;
    p.x = x;
    p.y = y;
    p.rows = static_cast<uint32_t>(rows);
    p.steps_total = static_cast<uint32_t>(w.in_features / kStepK);
    p.lut = ctx.gemv_lut;
    p.row_tiles = 0;

    // One chunk (32 steps = 2048 inputs) per cluster rank where the cluster
    // limit of 8 allows it; longer contractions take several chunks per rank.
    const uint32_t chunk = rows > 16 ? chunk_steps_for<4>() : chunk_steps_for<1>();
    uint32_t ksplit = (p.steps_total + chunk - 1) / chunk;
    if (ksplit > 8) ksplit = 8;
    if (ksplit < 1) ksplit = 1;
    // Rows per CTA: as large as still leaves every SM at least one tile.
    uint32_t wr = 8;
    while (wr > 1 && (w.out_features + 16 * wr - 1) / (16 * wr) * ksplit <
                         static_cast<uint64_t>(ctx.sm_count)) {
        wr >>= 1;
    }
    static const char* env_wr = getenv("B2_GEMV_WR");
    static const char* env_ks = getenv("B2_GEMV_KSPLIT");
    if (env_wr != nullptr) {
        const int v = atoi(env_wr);
        if (v == 1 || v == 2 || v == 4 || v == 8) wr = static_cast<uint32_t>(v);
    }
    if (env_ks != nullptr) {
        const int v = atoi(env_ks);
        if (v >= 1 && v <= 8) ksplit = static_cast<uint32_t>(v);
    }
    p.steps_per_cta = (p.steps_total + ksplit - 1) / ksplit;

    if (rows <= 8) return launch_mt<1>(ctx, p, wr, ksplit, stream);
    if (rows <= 16) return launch_mt<2>(ctx, p, wr, ksplit, stream);
    return launch_mt<4>(ctx, p, wr, ksplit, stream);
}

}  // namespace b2
