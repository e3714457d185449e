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
constexpr int kStepK = 64;    // weights per step; a step never straddles a scale block
constexpr int kWR = 2;        // warp rows: each warp owns 32 weight rows (two MMA row groups)
constexpr int kWK = 4;        // warps that split the contraction inside a CTA
constexpr int kRowsTile = 64; // weight rows per CTA
constexpr int kLutBytes = 256 * 256;

// Steps staged per chunk: the fp16 activations of a chunk live in the unused
// upper half of the 256 table rows (one 128-byte row per (step, batch row)).
template <int MT> constexpr int chunk_steps_for() { return 256 / (8 * MT); }

struct GemvParams {
    WeightView w;
    const float* x;
    float* y;
    uint32_t rows;           // batch rows M
    uint32_t steps_total;    // in_features / 64
    uint32_t steps_per_cta;  // contraction slice of one cluster rank
    const uint32_t* lut;     // compact [256][32] words
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

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(gmem_src));
}

// Shared memory (dynamic): 64 KB of 256-byte rows - bytes [0,128) of row v are
// the byte table entry v for the 32 lanes, bytes [128,256) of row h hold the
// 64 fp16 activations of (step, batch row) h - then scales / reduction scratch.
template <int MT>
struct Smem {
    static constexpr int kChunkSteps = chunk_steps_for<MT>();
    static constexpr int kScaleBytes = kRowsTile * (kChunkSteps + 1) * 4;  // +1: rows land in different banks
    static constexpr int kRedBytes = kWK * kRowsTile * 8 * MT * 4;
    static constexpr int kScratchBytes = kScaleBytes > kRedBytes ? kScaleBytes : kRedBytes;
    static constexpr int kOutBytes = kRowsTile * 8 * MT * 4;
    static constexpr int kScratchOff = kLutBytes;
    static constexpr int kOutOff = kScratchOff + kScratchBytes;
    static constexpr int kTotal = kOutOff + kOutBytes;
};

template <int MT>
__global__ void __launch_bounds__(kThreads, 2) nf4_gemv_kernel(const GemvParams p) {
    using S = Smem<MT>;
    constexpr int NB = 8 * MT;                      // padded batch rows
    constexpr int CH = S::kChunkSteps;              // steps per chunk
    constexpr int SPW = CH / kWK;                   // steps per warp per chunk
    extern __shared__ __align__(1024) uint8_t smem[];
    float* s_scale = reinterpret_cast<float*>(smem + S::kScratchOff);  // [64][CH]
    float* s_red = reinterpret_cast<float*>(smem + S::kScratchOff);    // aliases s_scale after compute
    float* s_out = reinterpret_cast<float*>(smem + S::kOutOff);

    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t ksplit = cluster.num_blocks();
    const uint32_t krank = cluster.block_rank();

    const uint32_t tid = threadIdx.x;
    const uint32_t lane = tid & 31u, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t wr = warp % kWR, wk = warp / kWR;
    const uint32_t lane4 = lane * 4u;

    const WeightView& w = p.w;
    const uint64_t in = w.in_features, out = w.out_features;
    const uint64_t row_bytes = in >> 1;
    const uint32_t step_begin = min(krank * p.steps_per_cta, p.steps_total);
    const uint32_t step_end = min(step_begin + p.steps_per_cta, p.steps_total);
    const uint64_t row0 = static_cast<uint64_t>(blockIdx.x / ksplit) * kRowsTile;

    // The four weight rows of this thread (two MMA row groups), clamped for loads.
    const uint8_t* code_ptr[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint64_t r = min(row0 + wr * 32 + g + 8 * j, out - 1);
        code_ptr[j] = w.codes + r * row_bytes + t * 8;
    }

    float acc[2][MT][4];
#pragma unroll
    for (int rg = 0; rg < 2; ++rg)
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[rg][m][e] = 0.0f;

    // Byte table: 8 x 16 B per thread, asynchronously.
    for (uint32_t i = tid; i < 256 * 8; i += kThreads) {
        cp_async_16(smem + (i >> 3) * 256 + (i & 7u) * 16, p.lut + i * 4);
    }
    asm volatile("cp.async.commit_group;\n" ::);

    for (uint32_t chunk0 = step_begin; chunk0 < step_end; chunk0 += CH) {
        const uint32_t chunk_steps = min(static_cast<uint32_t>(CH), step_end - chunk0);

        // 1. All packed-code loads of the chunk: SPW steps x 4 rows x 8 B per thread.
        uint2 code[SPW][4];
#pragma unroll
        for (int u = 0; u < SPW; ++u) {
            const uint32_t s = wk + u * kWK;
            const uint64_t off = static_cast<uint64_t>(chunk0 + min(s, chunk_steps - 1)) * 32;
#pragma unroll
            for (int j = 0; j < 4; ++j) code[u][j] = ldg_stream_u2(code_ptr[j] + off);
        }

        __syncthreads();  // previous chunk done with activations / scales

        // 2. Activations of the chunk -> fp16 in the upper halves of the table rows.
        {
            constexpr int kQuads = CH * 16 * NB;            // float4 of a full chunk
            constexpr int kPerThread = kQuads / kThreads;   // 16 for every MT
            constexpr int kBatch = 8;                       // loads in flight per pass
#pragma unroll
            for (int k0 = 0; k0 < kPerThread; k0 += kBatch) {
                float4 v[kBatch];
#pragma unroll
                for (int k = 0; k < kBatch; ++k) {
                    const uint32_t i = tid + (k0 + k) * kThreads;
                    const uint32_t n = i / (CH * 16), q4 = i % (CH * 16);
                    v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (n < p.rows && (q4 >> 4) < chunk_steps) {
                        v[k] = __ldg(reinterpret_cast<const float4*>(
                            p.x + static_cast<uint64_t>(n) * in + static_cast<uint64_t>(chunk0) * kStepK + q4 * 4));
                    }
                }
#pragma unroll
                for (int k = 0; k < kBatch; ++k) {
                    const uint32_t i = tid + (k0 + k) * kThreads;
                    const uint32_t n = i / (CH * 16), q4 = i % (CH * 16);
                    const uint32_t s = q4 >> 4, c4 = q4 & 15u;       // c4: group of 4 halves (8 B)
                    const uint32_t chunk16 = (c4 >> 1) ^ (n & 1u);   // swizzled 16-byte chunk
                    __half2 lo = __floats2half2_rn(v[k].x, v[k].y), hi = __floats2half2_rn(v[k].z, v[k].w);
                    uint2 packed;
                    packed.x = *reinterpret_cast<uint32_t*>(&lo);
                    packed.y = *reinterpret_cast<uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(smem + (s * NB + n) * 256 + 128 + chunk16 * 16 + (c4 & 1u) * 8) = packed;
                }
            }
        }
        // 3. Decoded block scales of the tile's 64 rows for the chunk.
        {
            constexpr int kPerThread = kRowsTile * CH / kThreads;
            float sc[kPerThread];
#pragma unroll
            for (int k = 0; k < kPerThread; ++k) {
                const uint32_t i = tid + k * kThreads;
                const uint32_t r = i / CH, s = i % CH;
                const uint64_t row = min(row0 + r, out - 1);
                const uint64_t flat = row * in + static_cast<uint64_t>(chunk0 + min(s, chunk_steps - 1)) * kStepK;
                sc[k] = decode_block_scale(w, flat >> w.block_shift);
            }
#pragma unroll
            for (int k = 0; k < kPerThread; ++k) {
                const uint32_t i = tid + k * kThreads;
                s_scale[(i / CH) * (CH + 1) + i % CH] = sc[k];
            }
        }
        asm volatile("cp.async.wait_group 0;\n" ::);
        __syncthreads();

        // 4. Tensor-core accumulation of this warp's steps.
#pragma unroll
        for (int u = 0; u < SPW; ++u) {
            const uint32_t s = wk + u * kWK;
            if (s < chunk_steps) {
                uint4 xf[MT][2];
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const uint32_t n = m * 8 + g;
                    const uint8_t* xrow = smem + (s * NB + n) * 256 + 128;
                    xf[m][0] = *reinterpret_cast<const uint4*>(xrow + (((2 * t) ^ (n & 1u)) * 16));
                    xf[m][1] = *reinterpret_cast<const uint4*>(xrow + (((2 * t + 1) ^ (n & 1u)) * 16));
                }
#pragma unroll
                for (int rg = 0; rg < 2; ++rg) {
                    float part[MT][4];
#pragma unroll
                    for (int m = 0; m < MT; ++m)
#pragma unroll
                        for (int e = 0; e < 4; ++e) part[m][e] = 0.0f;
                    const uint32_t wa[2] = {code[u][2 * rg].x, code[u][2 * rg].y};
                    const uint32_t wb[2] = {code[u][2 * rg + 1].x, code[u][2 * rg + 1].y};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t word_a = wa[i >> 1], word_b = wb[i >> 1];
                        const uint32_t sel0 = (i & 1) ? 0x5524u : 0x5504u;
                        const uint32_t sel1 = (i & 1) ? 0x5534u : 0x5514u;
                        const uint32_t a0 = *reinterpret_cast<const uint32_t*>(smem + __byte_perm(word_a, lane4, sel0));
                        const uint32_t a2 = *reinterpret_cast<const uint32_t*>(smem + __byte_perm(word_a, lane4, sel1));
                        const uint32_t a1 = *reinterpret_cast<const uint32_t*>(smem + __byte_perm(word_b, lane4, sel0));
                        const uint32_t a3 = *reinterpret_cast<const uint32_t*>(smem + __byte_perm(word_b, lane4, sel1));
#pragma unroll
                        for (int m = 0; m < MT; ++m) {
                            const uint4& xv = xf[m][i >> 1];
                            const uint32_t b0 = (i & 1) ? xv.z : xv.x;
                            const uint32_t b1 = (i & 1) ? xv.w : xv.y;
                            mma_f16_16816(part[m], a0, a1, a2, a3, b0, b1);
                        }
                    }
                    const float sA = s_scale[(wr * 32 + rg * 16 + g) * (CH + 1) + s];
                    const float sB = s_scale[(wr * 32 + rg * 16 + g + 8) * (CH + 1) + s];
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        acc[rg][m][0] = fmaf(sA, part[m][0], acc[rg][m][0]);
                        acc[rg][m][1] = fmaf(sA, part[m][1], acc[rg][m][1]);
                        acc[rg][m][2] = fmaf(sB, part[m][2], acc[rg][m][2]);
                        acc[rg][m][3] = fmaf(sB, part[m][3], acc[rg][m][3]);
                    }
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::);
    __syncthreads();  // scales no longer needed: the scratch becomes the reduction buffer

    // ---- combine the kWK warps of the CTA (fixed order) ----
#pragma unroll
    for (int rg = 0; rg < 2; ++rg)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float* dst = s_red + (wk * kRowsTile + wr * 32 + rg * 16) * NB + m * 8;
            dst[g * NB + 2 * t] = acc[rg][m][0];
            dst[g * NB + 2 * t + 1] = acc[rg][m][1];
            dst[(g + 8) * NB + 2 * t] = acc[rg][m][2];
            dst[(g + 8) * NB + 2 * t + 1] = acc[rg][m][3];
        }
    __syncthreads();
    for (uint32_t i = tid; i < kRowsTile * NB; i += kThreads) {
        float v = 0.0f;
#pragma unroll
        for (int k = 0; k < kWK; ++k) v += s_red[k * kRowsTile * NB + i];
        s_out[i] = v;
    }

    // ---- combine the ranks of the cluster through distributed shared memory ----
    if (ksplit > 1) {
        cluster.sync();
    } else {
        __syncthreads();
    }
    // Element i = n * 64 + r: consecutive threads write consecutive outputs of a batch row.
    for (uint32_t i = tid + krank * kThreads; i < kRowsTile * NB; i += kThreads * ksplit) {
        const uint32_t n = i / kRowsTile, r = i % kRowsTile;
        float v = 0.0f;
        for (uint32_t k = 0; k < ksplit; ++k) {
            const float* remote = ksplit > 1 ? cluster.map_shared_rank(s_out, k) : s_out;
            v += remote[r * NB + n];
        }
        if (n < p.rows && row0 + r < out) p.y[static_cast<uint64_t>(n) * out + row0 + r] = v;
    }
    if (ksplit > 1) cluster.sync();  // peers may still be reading this CTA's s_out
}

__global__ void gemv_lut_init_kernel(uint32_t* lut) {
    // Compact [256][32] words: entry v, replicated for the 32 lanes, holds the
    // fp16 pair (low nibble's value in the low half) of packed byte v.
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= 256 * 32) return;
    const uint32_t v = i >> 5;
    const __half lo = __float2half_rn(kNf4Codebook[v & 15u]);
    const __half hi = __float2half_rn(kNf4Codebook[v >> 4]);
    lut[i] = static_cast<uint32_t>(__half_as_ushort(lo)) | (static_cast<uint32_t>(__half_as_ushort(hi)) << 16);
}

template <int MT>
int32_t launch_config(const DeviceContext& ctx, const GemvParams& p, uint32_t ksplit, cudaStream_t stream) {
    using S = Smem<MT>;
    auto kernel = nf4_gemv_kernel<MT>;
    static PerDeviceOnce configured;  // per template instance
    B2_TRY(once_per_device(configured, ctx.device, [&]() -> int32_t {
        B2_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
        return B2_STATUS_OK;
    }));
    const uint32_t row_tiles = static_cast<uint32_t>((p.w.out_features + kRowsTile - 1) / kRowsTile);
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(row_tiles * ksplit);
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

}  // namespace

int32_t init_gemv_lut(DeviceContext* ctx) {
    B2_CUDA_TRY(cudaMalloc(&ctx->gemv_lut, 256 * 32 * 4));
    gemv_lut_init_kernel<<<32, 256>>>(ctx->gemv_lut);
    B2_CUDA_TRY(cudaGetLastError());
    B2_CUDA_TRY(cudaDeviceSynchronize());
    return B2_STATUS_OK;
}

bool nf4_gemv_supported(const WeightView& w, const float* x, const float* y, uint64_t rows) {
    (void)y;
    return rows >= 1 && rows <= 32 && w.in_features % kStepK == 0 && w.block_size >= kStepK &&
           (reinterpret_cast<uintptr_t>(w.codes) & 7u) == 0 &&
           (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && w.in_features / kStepK <= 0xFFFFFFFFull &&
           w.out_features <= 0x3FFFFFFFull;
}

int32_t launch_nf4_gemv(const DeviceContext& ctx, const WeightView& w, const float* x, float* y,
                        uint64_t rows, cudaStream_t stream) {
    GemvParams p;
    p.w = w;
    p.x = x;
    p.y = y;
    p.rows = static_cast<uint32_t>(rows);
    p.steps_total = static_cast<uint32_t>(w.in_features / kStepK);
    p.lut = ctx.gemv_lut;
    const uint32_t chunk = rows <= 8 ? chunk_steps_for<1>() : rows <= 16 ? chunk_steps_for<2>() : chunk_steps_for<4>();
    // One chunk per cluster rank where the portable cluster limit of 8 allows.
    uint32_t ksplit = (p.steps_total + chunk - 1) / chunk;
    if (ksplit > 8) ksplit = 8;
    p.steps_per_cta = (p.steps_total + ksplit - 1) / ksplit;
    if (rows <= 8) return launch_config<1>(ctx, p, ksplit, stream);
    if (rows <= 16) return launch_config<2>(ctx, p, ksplit, stream);
    return launch_config<4>(ctx, p, ksplit, stream);
}

}  // namespace b2
