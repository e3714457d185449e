// QLoRA input-backward for many rows: dX[M, in] = dY[M, out] * W[out, in]
// (reference loop: src/core/backend/nn/quantized_linear/reference/operations.cpp:83-115).
//
// The contraction runs over the OUTPUT rows of W, i.e. across the packed rows,
// so a fused kernel has to transpose nibbles inside the SM (nf4_gemm_sm100.cu
// does, and is bound by shared memory at about a third of the tensor peak).
// With thousands of rows of dY the cheaper plan is to pay the transposition
// once per call: a streaming pre-pass expands W to bf16 and writes it
// transposed, Wt[in, out] (29 MB read, 117 MB written for a 14336 x 4096 layer,
// ~3 % of the GEMM's time at M = 4096), and the GEMM itself is then a plain
// bf16 x bf16 tcgen05 kernel whose two operands both arrive by TMA:
//   D[256 tokens, 256 in-columns] += dY_tile[256, 64] * Wt_tile[256, 64]^T
// One producer thread, one issuing thread (one wait and one commit per
// k-block), epilogue by sixteen warps. Every mbarrier wait is bounded.
//
// Numerics: weight = bf16(codebook * scale) with the product in FP32 (one
// rounding; the fused kernel rounds the codebook value and the scale first).
#include "b2_common.cuh"
#include "b2_kernels.h"
#include "sm100_ptx.cuh"

#include <cuda_bf16.h>

#include <mutex>

namespace b2 {
namespace {

using namespace sm100;

// ---- pre-pass: Wt[i, o] = bf16(W[o, i]) ----------------------------------------------------------

constexpr int kTrRows = 64;              // output rows of W per CTA (the GEMM's contraction)
constexpr int kTrCols = 256;             // input columns of W per CTA: 128 contiguous packed bytes per row
constexpr int kTrPitch = kTrRows + 8;    // bf16 per shared-memory row: 144 B, rows stay 16-byte aligned

// A CTA expands a [64 x 256] tile of W and writes it transposed: 256 rows of Wt, 128 contiguous
// bytes each. Thread (row = t % 64, q = t / 64) expands the 64 weights [64q, 64q + 64) of its row
// (one scale block, as blocks hold at least 64 weights and start on multiples of 64): a warp is 32
// consecutive rows of one q, so its 2-byte stores into the transposed tile fall into 64 contiguous
// bytes. The store phase moves 16 bytes per thread, eight threads per 128-byte row of Wt.
__global__ void __launch_bounds__(256)
nf4_dequant_transpose_kernel(const WeightView w, __nv_bfloat16* __restrict__ wt) {
    pdl_launch_dependents();
    __shared__ __align__(16) __nv_bfloat16 tile[kTrCols][kTrPitch];
    __shared__ float codebook[16];   // a per-lane index into __constant__ memory would serialise the warp
    if (threadIdx.x < 16) codebook[threadIdx.x] = kNf4Codebook[threadIdx.x];
    __syncthreads();
    const uint64_t in = w.in_features, out = w.out_features;
    const uint32_t i0 = blockIdx.x * kTrCols, o0 = blockIdx.y * kTrRows;
    const uint32_t t = threadIdx.x;
    {
        const uint32_t row = t & 63u, q = t >> 6;
        if (i0 + 64u * q < in) {
            const uint64_t flat = (static_cast<uint64_t>(o0) + row) * in + i0 + 64u * q;
            const uint2* src = reinterpret_cast<const uint2*>(w.codes + (flat >> 1));
            const uint2 p0 = __ldg(src), p1 = __ldg(src + 1), p2 = __ldg(src + 2), p3 = __ldg(src + 3);
            const float scale = decode_block_scale(w, flat >> w.block_shift);
            const uint32_t words[8] = {p0.x, p0.y, p1.x, p1.y, p2.x, p2.y, p3.x, p3.y};
#pragma unroll
            for (int k = 0; k < 64; ++k) {
                const uint32_t code = (words[k >> 3] >> (4 * (k & 7))) & 0xFu;
                tile[64u * q + k][row] = __float2bfloat16_rn(codebook[code] * scale);
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (uint32_t it = 0; it < 8u; ++it) {
        const uint32_t idx = t + 256u * it, col = idx >> 3, chunk = idx & 7u;
        if (i0 + col < in) {
            const uint4 v = *reinterpret_cast<const uint4*>(&tile[col][chunk * 8u]);
            *reinterpret_cast<uint4*>(wt + (static_cast<uint64_t>(i0) + col) * out + o0 + chunk * 8u) = v;
        }
    }
}

// ---- GEMM: both operands bf16 K-major in global memory ----------------------------------------------

constexpr int kBM = 256, kBK = 64;
constexpr int kStages = 3;
constexpr int kOperandBytes = 256 * kBK * 2;            // 32 KB per operand and stage
constexpr int kStageBytes = 2 * kOperandBytes;
constexpr int kWarps = 18;                              // producer, issuer, 16 epilogue warps
constexpr int kThreads = kWarps * 32;
constexpr int kSmemBytes = kStages * kStageBytes + 1024;
constexpr uint32_t kTmemColumns = 512;

struct Params {
    float* out;        // [m, n] fp32
    uint32_t m, n, k;
    uint32_t* error;
};

struct Barriers {
    uint64_t full[kStages];
    uint64_t done[kStages];
    uint64_t acc_full;
    uint32_t tmem_base;
    uint32_t abort;
};

// BN: in-columns per tile (256, 224 or 192). The host picks the width that needs the fewest
// tile-widths of time on the device's SMs: 14336 in-columns at 4096 rows are 896 tiles of 256
// (6.05 waves of 148, paid as 7) but 1024 tiles of 224 (6.9 waves, paid as 7 x 224 / 256).
template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
bf16_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
    constexpr uint32_t kBytesB = BN * kBK * 2;   // B operand of a stage (its slot stays 32 KB)
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) Barriers bars;
    const uint32_t raw32 = smem_u32(smem_raw);
    const uint32_t base32 = (raw32 + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base32 - raw32);
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t n0 = blockIdx.x * BN, m0 = blockIdx.y * kBM;
    const uint32_t num_kb = p.k / kBK;
    volatile uint32_t* abort = &bars.abort;

    if (warp == 0) {
        if (lane == 0) {
            for (int s = 0; s < kStages; ++s) {
                mbar_init(&bars.full[s], 1);
                mbar_init(&bars.done[s], 1);
            }
            mbar_init(&bars.acc_full, 1);
            bars.abort = 0;
            mbar_fence_init();
            tma_prefetch_descriptor(&map_a);
            tma_prefetch_descriptor(&map_b);
        }
        __syncwarp();
        tmem_alloc(&bars.tmem_base, kTmemColumns);
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = bars.tmem_base;
    pdl_launch_dependents();
    pdl_wait();   // both operands were written by the pre-passes just before this launch

    if (warp == 0) {
        if (lane == 0) {
            uint32_t s = 0, ph = 0;
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                if (kb >= kStages) mbar_wait(&bars.done[s], ph ^ 1u, abort);
                mbar_expect_tx(&bars.full[s], kOperandBytes + kBytesB);
                tma_load_2d(smem + s * kStageBytes, &map_a, static_cast<int>(kb * kBK), static_cast<int>(m0),
                            &bars.full[s]);
                tma_load_2d(smem + s * kStageBytes + kOperandBytes, &map_b, static_cast<int>(kb * kBK),
                            static_cast<int>(n0), &bars.full[s]);
                if (++s == kStages) {
                    s = 0;
                    ph ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16_f32(128, BN);
            const uint64_t d0 = umma_desc_k_major_sw128(base32);
            uint32_t s = 0, ph = 0;
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                mbar_wait(&bars.full[s], ph, abort);
                tcgen05_fence_after_sync();
                const uint64_t da_s = d0 + ((s * static_cast<uint32_t>(kStageBytes)) >> 4);
                const uint64_t db_s = da_s + (kOperandBytes >> 4);
#pragma unroll
                for (uint32_t h = 0; h < 2; ++h) {
#pragma unroll
                    for (uint32_t kk = 0; kk < kBK / 16; ++kk) {
                        umma_bf16(tmem_base + h * 256u, da_s + ((h * 16384u + kk * 32u) >> 4), db_s + ((kk * 32u) >> 4),
                                  idesc, (kb | kk) != 0u ? 1u : 0u);
                    }
                }
                umma_commit(&bars.done[s]);
                if (++s == kStages) {
                    s = 0;
                    ph ^= 1u;
                }
            }
            umma_commit(&bars.acc_full);
        }
    } else {
        // ---- epilogue: TMEM -> registers -> global ----
        mbar_wait(&bars.acc_full, 0u, abort, 20000000u);
        tcgen05_fence_after_sync();
        const uint32_t quarter = warp & 3u, half = ((warp - 2u) >> 2) & 1u, col_half = (warp - 2u) >> 3;
        constexpr uint32_t kChunks = BN / 32, kFirstHalf = (kChunks + 1) / 2;   // 32-column chunks per accumulator
        for (uint32_t c = col_half == 0u ? 0u : kFirstHalf; c < (col_half == 0u ? kFirstHalf : kChunks); ++c) {
            uint32_t v[32];
            tmem_ld_32x32(tmem_base + ((quarter * 32u) << 16) + half * 256u + c * 32u, v);
            tmem_ld_wait();
            const uint32_t col0 = n0 + c * 32u;
            // Transpose the warp's [32 rows x 32 columns] chunk through shared memory (the operand
            // ring is free: every MMA has completed) so that each store instruction writes one
            // row's 128 contiguous bytes instead of 16 bytes of 32 different rows.
            float* scratch = reinterpret_cast<float*>(smem) + (warp - 2u) * (32u * 33u);
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 32; ++i) scratch[lane * 33u + i] = __uint_as_float(v[i]);
            __syncwarp();
            const uint32_t row_base = m0 + half * 128u + quarter * 32u;
            if (col0 + lane < p.n) {
#pragma unroll 8
                for (uint32_t r = 0; r < 32u; ++r) {
                    if (row_base + r < p.m) {
                        p.out[static_cast<uint64_t>(row_base + r) * p.n + col0 + lane] = scratch[r * 33u + lane];
                    }
                }
            }
        }
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        tmem_dealloc(tmem_base, kTmemColumns);
        if (lane == 0 && bars.abort != 0 && p.error != nullptr) atomicOr(p.error, 1u);
    }
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

// bf16 [rows][cols] row-major, box = 64 columns x `box_rows` rows, 128-byte swizzle, zero fill outside.
int32_t operand_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {kBK, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode_tiled()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                                      box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B2_STATUS_RUNTIME_ERROR, "cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
    return B2_STATUS_OK;
}

}  // namespace

// Worth it from a few hundred rows of dY on (the transposed expansion costs about as much as 150
// rows of the GEMM); whole 64 x 64 tiles of W, blocks that do not straddle a 64-wide tile.
bool nf4_backward_dense_supported(const WeightView& w, const float* dy, uint64_t rows) {
    return rows >= 512 && w.in_features % 64 == 0 && w.out_features % 64 == 0 && w.block_size >= 64 &&
           w.in_features % w.block_size == 0 && (reinterpret_cast<uintptr_t>(w.codes) & 7u) == 0 &&
           (reinterpret_cast<uintptr_t>(dy) & 15u) == 0 && encode_tiled() != nullptr && rows <= 0x7FFFFFFFull &&
           w.out_features <= 0x7FFFFFFFull && w.in_features <= 0x7FFFFFFFull;
}

// bf16 copy of dY (rows * out) followed by the transposed bf16 weight (in * out), each 256-byte aligned.
size_t nf4_backward_dense_workspace_bytes(const WeightView& w, uint64_t rows) {
    const size_t dy_bytes = (static_cast<size_t>(rows) * w.out_features * 2 + 255) & ~static_cast<size_t>(255);
    return dy_bytes + static_cast<size_t>(w.in_features) * w.out_features * 2;
}

int32_t launch_nf4_backward_dense(const DeviceContext& ctx, const WeightView& w, const float* dy, float* dx,
                                  uint64_t rows, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    const size_t need = nf4_backward_dense_workspace_bytes(w, rows);
    if (workspace == nullptr || workspace_bytes < need) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 GEMM workspace too small: need %zu bytes", need);
    }
    if ((reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 GEMM workspace must be 16-byte aligned");
    }
    const size_t dy_bytes = (static_cast<size_t>(rows) * w.out_features * 2 + 255) & ~static_cast<size_t>(255);
    uint8_t* dy16 = static_cast<uint8_t*>(workspace);
    uint8_t* wt16 = dy16 + dy_bytes;
    B2_TRY(launch_f32_to_bf16(ctx, dy, dy16, rows * w.out_features, stream));
    const dim3 tgrid(static_cast<unsigned>((w.in_features + kTrCols - 1) / kTrCols),
                     static_cast<unsigned>(w.out_features / kTrRows));
    nf4_dequant_transpose_kernel<<<tgrid, 256, 0, stream>>>(w, reinterpret_cast<__nv_bfloat16*>(wt16));
    B2_CUDA_TRY(cudaGetLastError());

    // tile width: the fewest tile-widths of time over the device's SMs (ties go to the wider tile)
    const uint64_t m_tiles = (rows + kBM - 1) / kBM;
    uint32_t bn = 256;
    uint64_t best = ~0ull;
    for (uint32_t cand : {256u, 224u, 192u}) {
        const uint64_t tiles = ((w.in_features + cand - 1) / cand) * m_tiles;
        const uint64_t cost = ((tiles + ctx.sm_count - 1) / ctx.sm_count) * cand;
        if (cost < best) {
            best = cost;
            bn = cand;
        }
    }
    CUtensorMap map_a, map_b;
    B2_TRY(operand_map(&map_a, dy16, rows, w.out_features, 256));            // dY  [M, K = out]
    B2_TRY(operand_map(&map_b, wt16, w.in_features, w.out_features, bn));    // Wt  [N = in, K = out]
    static PerDeviceOnce configured;
    B2_TRY(once_per_device(configured, ctx.device, []() -> int32_t {
        B2_CUDA_TRY(cudaFuncSetAttribute(bf16_gemm_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        B2_CUDA_TRY(cudaFuncSetAttribute(bf16_gemm_kernel<224>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        B2_CUDA_TRY(cudaFuncSetAttribute(bf16_gemm_kernel<192>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        return B2_STATUS_OK;
    }));
    Params p;
    p.out = dx;
    p.m = static_cast<uint32_t>(rows);
    p.n = static_cast<uint32_t>(w.in_features);
    p.k = static_cast<uint32_t>(w.out_features);
    p.error = ctx.gemm_error;
    const dim3 grid(static_cast<unsigned>((w.in_features + bn - 1) / bn), static_cast<unsigned>(m_tiles));
    if (bn == 256) {
        bf16_gemm_kernel<256><<<grid, kThreads, kSmemBytes, stream>>>(map_a, map_b, p);
    } else if (bn == 224) {
        bf16_gemm_kernel<224><<<grid, kThreads, kSmemBytes, stream>>>(map_a, map_b, p);
    } else {
        bf16_gemm_kernel<192><<<grid, kThreads, kSmemBytes, stream>>>(map_a, map_b, p);
    }
    B2_CUDA_TRY(cudaGetLastError());
    return B2_STATUS_OK;
}

}  // namespace b2
