// Prefill packed-NF4 linear, forward, with the dequantised weights in TENSOR memory.
//   Y[M, out] = X[M, in] * W[out, in]^T      (reference loop:
//   src/core/backend/nn/quantized_linear/reference/operations.cpp:49-81)
//
// The 256 x 256 kernel of nf4_gemm_sm100.cu writes the expanded weight tile to
// shared memory and lets tcgen05.mma read it back, which makes the 128 B/clk
// shared-memory port - not the tensor pipe - its limit. Here the roles are
// swapped: a CTA computes the transposed tile D[128 weight rows, 256 tokens];
// the weight tile is the A operand and lives in tensor memory (each expansion
// thread owns one weight row = one TMEM lane and writes its 64 bf16 values of a
// k-block with one tcgen05.st), the activations (bf16 by the streaming
// pre-pass) are the B operand and arrive by TMA. Shared memory then carries only
// the activation tile (written once by TMA, read once by the MMAs) and the
// byte -> bf16x2 table lookups.
//
// Sixteen expansion warps form four groups of four (a group covers the 128
// lanes); group g expands the k-blocks kb = g mod 4 into TMEM stage g, so four
// k-blocks are in expansion at any time. tcgen05.mma (M128, N = tokens of the tile,
// K16, A from TMEM) is issued by one thread, tcgen05.commit releases the activation
// stage and the TMEM stage. With a full 256-token tile the MMAs themselves set the
// pace and one issuing warp is enough; with at most 64 tokens (decode batches) the
// pace is the issuing thread's own instruction latency (~1000 cycles per k-block
// for two waits, four MMAs and two commits), so every expansion group then issues
// its own k-blocks into its own accumulator and the four accumulators are summed
// in the epilogue. Every mbarrier wait is bounded.
#include "b2_common.cuh"
#include "b2_kernels.h"
#include "sm100_ptx.cuh"

#include <cooperative_groups.h>
#include <cuda_bf16.h>

#include <cstdlib>
#include <mutex>

namespace cg = cooperative_groups;

namespace b2 {
namespace {

using namespace sm100;

constexpr int kTileW = 128;                    // weight rows per CTA (MMA M, TMEM lanes)
constexpr int kMaxTileT = 256;                 // tokens per CTA at most (MMA N, accumulator columns)
constexpr int kBK = 64;
constexpr int kGroups = 4;                     // expansion groups = weight stages in TMEM
constexpr int kXBytes = 4 * kMaxTileT * kBK * 2;   // 128 KB of activation stages (or of partial sums)
constexpr int kLutBytes = 256 * 128;
constexpr int kExpandWarps = 16;
constexpr int kThreads = (2 + kExpandWarps) * 32;
constexpr int kSmemBytes = kXBytes + kLutBytes + 32768 /* table alignment */ + 1024;
constexpr uint32_t kTmemColumns = 512;
constexpr uint32_t kAccColumns = kMaxTileT;    // D: columns [0, tile_t) of [0, 256)
constexpr uint32_t kWeightColumns = kBK / 2;   // one weight stage: 64 bf16 = 32 columns
constexpr uint32_t kMultiIssueTokens = 64;     // up to here: one accumulator (64 columns) and one issuer per group

constexpr int kMaxWeights = 4;                 // weights applied to the same activations in one launch

struct Params {
    WeightView w[kMaxWeights];
    float* out[kMaxWeights];         // [m, n[i]] fp32
    uint32_t n[kMaxWeights];         // output features of every weight
    uint32_t tile_end[kMaxWeights];  // running count of 128-row tiles: weight i owns tiles [tile_end[i-1], tile_end[i])
    uint32_t count;                  // weights in this launch
    uint32_t m, k;                   // tokens, contraction length
    uint32_t tile_t;     // tokens per CTA: multiple of 16, <= 256
    uint32_t kb_per_cta; // k-blocks per CTA (the contraction is split over the cluster along z)
    uint32_t* error;
    const uint32_t* lut; // compact [256][32] words of bf16 pairs
};

// K-block i of a CTA uses slot i % 4 for both its activation stage and its weight stage, so one
// barrier per slot says "operands ready" (the TMA's byte count plus one arrival of each of the
// group's four warps) and one says "MMAs done" (tcgen05.commit): one wait and one commit per
// k-block for the issuing thread, whose instruction latency paces the CTA.
struct Barriers {
    uint64_t full[kGroups];
    uint64_t done[kGroups];
    uint64_t acc_full;
    uint32_t tmem_base;
    uint32_t abort;
};

__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
    __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t shared_addr) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(shared_addr));
    return v;
}
__device__ __forceinline__ void sts_u4(uint32_t shared_addr, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(shared_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}
__device__ __forceinline__ uint4 ldg_u4(const uint8_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t scale_pair(float s) {
    __nv_bfloat162 p = __float2bfloat162_rn(s);
    return *reinterpret_cast<uint32_t*>(&p);
}

// 32 lanes x 32 columns: thread i of the warp writes its 32 registers to lane (base + i).
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
          "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
          "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

struct RawScale {
    uint32_t bits;
    float second;
};
__device__ __forceinline__ RawScale fetch_raw_scale(const WeightView& w, uint64_t block) {
    RawScale s;
    if (w.encoding == B2_SCALES_FLOAT32) {
        s.bits = __float_as_uint(__ldg(w.fp32_scales + block));
        s.second = 0.0f;
    } else {
        s.bits = __ldg(w.scale_codes + block);
        s.second = __ldg(w.second_level + ((w.flat_block_base + block) >> w.scale_block_shift));
    }
    return s;
}
__device__ __forceinline__ float finish_raw_scale(const WeightView& w, const RawScale& s, const float* factor) {
    return w.encoding == B2_SCALES_FLOAT32 ? __uint_as_float(s.bits) : dq_finish(factor[s.bits], s.second, w.offset);
}

__global__ void __launch_bounds__(kThreads, 1)
nf4_gemm_tmem_kernel(const __grid_constant__ CUtensorMap map_x, const Params p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) Barriers bars;
    __shared__ float s_factor[256];   // scale code -> (code - 128) / 127
    const uint32_t raw32 = smem_u32(smem_raw);
    const uint32_t base32 = (raw32 + 1023u) & ~1023u;
    const uint32_t x32 = base32;
    const uint32_t lut32 = (x32 + kXBytes + 32767u) & ~32767u;
    uint8_t* smem = smem_raw + (base32 - raw32);

    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t ksplit = cluster.num_blocks();     // cluster = (1, 1, ksplit)
    const uint32_t krank = cluster.block_rank();

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t tile_t = p.tile_t;
    const uint32_t stage_bytes = tile_t * (kBK * 2u);
    const bool multi_issue = tile_t <= kMultiIssueTokens;
    // Which weight this CTA's tile belongs to (a launch may apply up to four weights to the same
    // activations); the selected view is copied so that it lives in registers.
    uint32_t wi = 0;
#pragma unroll
    for (int i = 1; i < kMaxWeights; ++i) {
        if (static_cast<uint32_t>(i) < p.count && blockIdx.x >= p.tile_end[i - 1]) wi = static_cast<uint32_t>(i);
    }
    WeightView w = p.w[0];
    float* out = p.out[0];
    uint32_t n_out = p.n[0], tile0 = 0;
#pragma unroll
    for (int i = 1; i < kMaxWeights; ++i) {
        if (wi == static_cast<uint32_t>(i)) {
            w = p.w[i];
            out = p.out[i];
            n_out = p.n[i];
            tile0 = p.tile_end[i - 1];
        }
    }
    const uint32_t n0 = (blockIdx.x - tile0) * kTileW;   // first weight row (output feature) of the tile
    const uint32_t m0 = blockIdx.y * tile_t;   // first token of the tile
    const uint32_t total_kb = p.k / kBK;
    const uint32_t kb_begin = min(krank * p.kb_per_cta, total_kb);
    const uint32_t num_kb = min(p.kb_per_cta, total_kb - kb_begin);   // k-blocks of this CTA
    volatile uint32_t* abort = &bars.abort;

    if (warp == 0) {
        if (lane == 0) {
            for (int g = 0; g < kGroups; ++g) {
                mbar_init(&bars.full[g], 5);      // the producer's expect_tx + lane 0 of the group's four warps
                mbar_init(&bars.done[g], 1);
            }
            mbar_init(&bars.acc_full, p.tile_t <= kMultiIssueTokens ? kGroups : 1);
            bars.abort = 0;
            mbar_fence_init();
            tma_prefetch_descriptor(&map_x);
        }
        __syncwarp();
        tmem_alloc(&bars.tmem_base, kTmemColumns);
    }
    for (uint32_t i = tid; i < kLutBytes / 16; i += kThreads) {
        sts_u4(lut32 + i * 16u, __ldg(reinterpret_cast<const uint4*>(p.lut) + i));
    }
    if (tid < 256) s_factor[tid] = dq_factor(tid);
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = bars.tmem_base;
    const uint32_t tmem_w = tmem_base + kAccColumns;   // weight stages behind the accumulator
    // Everything above touched only this CTA's shared and tensor memory; caller tensors are read
    // and written below, after the kernels this launch depends on have completed.
    pdl_launch_dependents();
    pdl_wait();

    if (warp == 0) {
        // ---- TMA producer: activation tiles [tile_t tokens x 64] ----
        if (lane == 0) {
            for (uint32_t i = 0; i < num_kb; ++i) {
                const uint32_t j = i % kGroups;
                if (i >= kGroups) mbar_wait(&bars.done[j], ((i / kGroups) - 1u) & 1u, abort);
                mbar_expect_tx(&bars.full[j], stage_bytes);
                tma_load_2d(smem + j * stage_bytes, &map_x, static_cast<int>((kb_begin + i) * kBK),
                            static_cast<int>(m0), &bars.full[j]);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer (full tiles; small tiles are issued by the expansion groups) ----
        if (lane == 0 && !multi_issue) {
            const uint32_t idesc = umma_idesc_bf16_f32(kTileW, tile_t);
            const uint64_t dx0 = umma_desc_k_major_sw128(x32);
            const uint32_t stage16 = stage_bytes >> 4;
            for (uint32_t i = 0; i < num_kb; ++i) {
                const uint32_t j = i % kGroups;
                mbar_wait(&bars.full[j], (i / kGroups) & 1u, abort);
                tcgen05_fence_after_sync();
                const uint64_t dx_s = dx0 + j * stage16;
#pragma unroll
                for (uint32_t kk = 0; kk < kBK / 16; ++kk) {
                    // 16 contraction values = 8 columns of the weight stage, 32 bytes of an activation row
                    umma_bf16_a_tmem(tmem_base, tmem_w + j * kWeightColumns + kk * 8u, dx_s + kk * 2u, idesc,
                                     (i | kk) != 0u ? 1u : 0u);
                }
                umma_commit(&bars.done[j]);
            }
            umma_commit(&bars.acc_full);
        }
    } else {
        // ---- expansion warps: one weight row per thread, group g takes this CTA's k-blocks g, g+4, ... ----
        const uint32_t e = warp - 2u;
        const uint32_t g = e >> 2;
        const uint32_t quarter = warp & 3u;           // the TMEM lanes this warp may touch
        const uint32_t row = quarter * 32u + lane;    // weight row of the tile = TMEM lane
        const uint32_t n = n0 + row;
        const uint32_t lut_lane = lut32 | (lane * 4u);
        const bool live = n < n_out;
        const uint8_t* codes = live ? w.codes + static_cast<uint64_t>(n) * (p.k >> 1) + kb_begin * 32u : nullptr;
        const uint64_t flat0 = static_cast<uint64_t>(n) * p.k + static_cast<uint64_t>(kb_begin) * kBK;
        const uint32_t taddr = tmem_w + g * kWeightColumns + ((quarter * 32u) << 16);
        const bool leader = (e & 3u) == 0u;           // first warp of the group: issues the group's MMAs for small tiles
        const uint32_t idesc = umma_idesc_bf16_f32(kTileW, tile_t);
        const uint64_t dx0 = umma_desc_k_major_sw128(x32);

        // This group's k-blocks; codes and raw scale are fetched two of them (eight k-blocks) ahead
        // into a ring of three register sets. The loop is unrolled by three so that every set is
        // addressed statically: copying a set whose load is still in flight (a rotating
        // "next = next-next") would make the thread wait for memory in every iteration.
        uint4 c[3][2];
        RawScale raw[3];
        auto fetch = [&](uint32_t i, uint4 (&cc)[2], RawScale& rr) {
            cc[0] = cc[1] = make_uint4(0, 0, 0, 0);
            rr.bits = 0u;
            rr.second = 0.0f;
            if (live && i < num_kb) {
                cc[0] = ldg_u4(codes + i * 32u);
                cc[1] = ldg_u4(codes + i * 32u + 16u);
                rr = fetch_raw_scale(w, (flat0 + static_cast<uint64_t>(i) * kBK) >> w.block_shift);
            }
        };
        fetch(g, c[0], raw[0]);
        fetch(g + kGroups, c[1], raw[1]);
        uint32_t use = 0;   // how often this group's stage has been filled
        for (uint32_t i0 = g; i0 < num_kb; i0 += 3u * kGroups) {
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                const uint32_t i = i0 + static_cast<uint32_t>(j) * kGroups;
                if (i < num_kb) {   // warp-uniform
                    fetch(i + 2u * kGroups, c[(j + 2) % 3], raw[(j + 2) % 3]);
                    if (use > 0) mbar_wait(&bars.done[g], (use - 1u) & 1u, abort);
                    tcgen05_fence_after_sync();
                    const uint32_t s2 = scale_pair(live ? finish_raw_scale(w, raw[j], s_factor) : 0.0f);
                    uint32_t v[32];
                    const uint32_t words[8] = {c[j][0].x, c[j][0].y, c[j][0].z, c[j][0].w,
                                               c[j][1].x, c[j][1].y, c[j][1].z, c[j][1].w};
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        const uint32_t word = words[q];
                        v[4 * q + 0] = bf16x2_mul(lds_u32(((word << 7) & 0x7F80u) | lut_lane), s2);
                        v[4 * q + 1] = bf16x2_mul(lds_u32(((word >> 1) & 0x7F80u) | lut_lane), s2);
                        v[4 * q + 2] = bf16x2_mul(lds_u32(((word >> 9) & 0x7F80u) | lut_lane), s2);
                        v[4 * q + 3] = bf16x2_mul(lds_u32(((word >> 17) & 0x7F80u) | lut_lane), s2);
                    }
                    tmem_st_32x32(taddr, v);
                    tmem_st_wait();
                    tcgen05_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars.full[g]);
                    if (multi_issue && leader && lane == 0) {
                        // this group's k-block: slot g, its own accumulator
                        mbar_wait(&bars.full[g], use & 1u, abort);
                        tcgen05_fence_after_sync();
                        const uint64_t dx_s = dx0 + g * (stage_bytes >> 4);
#pragma unroll
                        for (uint32_t kk = 0; kk < kBK / 16; ++kk) {
                            umma_bf16_a_tmem(tmem_base + g * kMultiIssueTokens, tmem_w + g * kWeightColumns + kk * 8u,
                                             dx_s + kk * 2u, idesc, (use | kk) != 0u ? 1u : 0u);
                        }
                        umma_commit(&bars.done[g]);
                    }
                    __syncwarp();
                    ++use;
                }
            }
        }
        if (multi_issue && leader && lane == 0) umma_commit(&bars.acc_full);   // after this group's last MMA

        // ---- epilogue: lane = weight row, column = token ----
        mbar_wait(&bars.acc_full, 0u, abort);
        tcgen05_fence_after_sync();
        float* partial = reinterpret_cast<float*>(smem);   // [tile_t][128] when the contraction is split
        const uint32_t accumulators = multi_issue ? min(static_cast<uint32_t>(kGroups), num_kb) : (num_kb > 0 ? 1u : 0u);
        for (uint32_t c = g; c * 32u < tile_t; c += kGroups) {
            float acc[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = 0.0f;   // a CTA without k-blocks contributes zeros
            for (uint32_t a = 0; a < accumulators; ++a) {  // warp-uniform
                uint32_t v[32];
                tmem_ld_32x32(tmem_base + ((quarter * 32u) << 16) + a * kMultiIssueTokens + c * 32u, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[i] += __uint_as_float(v[i]);
            }
#pragma unroll
            for (uint32_t i = 0; i < 32u; ++i) {
                const uint32_t t = c * 32u + i;          // token inside the tile
                if (t < tile_t) {
                    if (ksplit == 1) {
                        if (live && m0 + t < p.m) out[static_cast<uint64_t>(m0 + t) * n_out + n] = acc[i];
                    } else {
                        partial[t * kTileW + row] = acc[i];
                    }
                }
            }
        }
    }
    if (ksplit > 1) {
        // ---- the cluster's partial tiles: every rank sums a slice of the tokens, in rank order ----
        // (the activation stages are free by now: all of this CTA's MMAs have completed)
        cluster.sync();
        const float* mine = reinterpret_cast<const float*>(smem);
        const uint32_t total = tile_t * kTileW;
        for (uint32_t i = tid + krank * kThreads; i < total; i += kThreads * ksplit) {
            const uint32_t t = i / kTileW, row = i % kTileW;
            float v = 0.0f;
            for (uint32_t r = 0; r < ksplit; ++r) v += cluster.map_shared_rank(mine, r)[i];
            if (n0 + row < n_out && m0 + t < p.m) out[static_cast<uint64_t>(m0 + t) * n_out + n0 + row] = v;
        }
        cluster.sync();
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

}  // namespace

// Forward only; whole 64-wide contraction blocks inside one scale block, 16-byte aligned rows.
bool nf4_gemm_tmem_supported(const WeightView& w, const float* x, uint64_t rows) {
    return rows >= 1 && w.in_features % kBK == 0 && w.block_size >= 64 &&
           (reinterpret_cast<uintptr_t>(w.codes) & 15u) == 0 && (w.in_features / 2) % 16 == 0 &&
           (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && encode_tiled() != nullptr &&
           rows <= 0x7FFFFFFFull && w.out_features <= 0x7FFFFFFFull && w.in_features <= 0x7FFFFFFFull;
}

size_t nf4_gemm_tmem_workspace_bytes(const WeightView& w, uint64_t rows) {
    return static_cast<size_t>(rows) * w.in_features * 2;   // bf16 copy of the activations
}

// `x_bf16` is the bf16 copy of the activations (rows * in * 2 bytes), already converted. Applies
// `count` (<= 4) weights with the same in_features to it in one launch; ys[i] is [rows, out_i].
int32_t launch_nf4_gemm_tmem_multi(const DeviceContext& ctx, const WeightView* ws, float* const* ys, uint32_t count,
                                   const void* x_bf16, uint64_t rows, cudaStream_t stream) {
    if (count == 0 || count > static_cast<uint32_t>(kMaxWeights)) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "between one and four weights per launch");
    }
    Params p;
    uint64_t weight_tiles = 0;
    for (uint32_t i = 0; i < static_cast<uint32_t>(kMaxWeights); ++i) {
        const uint32_t src = i < count ? i : 0;
        p.w[i] = ws[src];
        p.out[i] = ys[src];
        p.n[i] = static_cast<uint32_t>(ws[src].out_features);
        if (i < count) weight_tiles += (ws[i].out_features + kTileW - 1) / kTileW;
        p.tile_end[i] = static_cast<uint32_t>(weight_tiles);
    }
    p.count = count;
    p.m = static_cast<uint32_t>(rows);
    p.k = static_cast<uint32_t>(ws[0].in_features);
    p.tile_t = rows >= kMaxTileT ? kMaxTileT : static_cast<uint32_t>((rows + 15) / 16 * 16);
    const uint32_t total_kb = p.k / kBK;
    const uint64_t tiles = weight_tiles * ((rows + p.tile_t - 1) / p.tile_t);
    // Few tiles (a handful of tokens against a weight of a few thousand rows): split the
    // contraction over a cluster so that most SMs take part; the ranks' partial tiles are summed
    // through distributed shared memory in rank order.
    uint32_t ksplit = 1;
    while (ksplit < 8 && tiles * (ksplit * 2) <= static_cast<uint64_t>(ctx.sm_count) && total_kb / (ksplit * 2) >= 8) {
        ksplit *= 2;
    }
    p.kb_per_cta = (total_kb + ksplit - 1) / ksplit;
    p.error = ctx.gemm_error;
    p.lut = ctx.gemm_lut;

    CUtensorMap map;
    const cuuint64_t dims[2] = {ws[0].in_features, rows};
    const cuuint64_t strides[1] = {ws[0].in_features * 2};
    const cuuint32_t box[2] = {kBK, p.tile_t};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode_tiled()(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x_bf16), dims,
                                      strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B2_STATUS_RUNTIME_ERROR, "cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
    static PerDeviceOnce configured;
    B2_TRY(once_per_device(configured, ctx.device, []() -> int32_t {
        B2_CUDA_TRY(cudaFuncSetAttribute(nf4_gemm_tmem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        return B2_STATUS_OK;
    }));
    cudaLaunchConfig_t config = {};
    // weight-row tiles vary fastest: CTAs that run together share the activation tile in L2
    config.gridDim = dim3(static_cast<unsigned>(weight_tiles), static_cast<unsigned>((rows + p.tile_t - 1) / p.tile_t),
                          ksplit);
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = kSmemBytes;
    config.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = ksplit;
    // The kernel calls griddepcontrol.wait before it touches a caller tensor, so it may be
    // scheduled while the conversion pre-pass drains.
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = 2;
    B2_CUDA_TRY(cudaLaunchKernelEx(&config, nf4_gemm_tmem_kernel, map, p));
    return B2_STATUS_OK;
}

int32_t launch_nf4_gemm_tmem(const DeviceContext& ctx, const WeightView& w, const void* x_bf16, float* y,
                             uint64_t rows, cudaStream_t stream) {
    float* ys[1] = {y};
    return launch_nf4_gemm_tmem_multi(ctx, &w, ys, 1, x_bf16, rows, stream);
}

}  // namespace b2
