// Packed-NF4 linear on the 5th-generation tensor cores with the expanded weight tile in SHARED
// memory:
//   backward  dX[M, in] = dY[M, out] * W[out, in]      (in use for 33..511 rows; from 512 rows
//                                                      nf4_backward_dense.cu)
//   (the template's forward form, Y = X * W^T, is not instantiated: the library's forward
//   calls go to nf4_gemm_tmem.cu and nf4_decode_tmem.cu)
// (reference loops: src/core/backend/nn/quantized_linear/reference/operations.cpp:49-115).
//
// One CTA owns a 256 x 256 output tile as two 128 x 256 FP32 accumulators in
// tensor memory (all 512 TMEM columns). The left operand (activations, first
// converted to bf16 by a streaming pre-pass into caller scratch) arrives by TMA
// in 128-byte-swizzled K-major tiles; the packed weights are read straight from
// global memory by sixteen dequantisation warps, expanded through a per-lane
// replicated byte -> bf16x2 table, multiplied by their block scale and written
// to shared memory in the same swizzled K-major layout, so the weights exist
// as bf16 only inside the SM. One thread issues tcgen05.mma (M128 N256 K16,
// bf16 x bf16 -> f32); completion is tracked with mbarriers through
// tcgen05.commit. Every mbarrier wait is bounded and reports a timeout in a
// status word instead of spinning.
//
// Tensor-pipe bound in principle: 2*M*out*in flops per launch. In practice the 128 B/clk
// shared-memory port (weight tile written, then read twice by the MMAs, plus the activation tile
// and the table lookups) and the issuing thread's two waits and two commits per k-block set the
// pace: about half of the tensor peak.
#include "b2_common.cuh"
#include "b2_kernels.h"
#include "sm100_ptx.cuh"

#include <cuda_bf16.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

namespace b2 {
namespace {

using namespace sm100;

constexpr int kBM = 256, kBN = 256, kBK = 64;
constexpr int kStagesA = 3, kStagesB = 2;
constexpr int kStageABytes = kBM * kBK * 2;   // 32 KB
constexpr int kStageBBytes = kBN * kBK * 2;   // 32 KB
constexpr int kLutBytes = 256 * 128;          // byte -> bf16x2, one copy per lane (128-byte rows)
constexpr int kDequantWarps = 16;
constexpr int kThreads = (2 + kDequantWarps) * 32;
constexpr int kSmemBytes = kStagesA * kStageABytes + kStagesB * kStageBBytes + kLutBytes + 32768 /* table alignment */;
constexpr uint32_t kTmemColumns = 512;

struct GemmParams {
    WeightView w;
    float* out;          // [M, N] fp32
    uint32_t m, n, k;    // output rows, output columns, contraction length
    uint32_t* error;     // device word: bit 0 set when a barrier wait timed out
    const uint32_t* lut; // compact [256][32] words of bf16 pairs
};

struct Barriers {
    uint64_t full_a[kStagesA];
    uint64_t empty_a[kStagesA];
    uint64_t full_b[kStagesB];
    uint64_t empty_b[kStagesB];
    uint64_t acc_full;
    uint32_t tmem_base;
    uint32_t abort;
};

__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
    __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}

// Table read (the table is constant after the kernel's first barrier): not volatile, so the
// lookups of later chunks can be scheduled ahead of the stores of earlier ones.
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

// Eight weights (one packed word) -> four bf16 pairs, scaled. `lut_lane` is the
// 32 KB-aligned table base + 4*lane; entry v sits at v*128.
__device__ __forceinline__ uint4 expand_word(uint32_t word, uint32_t lut_lane, uint32_t scale2) {
    uint4 r;
    r.x = bf16x2_mul(lds_u32(((word << 7) & 0x7F80u) | lut_lane), scale2);
    r.y = bf16x2_mul(lds_u32(((word >> 1) & 0x7F80u) | lut_lane), scale2);
    r.z = bf16x2_mul(lds_u32(((word >> 9) & 0x7F80u) | lut_lane), scale2);
    r.w = bf16x2_mul(lds_u32(((word >> 17) & 0x7F80u) | lut_lane), scale2);
    return r;
}

__device__ __forceinline__ uint32_t scale_pair(float s) {
    __nv_bfloat162 p = __float2bfloat162_rn(s);
    return *reinterpret_cast<uint32_t*>(&p);
}

// A block scale as it sits in memory, fetched ahead of its use. Decoding (table lookup, multiply,
// add, clamp) is left to the moment the scale is needed: doing it right after the loads would
// stall the thread for a full trip to memory in every k-block.
struct RawScale {
    uint32_t bits;   // FP32 scale bits, or the scale code
    float second;    // second-level value (double-quantised scales)
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
// `factor` is the 256-entry table (code - 128) / 127 in shared memory.
__device__ __forceinline__ float finish_raw_scale(const WeightView& w, const RawScale& s, const float* factor) {
    return w.encoding == B2_SCALES_FLOAT32 ? __uint_as_float(s.bits) : dq_finish(factor[s.bits], s.second, w.offset);
}

// fp32 -> bf16 row-major copy of the left operand (streaming pre-pass).
__global__ void __launch_bounds__(256)
f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, uint64_t n4) {
    pdl_launch_dependents();   // the GEMM that follows may start its set-up now
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(src) + i);
        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&lo);
        packed.y = *reinterpret_cast<uint32_t*>(&hi);
        reinterpret_cast<uint2*>(dst)[i] = packed;
    }
}

// Forward dequantisation of one 256 x 64 weight tile: thread r owns weight row
// n0 + r, i.e. one 128-byte row of the K-major B tile (8 chunks of 8 weights).
struct ForwardRow {
    const uint8_t* codes;   // this row's packed codes (nullptr past the last row)
    uint64_t flat0;         // flat index of the row's first weight
};

// Two threads per weight row: thread (row, hf) expands chunks 4*hf .. 4*hf+3 (32 weights).
__device__ __forceinline__ void dequant_forward(const ForwardRow& row, uint32_t trow, uint32_t hf, uint4 c0,
                                                float scale, uint32_t b_stage32, uint32_t lut_lane) {
    const uint32_t s2 = scale_pair(scale);
    const uint32_t words[4] = {c0.x, c0.y, c0.z, c0.w};
    const uint32_t row32 = b_stage32 + trow * 128u;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (row.codes != nullptr) v = expand_word(words[c], lut_lane, s2);
        sts_u4(row32 + (((4u * hf + static_cast<uint32_t>(c)) ^ (trow & 7u)) << 4), v);
    }
}

// Backward: the B tile is W[o0 .. o0+64, n0 .. n0+256] read "transposed": shared-memory row n holds
// the 64 contraction values (output rows o) of input column n. Lane (kg = lane % 8, cgl = lane / 8)
// of dequant warp w owns the 8 x 8 sub-block rows o0 + 8*kg .. +8, columns n0 + 8*(4*w + cgl) .. +8:
// it loads one packed word (8 columns) per output row, pairs the words of two consecutive rows
// nibble by nibble into byte indices, so one table lookup yields the (o, o+1) bf16 pair of one
// column - already in K order - and stores one 16-byte chunk per column. The 8 lanes that share
// a column group fill one whole 128-byte row per store instruction (no bank conflicts).
struct BackwardState {
    uint32_t words[4];   // packed word of each of this thread's 4 output rows (8 input columns each)
    RawScale raw;        // scale this thread decodes for the CTA: (o = r % 64, in-block = r / 64), r < 256
    bool has_scale;
};

__device__ __forceinline__ void backward_fetch(const GemmParams& p, uint32_t kb, uint32_t n0, uint32_t r,
                                               uint32_t kg, uint32_t hf, uint32_t cg, BackwardState& st) {
    const uint64_t in = p.w.in_features;
    const uint32_t col = n0 + 8u * cg;
    const uint64_t o_base = static_cast<uint64_t>(kb) * kBK + 8u * kg + 4u * hf;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        st.words[i] = 0x77777777u;
        if (col < p.n) {
            st.words[i] = __ldg(reinterpret_cast<const uint32_t*>(p.w.codes + (((o_base + i) * in + col) >> 1)));
        }
    }
    st.raw.bits = 0u;
    st.raw.second = 0.0f;
    st.has_scale = false;
    if (r < 256u) {
        const uint32_t so = r & 63u, sib = r >> 6;
        if (n0 + 64u * sib < p.n) {
            const uint64_t flat = (static_cast<uint64_t>(kb) * kBK + so) * in + n0 + 64u * sib;
            st.raw = fetch_raw_scale(p.w, flat >> p.w.block_shift);
            st.has_scale = true;
        }
    }
}

template <bool kBackward>
__global__ void __launch_bounds__(kThreads, 1)
nf4_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const GemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    __shared__ __align__(8) Barriers bars;
    __shared__ __align__(16) __nv_bfloat16 s_scales[2][4][64];   // backward: [parity][in-block][output row]
    __shared__ float s_factor[256];                              // scale code -> (code - 128) / 127
    const uint32_t raw32 = smem_u32(smem_raw);
    const uint32_t base32 = (raw32 + 1023u) & ~1023u;
    const uint32_t a32 = base32;
    const uint32_t b32 = base32 + kStagesA * kStageABytes;
    const uint32_t lut32 = (b32 + kStagesB * kStageBBytes + 32767u) & ~32767u;
    uint8_t* smem = smem_raw + (base32 - raw32);

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t m0 = blockIdx.y * kBM, n0 = blockIdx.x * kBN;
    const uint32_t num_kb = p.k / kBK;
    volatile uint32_t* abort = &bars.abort;

    if (warp == 0) {
        if (lane == 0) {
            for (int s = 0; s < kStagesA; ++s) {
                mbar_init(&bars.full_a[s], 1);
                mbar_init(&bars.empty_a[s], 1);
            }
            for (int s = 0; s < kStagesB; ++s) {
                mbar_init(&bars.full_b[s], kDequantWarps);
                mbar_init(&bars.empty_b[s], 1);
            }
            mbar_init(&bars.acc_full, 1);
            bars.abort = 0;
            mbar_fence_init();
            tma_prefetch_descriptor(&map_a);
        }
        __syncwarp();
        tmem_alloc(&bars.tmem_base, kTmemColumns);
    }
    // byte table: straight 32 KB copy (entry v at v*128 + 4*lane)
    for (uint32_t i = tid; i < kLutBytes / 16; i += kThreads) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(p.lut) + i);
        sts_u4(lut32 + i * 16u, v);
    }
    if (tid < 256) s_factor[tid] = dq_factor(tid);
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = bars.tmem_base;

    if (warp == 0) {
        // ---- TMA producer: activation tiles ----
        if (lane == 0) {
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                const uint32_t s = kb % kStagesA;
                if (kb >= kStagesA) mbar_wait(&bars.empty_a[s], ((kb / kStagesA) - 1u) & 1u, abort);
                mbar_expect_tx(&bars.full_a[s], kStageABytes);
                tma_load_2d(smem + s * kStageABytes, &map_a, static_cast<int>(kb * kBK), static_cast<int>(m0),
                            &bars.full_a[s]);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16_f32(128, kBN);
            // Descriptors differ only in the start-address field (address / 16, the low 14 bits):
            // build one per operand here and add offsets in the loop. This thread's instruction
            // stream is the pace of the whole CTA, so it is kept to a few instructions per MMA.
            const uint64_t da0 = umma_desc_k_major_sw128(a32), db0 = umma_desc_k_major_sw128(b32);
            uint32_t s = 0, j = 0, pa = 0, pb = 0;
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                mbar_wait(&bars.full_a[s], pa, abort);
                mbar_wait(&bars.full_b[j], pb, abort);
                tcgen05_fence_after_sync();
                const uint64_t da_s = da0 + ((s * static_cast<uint32_t>(kStageABytes)) >> 4);
                const uint64_t db_s = db0 + ((j * static_cast<uint32_t>(kStageBBytes)) >> 4);
#pragma unroll
                for (uint32_t h = 0; h < 2; ++h) {
#pragma unroll
                    for (uint32_t k = 0; k < kBK / 16; ++k) {
                        umma_bf16(tmem_base + h * 256u, da_s + ((h * 16384u + k * 32u) >> 4), db_s + ((k * 32u) >> 4),
                                  idesc, (kb | k) != 0u ? 1u : 0u);
                    }
                }
                umma_commit(&bars.empty_a[s]);
                umma_commit(&bars.empty_b[j]);
                if (++s == kStagesA) {
                    s = 0;
                    pa ^= 1u;
                }
                if (++j == kStagesB) {
                    j = 0;
                    pb ^= 1u;
                }
            }
            umma_commit(&bars.acc_full);
        }
    } else {
        // ---- dequantisation warps, then epilogue ----
        const uint32_t r = tid - 64u;
        const uint32_t lut_lane = lut32 | (lane * 4u);
        if (!kBackward) {
            const uint32_t trow = r >> 1, hf = r & 1u;
            const uint32_t n = n0 + trow;
            ForwardRow row;
            row.codes = n < p.n ? p.w.codes + static_cast<uint64_t>(n) * (p.k >> 1) + hf * 16u : nullptr;
            row.flat0 = static_cast<uint64_t>(n) * p.k;
            // Packed codes and raw scales are fetched two k-blocks ahead: under load a trip to HBM
            // takes longer than one k-block of expansion.
            uint4 c0 = make_uint4(0, 0, 0, 0), c1 = c0;
            RawScale raw0 = {0u, 0.0f}, raw1 = raw0;
            if (row.codes != nullptr) {
                c0 = ldg_u4(row.codes);
                raw0 = fetch_raw_scale(p.w, row.flat0 >> p.w.block_shift);
                if (num_kb > 1) {
                    c1 = ldg_u4(row.codes + 32u);
                    raw1 = fetch_raw_scale(p.w, (row.flat0 + kBK) >> p.w.block_shift);
                }
            }
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                const uint32_t j = kb % kStagesB;
                uint4 c2 = make_uint4(0, 0, 0, 0);
                RawScale raw2 = {0u, 0.0f};
                if (row.codes != nullptr && kb + 2 < num_kb) {
                    c2 = ldg_u4(row.codes + (kb + 2) * 32u);
                    raw2 = fetch_raw_scale(p.w, (row.flat0 + static_cast<uint64_t>(kb + 2) * kBK) >> p.w.block_shift);
                }
                if (kb >= kStagesB) mbar_wait(&bars.empty_b[j], ((kb / kStagesB) - 1u) & 1u, abort);
                const float scale = row.codes != nullptr ? finish_raw_scale(p.w, raw0, s_factor) : 0.0f;
                dequant_forward(row, trow, hf, c0, scale, b32 + j * kStageBBytes, lut_lane);
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars.full_b[j]);
                c0 = c1;
                c1 = c2;
                raw0 = raw1;
                raw1 = raw2;
            }
        } else {
            // lane (kg = lane % 8, cgl = lane / 8) of dequant warp e: column group 4*(e % 8) + cgl,
            // output rows 8*kg + 4*(e / 8) .. +4 of the k-block
            const uint32_t e = warp - 2u;
            const uint32_t kg = lane & 7u, hf = e >> 3, cg = 4u * (e & 7u) + (lane >> 3);
            const uint32_t my_ib = cg >> 3;   // in-block (64 columns) of this thread's 8 columns
            BackwardState cur, nxt;
            backward_fetch(p, 0, n0, r, kg, hf, cg, cur);
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                const uint32_t j = kb % kStagesB, par = kb & 1u;
                if (kb + 1 < num_kb) backward_fetch(p, kb + 1, n0, r, kg, hf, cg, nxt);
                // publish this k-block's 256 decoded scales, then every thread reads its 4 (2 pairs)
                if (r < 256u) {
                    s_scales[par][r >> 6][r & 63u] =
                        __float2bfloat16_rn(cur.has_scale ? finish_raw_scale(p.w, cur.raw, s_factor) : 0.0f);
                }
                asm volatile("bar.sync 1, 512;" ::: "memory");
                const uint2 sc = *reinterpret_cast<const uint2*>(&s_scales[par][my_ib][8u * kg + 4u * hf]);
                const uint32_t sc2[2] = {sc.x, sc.y};
                uint4 even[2], odd[2];   // [row pair] -> columns (0,2,4,6) / (1,3,5,7), each an (o, o+1) pair
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const uint32_t wa = cur.words[2 * i], wb = cur.words[2 * i + 1];
                    const uint32_t idx_e = (wa & 0x0F0F0F0Fu) | ((wb << 4) & 0xF0F0F0F0u);
                    const uint32_t idx_o = ((wa >> 4) & 0x0F0F0F0Fu) | (wb & 0xF0F0F0F0u);
                    even[i] = expand_word(idx_e, lut_lane, sc2[i]);
                    odd[i] = expand_word(idx_o, lut_lane, sc2[i]);
                }
                if (kb >= kStagesB) mbar_wait(&bars.empty_b[j], ((kb / kStagesB) - 1u) & 1u, abort);
                const uint32_t stage32 = b32 + j * kStageBBytes;
                const bool live = n0 + 8u * cg < p.n;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const int q = c >> 1;
                    const uint4& s0 = (c & 1) ? odd[0] : even[0];
                    const uint4& s1 = (c & 1) ? odd[1] : even[1];
                    uint32_t vx = q == 0 ? s0.x : q == 1 ? s0.y : q == 2 ? s0.z : s0.w;
                    uint32_t vy = q == 0 ? s1.x : q == 1 ? s1.y : q == 2 ? s1.z : s1.w;
                    if (!live) vx = vy = 0u;
                    const uint32_t nrow = 8u * cg + static_cast<uint32_t>(c);
                    asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(stage32 + nrow * 128u + ((kg ^ (nrow & 7u)) << 4) + hf * 8u),
                                 "r"(vx), "r"(vy)
                                 : "memory");
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars.full_b[j]);
                cur = nxt;
            }
        }
        // epilogue: TMEM -> registers -> global
        mbar_wait(&bars.acc_full, 0u, abort);
        tcgen05_fence_after_sync();
        const uint32_t quarter = warp & 3u, half = ((warp - 2u) >> 2) & 1u, col_half = (warp - 2u) >> 3;
        const uint32_t row_out = m0 + half * 128u + quarter * 32u + lane;
        for (uint32_t c = col_half * (kBN / 64); c < (col_half + 1u) * (kBN / 64); ++c) {
            uint32_t v[32];
            tmem_ld_32x32(tmem_base + ((quarter * 32u) << 16) + half * 256u + c * 32u, v);
            tmem_ld_wait();
            const uint32_t col0 = n0 + c * 32u;
            if (row_out < p.m && col0 < p.n) {
                float* dst = p.out + static_cast<uint64_t>(row_out) * p.n + col0;
                if (col0 + 32u <= p.n && (p.n & 3u) == 0u) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        reinterpret_cast<float4*>(dst)[i] =
                            make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                        __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
                    }
                } else {
                    for (uint32_t i = 0; i < 32u && col0 + i < p.n; ++i) dst[i] = __uint_as_float(v[i]);
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

__global__ void gemm_lut_init_kernel(uint32_t* lut) {
    // [256][32] words: entry v (replicated for the 32 lanes) = bf16 pair of packed byte v,
    // low nibble's value in the low half.
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= 256 * 32) return;
    const uint32_t v = i >> 5;
    const __nv_bfloat16 lo = __float2bfloat16_rn(kNf4Codebook[v & 15u]);
    const __nv_bfloat16 hi = __float2bfloat16_rn(kNf4Codebook[v >> 4]);
    lut[i] = static_cast<uint32_t>(__bfloat16_as_ushort(lo)) | (static_cast<uint32_t>(__bfloat16_as_ushort(hi)) << 16);
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

// bf16 [rows][cols] row-major, box = 64 columns x 256 rows, 128-byte swizzle, zero fill outside.
int32_t make_operand_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows = kBM) {
    EncodeTiledFn encode = encode_tiled();
    if (encode == nullptr) return fail(B2_STATUS_RUNTIME_ERROR, "cuTensorMapEncodeTiled is not available");
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {kBK, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                              elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B2_STATUS_RUNTIME_ERROR, "cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
    return B2_STATUS_OK;
}

}  // namespace

int32_t init_gemm_lut(DeviceContext* ctx) {
    B2_CUDA_TRY(cudaMalloc(&ctx->gemm_lut, 256 * 32 * 4));
    gemm_lut_init_kernel<<<32, 256>>>(ctx->gemm_lut);
    B2_CUDA_TRY(cudaGetLastError());
    B2_CUDA_TRY(cudaMalloc(&ctx->gemm_error, sizeof(uint32_t)));
    B2_CUDA_TRY(cudaMemset(ctx->gemm_error, 0, sizeof(uint32_t)));
    B2_CUDA_TRY(cudaDeviceSynchronize());
    return B2_STATUS_OK;
}

// fp32 -> bf16 copy of `count` values (a multiple of 4) on `stream`.
int32_t launch_f32_to_bf16(const DeviceContext& ctx, const float* src, void* dst, uint64_t count, cudaStream_t stream) {
    const uint64_t n4 = count / 4;
    uint64_t blocks = (n4 + 255) / 256;
    if (blocks > static_cast<uint64_t>(ctx.sm_count) * 16) blocks = static_cast<uint64_t>(ctx.sm_count) * 16;
    if (blocks == 0) blocks = 1;
    f32_to_bf16_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(src, static_cast<__nv_bfloat16*>(dst), n4);
    B2_CUDA_TRY(cudaGetLastError());
    return B2_STATUS_OK;
}

// The tensor-core path needs whole 64-wide contraction blocks that never
// straddle a scale block, whole bytes per weight row and 16-byte aligned rows.
bool nf4_gemm_supported(const WeightView& w, const float* x, uint64_t rows, bool backward) {
    if (rows <= 32) return false;
    if (backward && (w.out_features % kBK != 0 || (reinterpret_cast<uintptr_t>(w.codes) & 3u) != 0)) return false;
    const uint64_t k = backward ? w.out_features : w.in_features;
    return k % kBK == 0 && w.in_features % 64 == 0 && w.block_size >= 64 &&
           (reinterpret_cast<uintptr_t>(w.codes) & 15u) == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 &&
           rows <= 0x7FFFFFFFull && w.out_features <= 0x7FFFFFFFull && w.in_features <= 0x7FFFFFFFull;
}

size_t nf4_gemm_workspace_bytes(const WeightView& w, uint64_t rows, bool backward) {
    const uint64_t k = backward ? w.out_features : w.in_features;
    return static_cast<size_t>(rows) * k * 2;   // bf16 copy of the left operand
}

int32_t launch_nf4_gemm(const DeviceContext& ctx, const WeightView& w, const float* x, float* y, uint64_t rows,
                        bool backward, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    if (!backward) return fail(B2_STATUS_RUNTIME_ERROR, "internal: this kernel serves the input backward only");
    const uint64_t k = w.out_features;
    const uint64_t n = w.in_features;
    const size_t need = nf4_gemm_workspace_bytes(w, rows, true);
    if (workspace == nullptr || workspace_bytes < need) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 GEMM workspace too small: need %zu bytes", need);
    }
    if ((reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 GEMM workspace must be 16-byte aligned");
    }
    const uint64_t n4 = rows * k / 4;
    uint64_t blocks = (n4 + 255) / 256;
    if (blocks > static_cast<uint64_t>(ctx.sm_count) * 16) blocks = static_cast<uint64_t>(ctx.sm_count) * 16;
    f32_to_bf16_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        x, static_cast<__nv_bfloat16*>(workspace), n4);
    B2_CUDA_TRY(cudaGetLastError());

    CUtensorMap map;
    B2_TRY(make_operand_map(&map, workspace, rows, k));
    static PerDeviceOnce configured;
    B2_TRY(once_per_device(configured, ctx.device, []() -> int32_t {
        B2_CUDA_TRY(cudaFuncSetAttribute(nf4_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemBytes));
        return B2_STATUS_OK;
    }));
    GemmParams p;
    p.w = w;
    p.out = y;
    p.m = static_cast<uint32_t>(rows);
    p.n = static_cast<uint32_t>(n);
    p.k = static_cast<uint32_t>(k);
    p.error = ctx.gemm_error;
    p.lut = ctx.gemm_lut;
    const dim3 grid(static_cast<unsigned>((n + kBN - 1) / kBN), static_cast<unsigned>((rows + kBM - 1) / kBM));
    nf4_gemm_kernel<true><<<grid, kThreads, kSmemBytes, stream>>>(map, p);
    B2_CUDA_TRY(cudaGetLastError());
    return B2_STATUS_OK;
}

}  // namespace b2
