// Decode-batch packed-NF4 linear (1..32 activation rows) on the 5th-generation tensor cores:
//   Y[m, out] = X[m, in] * W[out, in]^T      (reference loop:
//   src/core/backend/nn/quantized_linear/reference/operations.cpp:49-81)
//
// The kernel is bound by how fast the packed weights stream through the SMs, so it is built as
// a persistent weight-streaming pipeline, one CTA per SM:
//
//  * Work items are (128-row weight tile, 256-wide contraction round). The items of a launch -
//    all tiles of up to four weights that share the activations - are numbered tile-major and cut
//    into one contiguous range per CTA (stream-K), so every SM streams the same number of bytes
//    whatever the shape or the shard size. A CTA whose range ends inside a tile leaves a partial
//    tile; the partial tiles of one output tile are summed in a fixed order by whichever CTA
//    finishes last (a counter per tile), so results do not depend on timing.
//  * A launch with few tiles (tiles * 2 <= SMs: the q/k/v, o and down projections of a 7B-shaped
//    layer, and every sharded layer) is split differently: one thread-block cluster per tile, CTA r
//    of k takes the rounds [r * R / k, (r + 1) * R / k), the partial tiles stay in shared memory and
//    the cluster's leader adds them in rank order through distributed shared memory. That replaces
//    the global round trip (store, fence, counter, reload) at the end of such a launch by two
//    cluster barriers.
//  * One thread streams the packed codes ([128 rows x 128 bytes], 128-byte swizzle), the tile's
//    raw block scales and the second-level values they refer to into a shared-memory ring with
//    cp.async.bulk.tensor; weights are immutable, so this starts before the dependency wait of a
//    programmatic dependent launch, i.e. under the previous kernel's tail.
//  * Sixteen expansion warps, in two sets that alternate items, turn a round into its 16-bit
//    operand form: thread (row, half) reads its 64 packed bytes from the ring, looks every byte up
//    in a per-lane replicated byte -> pair table (one PRMT forms the address), multiplies by the
//    block scale and writes the values with two tcgen05.st of 32 columns into the round's stage of
//    TENSOR memory, where the weight tile is the A operand (lane = weight row). Three 256-wide
//    stages keep expansion and MMAs apart.
//  * One warp issues the sixteen tcgen05.mma (M128, N = 16 or 32 tokens, K16) of a round behind
//    ONE barrier wait and commits once per round (warp-convergent loop, the instructions under
//    elect.sync); the activations (16-bit, by TMA) are the B operand in shared memory. Two
//    accumulators alternate between the segments of a CTA's range.
//
// Two operand types share the code: bf16 (activations handed over as bf16, rel-L2 ~3e-3, used
// above 16 rows) and fp16 with an FP32 row normaliser (rel-L2 ~5e-4, used up to 16 rows, where
// the tolerance is 2e-3). Every mbarrier wait is bounded; a timeout sets an error word and the
// kernel drains.
#include "b2_common.cuh"
#include "b2_kernels.h"
#include "sm100_ptx.cuh"

#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <mutex>

namespace cg = cooperative_groups;

namespace b2 {
namespace {

using namespace sm100;

constexpr int kTileW = 128;                       // weight rows per tile (MMA M, TMEM lanes)
constexpr int kRoundK = 256;                      // contraction values per round
constexpr int kMaxTokens = 32;                    // activation rows per launch at most (MMA N)
constexpr int kCodeBytes = kTileW * (kRoundK / 2);            // 16384: packed codes of one item
constexpr int kScaleBoxBytes = kTileW * 16;                   // 2048: 16 bytes of raw scales per row
constexpr int kSecondBox = 128;                               // second-level floats per item
constexpr int kScaleOff = kCodeBytes;
constexpr int kSecondOff = kCodeBytes + kScaleBoxBytes;
constexpr int kWStageBytes = 19 * 1024;                       // codes + scales + second level, 1 KB granular
constexpr int kMaxWStages = 6;
constexpr int kXStages = 4;                                   // activation stages
constexpr int kAStages = 3;                                   // tensor-memory stages of the expanded weights
constexpr int kLutBytes = 65536;                              // 256 rows of 256 bytes (lane l at byte 4*l)
constexpr int kLowHeader = 3072;                              // barriers, slot lists
constexpr int kExpandWarps = 16;
constexpr int kFirstExpandWarp = 3;
constexpr int kThreads = (kFirstExpandWarp + kExpandWarps) * 32;   // 608
constexpr int kExpandThreads = kExpandWarps * 32;
constexpr int kSetWarps = kExpandWarps / 2;                   // the expansion warps form two sets that alternate items
constexpr int kSetThreads = kSetWarps * 32;
constexpr int kSmemBytes = 232448;                            // all of it: the ring takes what the rest leaves
constexpr uint32_t kTmemColumns = 512;
constexpr uint32_t kAccColumns = 128;                         // accumulator region (kMaxTokens used)
constexpr uint32_t kStageColumns = kRoundK / 2;               // 128 columns: one round of 16-bit pairs
constexpr int kMaxWeights = 4;
constexpr int kPartialFloats = kMaxTokens * kTileW;           // one partial tile
// Polls before a wait gives up (a fraction of a second; every wait starts after the dependency wait
// of a programmatic launch, so a healthy one lasts microseconds).
constexpr uint32_t kPollBudget = 400000u;

struct DecodeMaps {
    CUtensorMap codes[kMaxWeights];     // u8 [out, in/2], box {128, 128}, 128-byte swizzle
    CUtensorMap scales[kMaxWeights];    // u8 [out, blocks/row] box {16, 128}  or  f32 box {4, 128}
    CUtensorMap second[kMaxWeights];    // f32 [n_second], box {128}
};

struct DecodeParams {
    WeightView w[kMaxWeights];
    float* out[kMaxWeights];
    uint32_t n[kMaxWeights];
    uint32_t tile_end[kMaxWeights];   // running count of 128-row tiles
    uint32_t count;
    uint32_t m, k;
    uint32_t n_pad;            // 16 or 32: MMA N
    uint32_t rounds;           // k / 256
    uint32_t total_items;      // tiles * rounds
    uint32_t blocks_per_row;   // k >> block_shift
    uint32_t kshift;           // block_shift - 6: 64-wide k-blocks per scale block, as a shift
    uint32_t cluster_k;        // > 1: the CTAs of a cluster of this size split one tile's rounds
    float* partial;            // [2 * gridDim.x][kPartialFloats]
    uint32_t* counters;        // [tiles], zero before the launch; the kernel leaves them zero
    uint32_t* error;
};

struct Barriers {
    uint64_t w_full[kMaxWStages];
    uint64_t w_empty[kMaxWStages];
    uint64_t x_full[kXStages];
    uint64_t x_empty[kXStages];     // tcgen05.commit: the round's MMAs have read the activation stage
    uint64_t a_full[kAStages];
    uint64_t done[kAStages];        // tcgen05.commit: the round's MMAs have read the tensor-memory stage
    uint64_t acc_full[2];           // per accumulator (segment parity): the segment's MMAs have completed
    uint64_t acc_empty[2];          // ... and its epilogue has read the accumulator
    uint32_t tmem_base;
    uint32_t abort;
    uint32_t last_flag[2];          // per expansion set
};
static_assert(sizeof(Barriers) <= 256, "barrier block");

template <bool kHalf>
__device__ __forceinline__ uint32_t pair_mul(uint32_t a, uint32_t b) {
    if (kHalf) {
        __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
        return *reinterpret_cast<uint32_t*>(&r);
    }
    __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}
template <bool kHalf>
__device__ __forceinline__ uint32_t pair_of(float s) {
    if (kHalf) {
        __half2 p = __float2half2_rn(s);
        return *reinterpret_cast<uint32_t*>(&p);
    }
    __nv_bfloat162 p = __float2bfloat162_rn(s);
    return *reinterpret_cast<uint32_t*>(&p);
}

__device__ __forceinline__ uint32_t lds_u32(uint32_t a) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint4 lds_u4(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ float lds_f32(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ float2 lds_f32x2(uint32_t a) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
// (code - 128) / 127 rounded like the IEEE division of dq_factor, without the division: the
// product with the rounded reciprocal, corrected by one Newton step, is the correctly rounded
// quotient for each of the 256 codes (checked exhaustively against the division).
__device__ __forceinline__ float dq_factor_fma(uint32_t scale_code) {
    const float x = static_cast<float>(static_cast<int>(scale_code) - 128);
    const float r = 1.0f / 127.0f;
    const float q0 = __fmul_rn(x, r);
    const float e = __fmaf_rn(-q0, 127.0f, x);
    return __fmaf_rn(e, r, q0);
}
__device__ __forceinline__ uint32_t lds_u8(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void cp_async_16(uint32_t dst32, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst32), "l"(src));
}
__device__ __forceinline__ void tma_2d_at(uint32_t dst32, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst32), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_1d_at(uint32_t dst32, const CUtensorMap* map, int x, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.1d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2}], [%3];"
                 ::"r"(dst32), "l"(map), "r"(x), "r"(smem_u32(bar))
                 : "memory");
}
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
// 32 lanes x 16 consecutive columns: thread i of the warp gets lane (base + i).
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void umma_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Instruction descriptor, kind::f16: 16-bit x 16-bit -> f32, both operands K-major.
__device__ __forceinline__ uint32_t idesc_16bit(bool half, uint32_t m, uint32_t n) {
    const uint32_t fmt = half ? 0u : 1u;   // 0 = f16, 1 = bf16
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
// True in exactly one lane of a converged warp. Loops that issue TMA or tcgen05 instructions run
// on the whole warp with the instruction itself under this predicate: the loop state stays
// warp-uniform, so descriptors and addresses can live in uniform registers.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{ .reg .pred p; elect.sync _|p, 0xFFFFFFFF; selp.u32 %0, 1, 0, p; }" : "=r"(pred));
    return pred != 0;
}
// Named barriers: 1 for all expansion warps, 2 + set for the warps of one set.
__device__ __forceinline__ void expand_barrier() {
    asm volatile("bar.sync 1, %0;" ::"n"(kExpandThreads) : "memory");
}
__device__ __forceinline__ void set_barrier(uint32_t set) {
    asm volatile("bar.sync %0, %1;" ::"r"(2u + set), "n"(kSetThreads) : "memory");
}

// Where the pieces of shared memory lie for this CTA: a pure function of the dynamic allocation's
// address and of the token tile, so every role computes the same answer.
struct SmemPlan {
    uint32_t low32;       // barriers, slot lists
    uint32_t x32;         // activation stages
    uint32_t lut32;       // 64 KB aligned table
    uint32_t high32;      // ring stages behind the table
    uint32_t low_w32;     // ring stages that fit below the table
    uint32_t n_high, n_stages;
    uint32_t x_stage_bytes;
};
__device__ __forceinline__ SmemPlan plan_smem(uint32_t raw32, uint32_t n_pad) {
    SmemPlan s;
    s.low32 = (raw32 + 1023u) & ~1023u;
    s.x32 = s.low32 + kLowHeader;
    s.x_stage_bytes = n_pad * (kRoundK * 2u);
    const uint32_t low_end = s.x32 + kXStages * s.x_stage_bytes;
    s.lut32 = (low_end + 65535u) & ~65535u;
    s.high32 = s.lut32 + kLutBytes;
    const uint32_t end32 = raw32 + kSmemBytes;
    s.n_high = end32 > s.high32 ? (end32 - s.high32) / kWStageBytes : 0u;
    s.low_w32 = (low_end + 1023u) & ~1023u;
    const uint32_t n_low = s.lut32 > s.low_w32 ? (s.lut32 - s.low_w32) / kWStageBytes : 0u;
    s.n_stages = min(s.n_high + n_low, static_cast<uint32_t>(kMaxWStages));
    if (s.n_high > s.n_stages) s.n_high = s.n_stages;
    return s;
}
__device__ __forceinline__ uint32_t w_stage_addr(const SmemPlan& s, uint32_t stage) {
    return stage < s.n_high ? s.high32 + stage * kWStageBytes : s.low_w32 + (stage - s.n_high) * kWStageBytes;
}

// The weight (index, first row of the tile, output width) that owns tile `tile`.
struct TileRef {
    uint32_t wi, n0, n_out;
};
__device__ __forceinline__ TileRef locate_tile(const DecodeParams& p, uint32_t tile) {
    uint32_t wi = 0, base = 0;
#pragma unroll
    for (int i = 1; i < kMaxWeights; ++i) {
        if (static_cast<uint32_t>(i) < p.count && tile >= p.tile_end[i - 1]) {
            wi = static_cast<uint32_t>(i);
            base = p.tile_end[i - 1];
        }
    }
    TileRef t;
    t.wi = wi;
    t.n0 = (tile - base) * kTileW;
    t.n_out = p.n[0];
#pragma unroll
    for (int i = 1; i < kMaxWeights; ++i) {
        if (wi == static_cast<uint32_t>(i)) t.n_out = p.n[i];
    }
    return t;
}

__device__ __forceinline__ uint32_t range_begin(uint32_t cta, uint32_t ctas, uint32_t items) {
    return static_cast<uint32_t>(static_cast<uint64_t>(cta) * items / ctas);
}
// The CTA whose range holds `item`.
__device__ __forceinline__ uint32_t cta_of_item(uint32_t item, uint32_t ctas, uint32_t items) {
    return static_cast<uint32_t>(((static_cast<uint64_t>(item) + 1u) * ctas - 1u) / items);
}

template <bool kHalf>
__global__ void __launch_bounds__(kThreads, 1)
nf4_decode_tmem_kernel(const __grid_constant__ DecodeMaps maps, const __grid_constant__ CUtensorMap map_x,
                       const DecodeParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t raw32 = smem_u32(smem_raw);
    const SmemPlan plan = plan_smem(raw32, p.n_pad);
    uint8_t* low = smem_raw + (plan.low32 - raw32);
    Barriers& bars = *reinterpret_cast<Barriers*>(low);
    uint32_t* s_slots = reinterpret_cast<uint32_t*>(low + 1280);   // partial-tile slots of one output tile (<= 160), per set
    volatile uint32_t* abort = &bars.abort;

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t ctas = gridDim.x, cta = blockIdx.x;
    const uint32_t R = p.rounds;
    // Work split. Few tiles (tiles * 2 <= SMs): a cluster of cluster_k CTAs owns one tile, CTA r of it
    // the rounds [r * R / k, (r + 1) * R / k), and the partial tiles meet in the leader's registers
    // through distributed shared memory. Otherwise stream-K: CTA c takes the c-th equal share of the
    // (tile, round) list, and partial tiles meet in global memory.
    const bool clustered = p.cluster_k > 1u;
    uint32_t item_begin, item_end;
    if (clustered) {
        const uint32_t tile = cta / p.cluster_k, r = cta - tile * p.cluster_k;
        item_begin = tile * R + r * R / p.cluster_k;
        item_end = tile * R + (r + 1u) * R / p.cluster_k;
    } else {
        item_begin = range_begin(cta, ctas, p.total_items);
        item_end = range_begin(cta + 1u, ctas, p.total_items);
    }
    const uint32_t n_stages = plan.n_stages;
    const bool fp32_scales = p.w[0].encoding == B2_SCALES_FLOAT32;

    if (n_stages < 3u) {   // the ring does not fit (never with the sizes this file is built for)
        if (tid == 0 && p.error != nullptr) atomicOr(p.error, 2u);
        return;
    }

    // ---- set-up that touches no caller tensor except the immutable weights ----
    if (warp == 0) {
        if (lane == 0) {
            for (uint32_t s = 0; s < n_stages; ++s) {
                mbar_init(&bars.w_full[s], 1);
                mbar_init(&bars.w_empty[s], kSetWarps);
            }
            for (int s = 0; s < kXStages; ++s) {
                mbar_init(&bars.x_full[s], 1);
                mbar_init(&bars.x_empty[s], 1);
            }
            for (int s = 0; s < kAStages; ++s) {
                mbar_init(&bars.a_full[s], kSetWarps);
                mbar_init(&bars.done[s], 1);
            }
            for (int a = 0; a < 2; ++a) {
                mbar_init(&bars.acc_full[a], 1);
                mbar_init(&bars.acc_empty[a], kSetWarps);
            }
            bars.abort = 0;
            bars.last_flag[0] = bars.last_flag[1] = 0;
            mbar_fence_init();
        }
        __syncwarp();
    } else if (warp == 1) {
        tmem_alloc(&bars.tmem_base, kTmemColumns);
    }
    // byte -> pair table, replicated per lane: entry v for lane l at v * 256 + 4 * l
    // (built here from the sixteen codebook values rather than copied from global memory: a CTA
    // that becomes resident late has this on its critical path, and the copy is an L2 round trip)
    for (uint32_t i = tid; i < 256u * 8u; i += kThreads) {
        const uint32_t v = i >> 3;
        const float lo = kNf4Codebook[v & 15u], hi = kNf4Codebook[v >> 4];
        uint32_t word;
        if (kHalf) {
            const __half2 pair = __floats2half2_rn(lo, hi);
            word = *reinterpret_cast<const uint32_t*>(&pair);
        } else {
            const __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
            word = *reinterpret_cast<const uint32_t*>(&pair);
        }
        asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(plan.lut32 + v * 256u + (i & 7u) * 16u), "r"(word)
                     : "memory");
    }

    const uint32_t w_tx = kCodeBytes + kScaleBoxBytes + (fp32_scales ? 0u : kSecondBox * 4u);
    // Streams item `it` (ring slot `s`): packed codes, raw scales, second-level values.
    auto issue_weights = [&](uint32_t it, uint32_t s) {
        const uint32_t tile = it / R, rho = it - tile * R;
        const TileRef t = locate_tile(p, tile);
        const uint32_t dst = w_stage_addr(plan, s);
        mbar_expect_tx(&bars.w_full[s], w_tx);
        tma_2d_at(dst, &maps.codes[t.wi], static_cast<int>(rho * (kRoundK / 2)), static_cast<int>(t.n0),
                  &bars.w_full[s]);
        const uint32_t blk0 = (4u * rho) >> p.kshift;
        if (fp32_scales) {
            tma_2d_at(dst + kScaleOff, &maps.scales[t.wi], static_cast<int>(blk0 & ~3u), static_cast<int>(t.n0),
                      &bars.w_full[s]);
        } else {
            tma_2d_at(dst + kScaleOff, &maps.scales[t.wi], static_cast<int>(blk0 & ~15u), static_cast<int>(t.n0),
                      &bars.w_full[s]);
            const WeightView& w = p.w[t.wi];
            const uint32_t first = static_cast<uint32_t>(
                (w.flat_block_base + static_cast<uint64_t>(t.n0) * p.blocks_per_row + blk0) >> w.scale_block_shift);
            tma_1d_at(dst + kSecondOff, &maps.second[t.wi], static_cast<int>(first & ~3u), &bars.w_full[s]);
        }
    };
    // The first ring fill goes out before the rest of the CTA has even synchronised.
    uint32_t w_issued = 0;
    if (warp == 0) {
        for (; w_issued < n_stages && item_begin + w_issued < item_end; ++w_issued) {
            if (elect_one()) issue_weights(item_begin + w_issued, w_issued);
            __syncwarp();
        }
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = bars.tmem_base;
    const uint32_t tmem_a = tmem_base + kAccColumns;
    pdl_launch_dependents();

    if (warp == 0) {
        // ---- weight producer ----
        // (its first ring fill is out; every later wait depends on warps that start after the
        // dependency wait, so it joins that wait and its own barrier waits stay short)
        pdl_wait();
        uint32_t s = w_issued == n_stages ? 0u : w_issued, round_trip = w_issued == n_stages ? 1u : 0u;
        for (uint32_t it = item_begin + w_issued; it < item_end; ++it) {
            mbar_wait(&bars.w_empty[s], (round_trip - 1u) & 1u, abort, kPollBudget);
            if (elect_one()) issue_weights(it, s);
            __syncwarp();
            if (++s == n_stages) {
                s = 0;
                ++round_trip;
            }
        }
    } else if (warp == 2) {
        // ---- activation producer: [n_pad tokens x 256] per item as four 64-wide swizzled boxes ----
        pdl_wait();
        uint32_t s = 0, trip = 0, rho = item_begin % R;
        for (uint32_t it = item_begin; it < item_end; ++it) {
            if (trip > 0) mbar_wait(&bars.x_empty[s], (trip - 1u) & 1u, abort, kPollBudget);
            if (elect_one()) {
                mbar_expect_tx(&bars.x_full[s], plan.x_stage_bytes);
                const uint32_t dst = plan.x32 + s * plan.x_stage_bytes;
#pragma unroll
                for (uint32_t b = 0; b < 4u; ++b) {
                    tma_2d_at(dst + b * (p.n_pad * 128u), &map_x, static_cast<int>(rho * kRoundK + b * 64u), 0,
                              &bars.x_full[s]);
                }
            }
            __syncwarp();
            if (++rho == R) rho = 0;
            if (++s == kXStages) {
                s = 0;
                ++trip;
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer: sixteen K16 steps per round behind one wait, one commit per round ----
        pdl_wait();   // nothing it waits for can happen earlier
        const uint32_t idesc = idesc_16bit(kHalf, kTileW, p.n_pad);
        const uint64_t dx0 = umma_desc_k_major_sw128(plan.x32);
        const uint32_t x_stage16 = plan.x_stage_bytes >> 4, kb16 = (p.n_pad * 128u) >> 4;
        uint32_t s = 0, trip = 0, xs = 0, x_trip = 0, rho = item_begin % R, seg = 0;
        for (uint32_t it = item_begin; it < item_end; ++it) {
            const bool first = it == item_begin || rho == 0u;
            const bool last = it + 1u == item_end || rho + 1u == R;
            // Segment s accumulates in accumulator s & 1; before it overwrites that accumulator the
            // epilogue of segment s - 2 must have read it.
            const uint32_t acc_index = seg & 1u;
            if (first && seg > 1u) mbar_wait(&bars.acc_empty[acc_index], ((seg >> 1) - 1u) & 1u, abort, kPollBudget);
            mbar_wait(&bars.a_full[s], trip & 1u, abort, kPollBudget);
            mbar_wait(&bars.x_full[xs], x_trip & 1u, abort, kPollBudget);
            tcgen05_fence_after_sync();
            if (elect_one()) {
                const uint64_t dx_s = dx0 + xs * x_stage16;
                const uint32_t a_s = tmem_a + s * kStageColumns;
#pragma unroll
                for (uint32_t kb = 0; kb < 4u; ++kb) {
#pragma unroll
                    for (uint32_t kk = 0; kk < 4u; ++kk) {
                        umma_a_tmem(tmem_base + acc_index * kMaxTokens, a_s + kb * 32u + kk * 8u,
                                    dx_s + kb * kb16 + kk * 2u, idesc, (first && kb == 0u && kk == 0u) ? 0u : 1u);
                    }
                }
                // the accumulator's barrier first: whoever has seen the stage barrier of a segment's last
                // item complete can rely on the accumulator barrier having completed too
                if (last) umma_commit(&bars.acc_full[acc_index]);
                umma_commit(&bars.done[s]);
                umma_commit(&bars.x_empty[xs]);
            }
            __syncwarp();
            if (last) ++seg;
            if (++rho == R) rho = 0;
            if (++s == kAStages) {
                s = 0;
                ++trip;
            }
            if (++xs == kXStages) {
                xs = 0;
                ++x_trip;
            }
        }
    } else {
        // ---- expansion warps ----
        // Two sets of eight warps alternate items (set 0 takes the CTA's items 0, 2, 4, ..., set 1
        // the others), so while one set waits for its tensor-memory stores the other is looking
        // bytes up. Inside a set, thread (row, half h) expands k-blocks 2h and 2h+1 of the item:
        // 64 packed bytes, in two passes of 32 through the same registers.
        // Expansion reads only the immutable weights, so it starts before the dependency wait of a
        // programmatic launch and runs up to three items ahead; the wait comes before the first
        // epilogue, which is the first thing here to touch memory an earlier kernel may write.
        // Waits that depend on the MMAs (and through them on the activations) come after it too, so
        // that no bounded wait has to outlast the previous kernel.
        bool dependency_waited = false;
        auto depend = [&] {
            if (!dependency_waited) {
                pdl_wait();
                dependency_waited = true;
            }
        };
        const uint32_t e = warp - kFirstExpandWarp;
        const uint32_t set = e >> 3;
        const uint32_t h = (e >> 2) & 1u;
        const uint32_t quarter = warp & 3u;           // the TMEM lanes this warp may touch
        const uint32_t row = quarter * 32u + lane;    // weight row of the tile = TMEM lane
        const uint32_t lut_lane = plan.lut32 | (lane * 4u);
        const uint32_t lane_addr = (quarter * 32u) << 16;
        const uint32_t sshift = p.w[0].scale_block_shift;
        // This thread's four 16-byte chunks inside a swizzled [128 x 128 B] box: chunk c of the row's
        // half h lies at ((4h + c) ^ (row & 7)) * 16, which is code_base + ((c ^ (row & 3)) << 4).
        const uint32_t code_base = row * 128u + (((4u * h) ^ (row & 4u)) << 4);
        const uint32_t code_low = (row & 3u) << 4;
        auto code_off = [&](uint32_t c) { return code_base + ((c << 4) ^ code_low); };

        const uint32_t n_items = item_end - item_begin;
        uint32_t ws = set, w_trip = 0;                 // ring slot / trip of this set's current item
        uint32_t as = set, a_trip = 0;                 // tensor-memory stage / trip
        TileRef tref = {0u, 0u, 0u};
        float dq_offset = 0.0f;
        uint32_t fbase_tile = 0, fbase_row = 0;        // flat index of the first scale block of the tile / of this row
        bool live = false;
        float inv_norm = 1.0f, norm = 1.0f;
        uint32_t stage32 = 0;
        uint32_t v[32];

        // Decoded scales of this thread's two k-blocks (blocks `b0` and `b1` of its row; b1 is b0 or
        // b0 + 1) from the raw values in the current ring slot. A row's raw scales are 16 bytes apart,
        // so every load here costs a warp four shared-memory wavefronts: both values come with one
        // load where they are neighbours, and the code -> factor step is arithmetic
        // ((code - 128) / 127, correctly rounded by one Newton step: exact for all 256 codes).
        auto block_scales = [&](uint32_t b0, uint32_t b1, uint32_t blk0, float& s0, float& s1) {
            if (fp32_scales) {
                const uint32_t at = stage32 + kScaleOff + row * 16u + (b0 - (blk0 & ~3u)) * 4u;
                if (b1 != b0 && (b0 & 1u) == 0u) {
                    const float2 both = lds_f32x2(at);
                    s0 = both.x;
                    s1 = both.y;
                } else {
                    s0 = lds_f32(at);
                    s1 = b1 != b0 ? lds_f32(at + 4u) : s0;
                }
                return;
            }
            const uint32_t at = stage32 + kScaleOff + row * 16u + (b0 - (blk0 & ~15u));
            uint32_t code0, code1;
            if (b1 != b0 && (b0 & 1u) == 0u) {
                const uint32_t both = lds_u16(at);
                code0 = both & 0xFFu;
                code1 = both >> 8;
            } else {
                code0 = lds_u8(at);
                code1 = b1 != b0 ? lds_u8(at + 1u) : code0;
            }
            const uint32_t first = ((fbase_tile + blk0) >> sshift) & ~3u;
            const uint32_t idx0 = ((fbase_row + b0) >> sshift) - first;
            const uint32_t idx1 = ((fbase_row + b1) >> sshift) - first;
            // (the second-level values are the same for nearly every lane: broadcast loads)
            s0 = dq_finish(dq_factor_fma(code0), lds_f32(stage32 + kSecondOff + idx0 * 4u), dq_offset);
            s1 = dq_finish(dq_factor_fma(code1), lds_f32(stage32 + kSecondOff + idx1 * 4u), dq_offset);
        };
        // Looks one k-block's 32 bytes up into v, scaled.
        auto lookup = [&](const uint4& c0, const uint4& c1, float scale) {
            const uint32_t s2 = pair_of<kHalf>(scale);
            const uint32_t words[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const uint32_t word = words[q];
                v[4 * q + 0] = pair_mul<kHalf>(lds_u32(__byte_perm(word, lut_lane, 0x7604u)), s2);
                v[4 * q + 1] = pair_mul<kHalf>(lds_u32(__byte_perm(word, lut_lane, 0x7614u)), s2);
                v[4 * q + 2] = pair_mul<kHalf>(lds_u32(__byte_perm(word, lut_lane, 0x7624u)), s2);
                v[4 * q + 3] = pair_mul<kHalf>(lds_u32(__byte_perm(word, lut_lane, 0x7634u)), s2);
            }
        };
        uint4 second_c0, second_c1;      // packed bytes of the item's second pass
        float second_scale = 0.0f;
        // First pass of item (tile, rho): waits for the ring slot, reads the thread's 64 packed bytes
        // and its two scales, expands k-block 2h into v and keeps the rest for the second pass.
        auto begin_item = [&](uint32_t tile, uint32_t rho, bool new_tile) {
            if (new_tile) {
                tref = locate_tile(p, tile);
                const WeightView& w = p.w[tref.wi];
                dq_offset = w.offset;
                fbase_tile = static_cast<uint32_t>(w.flat_block_base) + tref.n0 * p.blocks_per_row;
                fbase_row = fbase_tile + row * p.blocks_per_row;
                live = tref.n0 + row < tref.n_out;
            }
            stage32 = w_stage_addr(plan, ws);
            mbar_wait(&bars.w_full[ws], w_trip & 1u, abort, kPollBudget);
            const uint4 c0 = lds_u4(stage32 + code_off(0u));
            const uint4 c1 = lds_u4(stage32 + code_off(1u));
            second_c0 = lds_u4(stage32 + code_off(2u));
            second_c1 = lds_u4(stage32 + code_off(3u));
            const uint32_t blk0 = (4u * rho) >> p.kshift;
            float scale = 0.0f;
            second_scale = 0.0f;
            if (live) {
                block_scales((4u * rho + 2u * h) >> p.kshift, (4u * rho + 2u * h + 1u) >> p.kshift, blk0, scale,
                             second_scale);
                if (kHalf) {
                    scale *= inv_norm;
                    second_scale *= inv_norm;
                }
            }
            lookup(c0, c1, scale);
        };

        // Segments (runs of items inside one tile) are numbered from the CTA's first item: an item of
        // tile T lies in segment T - tile_begin, which starts at rho_begin in the first tile and at 0
        // in every later one.
        const uint32_t tile_begin = item_begin / R, rho_begin = item_begin - tile_begin * R;
        uint32_t tile = (item_begin + set) / R, rho = (item_begin + set) - tile * R;
        if (kHalf) {
            // Keep the fp16 operand in range whatever the magnitude of the weights: every expanded
            // value of this CTA is divided by one power of two, taken from the first scale of the
            // CTA's first item (row 0 of its tile), and the sums are multiplied back in the epilogue.
            const TileRef t0 = locate_tile(p, tile_begin);
            mbar_wait(&bars.w_full[0], 0u, abort, kPollBudget);
            const uint32_t s0 = w_stage_addr(plan, 0u);
            const uint32_t blk0 = (4u * rho_begin) >> p.kshift;
            float first_scale;
            if (fp32_scales) {
                first_scale = lds_f32(s0 + kScaleOff + (blk0 - (blk0 & ~3u)) * 4u);
            } else {
                const uint32_t code = lds_u8(s0 + kScaleOff + (blk0 - (blk0 & ~15u)));
                const uint32_t fb = static_cast<uint32_t>(p.w[t0.wi].flat_block_base) + t0.n0 * p.blocks_per_row;
                const uint32_t idx = ((fb + blk0) >> sshift) - (((fb + blk0) >> sshift) & ~3u);
                first_scale = dq_finish(dq_factor_fma(code), lds_f32(s0 + kSecondOff + idx * 4u), p.w[t0.wi].offset);
            }
            const uint32_t bits = __float_as_uint(first_scale) & 0x7F800000u;
            norm = (bits == 0u || bits == 0x7F800000u) ? 1.0f : __uint_as_float(bits);
            inv_norm = 1.0f / norm;
            expand_barrier();   // every warp has read slot 0 before set 0 may release it
        }
        if (set < n_items) begin_item(tile, rho, true);
        for (uint32_t j = set; j < n_items; j += 2u) {
            const uint32_t it = item_begin + j;
            if (a_trip > 0) depend();
            // ---- publish item j: both passes into tensor-memory stage `as` ----
            if (a_trip > 0) mbar_wait(&bars.done[as], (a_trip - 1u) & 1u, abort, kPollBudget);
            tcgen05_fence_after_sync();
            const uint32_t taddr = tmem_a + as * kStageColumns + h * 64u + lane_addr;
            tmem_st_32x32(taddr, v);
            lookup(second_c0, second_c1, second_scale);
            // the ring slot is free once every warp of the set has its bytes in registers
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.w_empty[ws]);
            tmem_st_32x32(taddr + 32u, v);
            // what the epilogue of item j needs, before the next item replaces it
            const uint32_t cur_tile = tile, cur_rho = rho, cur_seg = tile - tile_begin;
            const uint32_t cur_first_rho = tile == tile_begin ? rho_begin : 0u;
            const TileRef cur_ref = tref;
            const bool cur_live = live;
            const bool seg_ends = it + 1u == item_end || rho + 1u == R;
            // Publish before the next item is touched: a tensor-memory stage comes back only after the
            // MMAs that read it, so the time from "stage free" to "stage published" sets the pace of
            // the whole pipeline and must not contain the next item's lookups.
            tmem_st_wait();
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.a_full[as]);
            // ---- start this set's next item (j + 2) ----
            ws += 2u;
            if (ws >= n_stages) {
                ws -= n_stages;
                ++w_trip;
            }
            if (j + 2u < n_items) {
                bool new_tile = false;
                for (uint32_t step = 0; step < 2u; ++step) {   // walk two items ahead
                    if (rho + 1u == R) {
                        rho = 0;
                        ++tile;
                        new_tile = true;
                    } else {
                        ++rho;
                    }
                }
                begin_item(tile, rho, new_tile);
            }
            as += 2u;
            if (as >= kAStages) {
                as -= kAStages;
                ++a_trip;
            }
            if (!seg_ends) continue;

            // ---- epilogue of the segment [cur_first_rho, cur_rho] of tile cur_tile (this set's warps) ----
            // Segment s uses accumulator s & 1 and is phase s >> 1 of that accumulator's barrier. A parity
            // wait can only tell a phase from the one before it, so the phase before (segment s - 2) must
            // be complete when this wait starts: it is, because this set has published the segment's
            // last item, which lies at least three items after the end of segment s - 2 (tiles have two
            // or more rounds) and so reused a tensor-memory stage that segment s - 2's last MMAs released
            // - and those committed to the accumulator barrier first.
            depend();
            mbar_wait(&bars.acc_full[cur_seg & 1u], (cur_seg >> 1) & 1u, abort, kPollBudget);
            tcgen05_fence_after_sync();
            const bool whole = cur_first_rho == 0u && cur_rho + 1u == R;
            float* out = p.out[0];
#pragma unroll
            for (int i = 1; i < kMaxWeights; ++i) {
                if (cur_ref.wi == static_cast<uint32_t>(i)) out = p.out[i];
            }
            const uint32_t n = cur_ref.n0 + row;
            const uint32_t slot = 2u * cta + (item_begin < cur_tile * R ? 1u : 0u);
            // (in a cluster the partial tile stays in this CTA's shared memory: ring slot 0, which is
            // free because the segment's last MMAs, and with them every item of this CTA, are complete)
            float* partial = clustered ? reinterpret_cast<float*>(smem_raw + (w_stage_addr(plan, 0u) - raw32))
                                       : p.partial + static_cast<uint64_t>(slot) * kPartialFloats;
            if (h * 16u < p.n_pad) {
                uint32_t r[16];
                tmem_ld_32x16(tmem_base + (cur_seg & 1u) * kMaxTokens + lane_addr + h * 16u, r);
                tmem_ld_wait();
#pragma unroll
                for (uint32_t i = 0; i < 16u; ++i) {
                    const uint32_t t = h * 16u + i;
                    float val = __uint_as_float(r[i]);
                    if (kHalf) val *= norm;
                    if (t < p.m) {
                        if (whole) {
                            if (cur_live) out[static_cast<uint64_t>(t) * cur_ref.n_out + n] = val;
                        } else {
                            partial[t * kTileW + row] = val;
                        }
                    }
                }
            }
            // the accumulator may now be overwritten by the first MMA of the segment after next
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.acc_empty[cur_seg & 1u]);
            if (!whole && !clustered) {
                // Publish the partial tile; the CTA that arrives last sums all of them in CTA order.
                const uint32_t c_first = cta_of_item(cur_tile * R, ctas, p.total_items);
                const uint32_t c_last = cta_of_item(cur_tile * R + R - 1u, ctas, p.total_items);
                __threadfence();
                set_barrier(set);
                if ((e & 7u) == 0u && lane == 0) {
                    const uint32_t old = atomicAdd(&p.counters[cur_tile], 1u);
                    bars.last_flag[set] = old == c_last - c_first ? 1u : 0u;
                }
                set_barrier(set);
                if (bars.last_flag[set] != 0u) {
                    __threadfence();
                    const uint32_t st = (e & 7u) * 32u + lane;       // thread index inside the set
                    uint32_t* slots = s_slots + set * 160u;
                    const uint32_t parts = c_last - c_first + 1u;
                    // where each part of this tile lies (a 64-bit division per part, done once)
                    for (uint32_t c = st; c < parts; c += kSetThreads) {
                        const uint32_t cc = c_first + c;
                        slots[c] = 2u * cc + (range_begin(cc, ctas, p.total_items) < cur_tile * R ? 1u : 0u);
                    }
                    set_barrier(set);
                    // Four floats per thread and step; the loads of up to eight parts are in flight
                    // together (their sum order is still part 0, 1, 2, ...). Deliberately narrow: more
                    // loads in flight would need registers the expansion loop cannot spare.
                    const uint32_t total4 = p.m * (kTileW / 4);
                    for (uint32_t i4 = st; i4 < total4; i4 += kSetThreads) {
                        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                        for (uint32_t c0 = 0; c0 < parts; c0 += 8u) {
                            float4 pv[8];
#pragma unroll
                            for (uint32_t u = 0; u < 8u; ++u) {
                                pv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                                if (c0 + u < parts) {
                                    pv[u] = __ldcg(reinterpret_cast<const float4*>(
                                                p.partial + static_cast<uint64_t>(slots[c0 + u]) * kPartialFloats) + i4);
                                }
                            }
#pragma unroll
                            for (uint32_t u = 0; u < 8u; ++u) {
                                if (c0 + u < parts) {
                                    acc.x += pv[u].x;
                                    acc.y += pv[u].y;
                                    acc.z += pv[u].z;
                                    acc.w += pv[u].w;
                                }
                            }
                        }
                        const uint32_t t = i4 / (kTileW / 4), rr = (i4 % (kTileW / 4)) * 4u;
                        float* dst = out + static_cast<uint64_t>(t) * cur_ref.n_out + cur_ref.n0 + rr;
                        if (cur_ref.n0 + rr + 3u < cur_ref.n_out && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
                            *reinterpret_cast<float4*>(dst) = acc;
                        } else {
                            const float a4[4] = {acc.x, acc.y, acc.z, acc.w};
                            for (uint32_t u = 0; u < 4u; ++u) {
                                if (cur_ref.n0 + rr + u < cur_ref.n_out) dst[u] = a4[u];
                            }
                        }
                    }
                    if ((e & 7u) == 0u && lane == 0) p.counters[cur_tile] = 0u;   // every part has arrived: ready for the next launch
                }
                set_barrier(set);   // last_flag and the slot list are rewritten by the set's next partial segment
            }
        }
    }
    if (clustered) {
        // Every CTA of the cluster holds its partial tile [token][row] in its own shared memory. The
        // leader adds them in rank order (a fixed order: results repeat bit for bit) and writes the
        // output tile; the second barrier keeps the peers' shared memory alive until it has read it.
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        if (cluster.block_rank() == 0u && warp >= static_cast<uint32_t>(kFirstExpandWarp)) {
            const uint32_t tile = cta / p.cluster_k;
            const TileRef ref = locate_tile(p, tile);
            float* out = p.out[0];
#pragma unroll
            for (int i = 1; i < kMaxWeights; ++i) {
                if (ref.wi == static_cast<uint32_t>(i)) out = p.out[i];
            }
            const float4* mine = reinterpret_cast<const float4*>(smem_raw + (w_stage_addr(plan, 0u) - raw32));
            const uint32_t st = tid - kFirstExpandWarp * 32u;
            const uint32_t total4 = p.m * (kTileW / 4);
            for (uint32_t i4 = st; i4 < total4; i4 += kExpandThreads) {
                float4 pv[8];
#pragma unroll
                for (uint32_t q = 0; q < 8u; ++q) {
                    pv[q] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (q < p.cluster_k) pv[q] = cluster.map_shared_rank(mine, q)[i4];
                }
                float4 acc = pv[0];
#pragma unroll
                for (uint32_t q = 1; q < 8u; ++q) {
                    if (q < p.cluster_k) {
                        acc.x += pv[q].x;
                        acc.y += pv[q].y;
                        acc.z += pv[q].z;
                        acc.w += pv[q].w;
                    }
                }
                const uint32_t t = i4 / (kTileW / 4), rr = (i4 % (kTileW / 4)) * 4u;
                float* dst = out + static_cast<uint64_t>(t) * ref.n_out + ref.n0 + rr;
                if (ref.n0 + rr + 3u < ref.n_out && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
                    *reinterpret_cast<float4*>(dst) = acc;
                } else {
                    const float a4[4] = {acc.x, acc.y, acc.z, acc.w};
                    for (uint32_t u = 0; u < 4u; ++u) {
                        if (ref.n0 + rr + u < ref.n_out) dst[u] = a4[u];
                    }
                }
            }
        }
        // The peers only have to outlive the leader's reads of their shared memory, which are
        // complete when it gets here (their values have been stored): no memory ordering is needed,
        // and a releasing arrive would wait for the output stores to be acknowledged.
        asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after_sync();
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

int32_t encode(const char* what, CUtensorMap* map, CUtensorMapDataType type, uint32_t rank, const void* base,
               const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box, CUtensorMapSwizzle swizzle) {
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode_tiled()(map, type, rank, const_cast<void*>(base), dims, strides, box, elem,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        return fail(B2_STATUS_RUNTIME_ERROR, "cuTensorMapEncodeTiled failed (%d) for the %s map", static_cast<int>(r), what);
    }
    return B2_STATUS_OK;
}

// fp32 -> fp16 row-major copy of the activations (pre-pass of the fp16 form).
__global__ void __launch_bounds__(256)
f32_to_f16_kernel(const float* __restrict__ src, __half* __restrict__ dst, uint64_t n4) {
    pdl_launch_dependents();   // the linear that follows may start streaming its weights now
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(src) + i);
        __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&lo);
        packed.y = *reinterpret_cast<uint32_t*>(&hi);
        reinterpret_cast<uint2*>(dst)[i] = packed;
    }
}


}  // namespace

int32_t launch_f32_to_f16(const DeviceContext& ctx, const float* src, void* dst, uint64_t count, cudaStream_t stream) {
    const uint64_t n4 = count / 4;
    uint64_t blocks = (n4 + 255) / 256;
    if (blocks > static_cast<uint64_t>(ctx.sm_count) * 16) blocks = static_cast<uint64_t>(ctx.sm_count) * 16;
    if (blocks == 0) blocks = 1;
    f32_to_f16_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(src, static_cast<__half*>(dst), n4);
    B2_CUDA_TRY(cudaGetLastError());
    return B2_STATUS_OK;
}

size_t nf4_decode_tmem_workspace_bytes(const DeviceContext& ctx) {
    return static_cast<size_t>(2) * static_cast<size_t>(ctx.sm_count) * kPartialFloats * sizeof(float);
}

// Shapes this kernel takes: up to 32 rows, at least two whole 256-wide rounds, scale blocks of at least 64
// weights that divide a row, and arrays aligned the way a TMA descriptor needs them.
bool nf4_decode_tmem_supported(const WeightView& w, const void* x, uint64_t rows) {
    if (rows < 1 || rows > static_cast<uint64_t>(kMaxTokens)) return false;
    if (w.in_features % kRoundK != 0 || w.in_features < 2 * kRoundK) return false;   // whole rounds, two or more per tile
    if (w.block_size < 64 || w.in_features % w.block_size != 0) return false;
    if (encode_tiled() == nullptr) return false;
    if ((reinterpret_cast<uintptr_t>(w.codes) & 15u) != 0 || (reinterpret_cast<uintptr_t>(x) & 15u) != 0) return false;
    const uint64_t bpr = w.in_features / w.block_size;
    if (w.encoding == B2_SCALES_FLOAT32) {
        if ((reinterpret_cast<uintptr_t>(w.fp32_scales) & 15u) != 0 || bpr % 4 != 0) return false;
    } else {
        if ((reinterpret_cast<uintptr_t>(w.scale_codes) & 15u) != 0 || bpr % 16 != 0) return false;
        if ((reinterpret_cast<uintptr_t>(w.second_level) & 15u) != 0) return false;
        // second-level values one item can refer to must fit the 128-float box
        if ((((kTileW - 1) * bpr + 4) >> w.scale_block_shift) + 5 > static_cast<uint64_t>(kSecondBox)) return false;
    }
    const uint64_t tiles = (w.out_features + kTileW - 1) / kTileW;
    if (tiles * (w.in_features / kRoundK) > 0x3FFFFFFFull) return false;
    if ((w.out_features + kTileW) * bpr + w.flat_block_base > 0xFFFFFFFFull) return false;
    return w.out_features <= 0x7FFFFFFFull && w.in_features <= 0x7FFFFFFFull;
}

namespace {

// Clusters of `k` CTAs of this kernel that can be resident on the device at once (cached per device).
int32_t resident_clusters(const DeviceContext& ctx, bool half, uint32_t k, uint32_t* out) {
    static int cached[kMaxDevices][2][9] = {};
    static std::mutex cache_mutex;
    std::lock_guard<std::mutex> lock(cache_mutex);
    int& slot = cached[ctx.device][half ? 1 : 0][k];
    if (slot == 0) {
        cudaLaunchConfig_t config = {};
        config.blockDim = dim3(kThreads);
        config.dynamicSmemBytes = kSmemBytes;
        config.gridDim = dim3(static_cast<unsigned>(ctx.sm_count / k) * k);
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = k;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        config.attrs = attr;
        config.numAttrs = 1;
        int n = 0;
        if (half) {
            B2_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, nf4_decode_tmem_kernel<true>, &config));
        } else {
            B2_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, nf4_decode_tmem_kernel<false>, &config));
        }
        slot = n > 0 ? n : -1;
    }
    *out = slot > 0 ? static_cast<uint32_t>(slot) : 0u;
    return B2_STATUS_OK;
}

}  // namespace

// `x16` holds the activations as bf16 (half == false) or fp16 (half == true), [rows, in] row-major.
// `partial` is scratch of nf4_decode_tmem_workspace_bytes(); `counters` are `tiles` zeroed words.
int32_t launch_nf4_decode_tmem(const DeviceContext& ctx, const WeightView* ws, float* const* ys, uint32_t count,
                               const void* x16, bool half, uint64_t rows, void* partial, uint32_t* counters,
                               cudaStream_t stream) {
    if (count == 0 || count > static_cast<uint32_t>(kMaxWeights)) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "between one and four weights per launch");
    }
    DecodeParams p;
    DecodeMaps maps;
    uint64_t tiles = 0;
    for (uint32_t i = 0; i < static_cast<uint32_t>(kMaxWeights); ++i) {
        const uint32_t src = i < count ? i : 0;
        const WeightView& w = ws[src];
        p.w[i] = w;
        p.out[i] = ys[src];
        p.n[i] = static_cast<uint32_t>(w.out_features);
        if (i < count) tiles += (w.out_features + kTileW - 1) / kTileW;
        p.tile_end[i] = static_cast<uint32_t>(tiles);
        if (w.encoding != ws[0].encoding || w.block_size != ws[0].block_size ||
            w.scale_block_shift != ws[0].scale_block_shift || w.in_features != ws[0].in_features) {
            return fail(B2_STATUS_INVALID_ARGUMENT, "weights of one launch must share encoding, block sizes and width");
        }
        const uint64_t bpr = w.in_features / w.block_size;
        {
            const cuuint64_t dims[2] = {w.in_features / 2, w.out_features};
            const cuuint64_t strides[1] = {w.in_features / 2};
            const cuuint32_t box[2] = {kRoundK / 2, kTileW};
            B2_TRY(encode("codes", &maps.codes[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w.codes, dims, strides, box,
                          CU_TENSOR_MAP_SWIZZLE_128B));
        }
        if (w.encoding == B2_SCALES_FLOAT32) {
            const cuuint64_t dims[2] = {bpr, w.out_features};
            const cuuint64_t strides[1] = {bpr * 4};
            const cuuint32_t box[2] = {4, kTileW};
            B2_TRY(encode("fp32 scales", &maps.scales[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, w.fp32_scales, dims,
                          strides, box, CU_TENSOR_MAP_SWIZZLE_NONE));
            maps.second[i] = maps.scales[i];   // unused for this encoding
        } else {
            const cuuint64_t dims[2] = {bpr, w.out_features};
            const cuuint64_t strides[1] = {bpr};
            const cuuint32_t box[2] = {16, kTileW};
            B2_TRY(encode("scale codes", &maps.scales[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w.scale_codes, dims,
                          strides, box, CU_TENSOR_MAP_SWIZZLE_NONE));
            const uint64_t last = (w.flat_block_base + w.out_features * bpr - 1) >> w.scale_block_shift;
            const cuuint64_t dims2[1] = {last + 1};
            const cuuint64_t strides2[1] = {0};
            const cuuint32_t box2[1] = {kSecondBox};
            B2_TRY(encode("second-level", &maps.second[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 1, w.second_level, dims2,
                          strides2, box2, CU_TENSOR_MAP_SWIZZLE_NONE));
        }
    }
    p.count = count;
    p.m = static_cast<uint32_t>(rows);
    p.k = static_cast<uint32_t>(ws[0].in_features);
    p.n_pad = rows <= 16 ? 16u : 32u;
    p.rounds = p.k / kRoundK;
    p.total_items = static_cast<uint32_t>(tiles) * p.rounds;
    p.blocks_per_row = static_cast<uint32_t>(ws[0].in_features / ws[0].block_size);
    p.kshift = ws[0].block_shift - 6u;
    p.partial = static_cast<float*>(partial);
    p.counters = counters;
    p.error = ctx.gemm_error;

    CUtensorMap map_x;
    {
        const cuuint64_t dims[2] = {ws[0].in_features, rows};
        const cuuint64_t strides[1] = {ws[0].in_features * 2};
        const cuuint32_t box[2] = {64, p.n_pad};
        B2_TRY(encode("activations", &map_x, half ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                      2, x16, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B));
    }
    static PerDeviceOnce configured;
    B2_TRY(once_per_device(configured, ctx.device, []() -> int32_t {
        B2_CUDA_TRY(cudaFuncSetAttribute(nf4_decode_tmem_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemBytes));
        B2_CUDA_TRY(cudaFuncSetAttribute(nf4_decode_tmem_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemBytes));
        return B2_STATUS_OK;
    }));
    cudaLaunchConfig_t config = {};
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = kSmemBytes;
    config.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    // Few tiles: one cluster per tile, as many CTAs per cluster as the SMs allow (at least two rounds
    // each), provided every cluster can be resident at once.
    const uint32_t sms = static_cast<uint32_t>(ctx.sm_count);
    uint32_t cluster_k = 1;
    if (tiles * 2 <= sms) {
        uint32_t k = sms / static_cast<uint32_t>(tiles);
        if (k > 8u) k = 8u;
        if (k > p.rounds / 2u) k = p.rounds / 2u;
        for (; k >= 2u; --k) {
            uint32_t resident = 0;
            B2_TRY(resident_clusters(ctx, half, k, &resident));
            if (resident >= tiles) {
                cluster_k = k;
                break;
            }
        }
    }
    p.cluster_k = cluster_k;
    if (cluster_k > 1u) {
        config.gridDim = dim3(static_cast<uint32_t>(tiles) * cluster_k);
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = cluster_k;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        config.numAttrs = 2;
    } else {
        config.gridDim = dim3(p.total_items < sms ? p.total_items : sms);
    }
    if (half) {
        B2_CUDA_TRY(cudaLaunchKernelEx(&config, nf4_decode_tmem_kernel<true>, maps, map_x, p));
    } else {
        B2_CUDA_TRY(cudaLaunchKernelEx(&config, nf4_decode_tmem_kernel<false>, maps, map_x, p));
    }
    return B2_STATUS_OK;
}

}  // namespace b2
