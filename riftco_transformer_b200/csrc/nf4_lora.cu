// The low-rank adapter branch of a packed-NF4 linear:
//   y[r, o] += scale * sum_j (sum_i x[r, i] * A[j, i]) * B[o, j]
// (LowRankAdapter::forward, src/nn/low_rank_adapter.cpp:132-158, added to the base projection as
// src/nn/linear.cpp:165-172 does). A is [rank, in], B is [out, rank], both FP32 like the reference's
// adapter parameters. Two FP32 kernels behind the base linear:
//   lora_reduce_kernel  t[r, j] = sum_i x[r, i] * A[j, i]   one CTA per activation row: the row is read
//                       once (HBM-bound on x for many rows) and meets A from L2
//   lora_expand_kernel  y[r, o] += scale * sum_j t[r, j] * B[o, j]   one pass over y with B's rows in
//                       registers (HBM-bound: 8 bytes per output)
// The arithmetic is FP32 throughout; the sum over i is a tree, not the reference's sequential loop,
// which is within the tolerance of the base kernels by orders of magnitude.
#include "b2_common.cuh"
#include "b2_kernels.h"

namespace b2 {
namespace {

constexpr int kReduceThreads = 256;
constexpr int kMaxRank = 64;

__global__ void __launch_bounds__(kReduceThreads)
lora_reduce_kernel(const float* __restrict__ x, const float* __restrict__ a, float* __restrict__ t,
                   uint32_t in_features, uint32_t rank) {
    __shared__ float partial[kReduceThreads / 32][kMaxRank];
    const uint32_t row = blockIdx.x;
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const float* xr = x + static_cast<uint64_t>(row) * in_features;
    // each thread keeps `rank` running sums over its strided slice of the row
    for (uint32_t j0 = 0; j0 < rank; j0 += 8) {
        float sum[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) sum[u] = 0.0f;
        for (uint32_t i = threadIdx.x; i < in_features; i += kReduceThreads) {
            const float xv = xr[i];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (j0 + u < rank) sum[u] = fmaf(xv, __ldg(a + static_cast<uint64_t>(j0 + u) * in_features + i), sum[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) sum[u] += __shfl_xor_sync(0xFFFFFFFFu, sum[u], off);
            if (lane == 0 && j0 + u < rank) partial[warp][j0 + u] = sum[u];
        }
    }
    __syncthreads();
    if (threadIdx.x < rank) {
        float total = 0.0f;
#pragma unroll
        for (int w = 0; w < kReduceThreads / 32; ++w) total += partial[w][threadIdx.x];
        t[static_cast<uint64_t>(row) * rank + threadIdx.x] = total;
    }
}

// Thread = one output feature o for a slab of rows: B[o, :] stays in registers.
template <int RANK_PAD>
__global__ void __launch_bounds__(256)
lora_expand_kernel(const float* __restrict__ t, const float* __restrict__ b, float* __restrict__ y, uint32_t rows,
                   uint32_t out_features, uint32_t rank, float scale, uint32_t rows_per_cta) {
    extern __shared__ float s_t[];   // [rows_per_cta][rank]
    const uint32_t o = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t r0 = blockIdx.y * rows_per_cta;
    const uint32_t r1 = r0 + rows_per_cta < rows ? r0 + rows_per_cta : rows;
    for (uint32_t i = threadIdx.x; i < (r1 - r0) * rank; i += blockDim.x) s_t[i] = t[static_cast<uint64_t>(r0) * rank + i];
    __syncthreads();
    if (o >= out_features) return;
    float bo[RANK_PAD];
#pragma unroll
    for (int j = 0; j < RANK_PAD; ++j) bo[j] = static_cast<uint32_t>(j) < rank ? b[static_cast<uint64_t>(o) * rank + j] : 0.0f;
    for (uint32_t r = r0; r < r1; ++r) {
        const float* tr = s_t + (r - r0) * rank;
        float total = 0.0f;
#pragma unroll
        for (int j = 0; j < RANK_PAD; ++j) {
            if (static_cast<uint32_t>(j) < rank) total = fmaf(tr[j], bo[j], total);
        }
        float* dst = y + static_cast<uint64_t>(r) * out_features + o;
        *dst = __fadd_rn(*dst, __fmul_rn(total, scale));
    }
}

}  // namespace

bool lora_rank_supported(uint64_t rank) { return rank >= 1 && rank <= static_cast<uint64_t>(kMaxRank); }

size_t lora_workspace_bytes(uint64_t rows, uint64_t rank) { return static_cast<size_t>(rows) * rank * sizeof(float); }

// `reduced` is scratch of lora_workspace_bytes(rows, rank); y already holds the base projection.
int32_t launch_lora_branch(const DeviceContext& ctx, const float* x, const float* a, const float* b, float* y,
                           uint64_t rows, uint64_t in_features, uint64_t out_features, uint32_t rank, float scale,
                           float* reduced, cudaStream_t stream) {
    (void)ctx;
    lora_reduce_kernel<<<static_cast<unsigned>(rows), kReduceThreads, 0, stream>>>(
        x, a, reduced, static_cast<uint32_t>(in_features), rank);
    B2_CUDA_TRY(cudaGetLastError());
    const uint32_t rows_per_cta = 64;
    const dim3 grid(static_cast<unsigned>((out_features + 255) / 256), static_cast<unsigned>((rows + rows_per_cta - 1) / rows_per_cta));
    const size_t smem = static_cast<size_t>(rows_per_cta) * rank * sizeof(float);
    if (rank <= 8) {
        lora_expand_kernel<8><<<grid, 256, smem, stream>>>(reduced, b, y, static_cast<uint32_t>(rows),
                                                            static_cast<uint32_t>(out_features), rank, scale, rows_per_cta);
    } else if (rank <= 16) {
        lora_expand_kernel<16><<<grid, 256, smem, stream>>>(reduced, b, y, static_cast<uint32_t>(rows),
                                                             static_cast<uint32_t>(out_features), rank, scale, rows_per_cta);
    } else if (rank <= 32) {
        lora_expand_kernel<32><<<grid, 256, smem, stream>>>(reduced, b, y, static_cast<uint32_t>(rows),
                                                             static_cast<uint32_t>(out_features), rank, scale, rows_per_cta);
    } else {
        lora_expand_kernel<64><<<grid, 256, smem, stream>>>(reduced, b, y, static_cast<uint32_t>(rows),
                                                             static_cast<uint32_t>(out_features), rank, scale, rows_per_cta);
    }
    B2_CUDA_TRY(cudaGetLastError());
    return B2_STATUS_OK;
}

}  // namespace b2
