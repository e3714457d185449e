// Shape-agnostic packed-NF4 linear kernels (FP32 CUDA-core math). They accept
// every legal payload: odd element counts, rows that start in the middle of a
// byte or of a block, block sizes down to 32, both scale encodings. The tuned
// decode and prefill kernels take over when their layout requirements hold;
// these cover the rest (for example the reference's 33x33 edge fixture,
// tests/core/backend/test_quantized_linear_backend.cpp:126-169).
#include "b2_common.cuh"
#include "b2_kernels.h"

namespace b2 {
namespace {

constexpr int kRowChunk = 8;

__device__ __forceinline__ float dequant_at(const WeightView& w, uint64_t flat) {
    return kNf4Codebook[nf4_code_at(w.codes, flat)] * decode_block_scale(w, flat >> w.block_shift);
}

// y[r,o] = sum_i x[r,i] * W[o,i]. One warp per (output column, chunk of 8
// rows): lanes stride over the input dimension, each weight is decoded once
// and used for all rows of the chunk, partial sums meet in a shuffle tree.
__global__ void __launch_bounds__(256)
nf4_forward_generic_kernel(WeightView w, const float* __restrict__ x, float* __restrict__ y,
                           uint64_t rows) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t warps_per_grid = (static_cast<uint64_t>(gridDim.x) * blockDim.x) >> 5;
    const uint64_t row_chunks = (rows + kRowChunk - 1) / kRowChunk;
    const uint64_t tasks = w.out_features * row_chunks;
    for (uint64_t task = (static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
         task < tasks; task += warps_per_grid) {
        const uint64_t o = task / row_chunks;
        const uint64_t r0 = (task % row_chunks) * kRowChunk;
        const int nr = static_cast<int>(rows - r0 < kRowChunk ? rows - r0 : kRowChunk);
        float acc[kRowChunk];
#pragma unroll
        for (int r = 0; r < kRowChunk; ++r) acc[r] = 0.0f;
        const uint64_t base = o * w.in_features;
        for (uint64_t i = lane; i < w.in_features; i += 32) {
            const float wv = dequant_at(w, base + i);
#pragma unroll
            for (int r = 0; r < kRowChunk; ++r) {
                if (r < nr) acc[r] = fmaf(__ldg(x + (r0 + r) * w.in_features + i), wv, acc[r]);
            }
        }
#pragma unroll
        for (int r = 0; r < kRowChunk; ++r) {
            float v = acc[r];
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, s);
            if (lane == 0 && r < nr) y[(r0 + r) * w.out_features + o] = v;
        }
    }
}

// dx[r,i] = sum_o dy[r,o] * W[o,i]. One thread per input column (adjacent
// threads read adjacent nibbles of every weight row) for a chunk of 8 rows.
__global__ void __launch_bounds__(128)
nf4_input_backward_generic_kernel(WeightView w, const float* __restrict__ dy,
                                  float* __restrict__ dx, uint64_t rows) {
    const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const uint64_t r0 = static_cast<uint64_t>(blockIdx.y) * kRowChunk;
    if (i >= w.in_features) return;
    const int nr = static_cast<int>(rows - r0 < kRowChunk ? rows - r0 : kRowChunk);
    float acc[kRowChunk];
#pragma unroll
    for (int r = 0; r < kRowChunk; ++r) acc[r] = 0.0f;
    for (uint64_t o = 0; o < w.out_features; ++o) {
        const float wv = dequant_at(w, o * w.in_features + i);
#pragma unroll
        for (int r = 0; r < kRowChunk; ++r) {
            if (r < nr) acc[r] = fmaf(__ldg(dy + (r0 + r) * w.out_features + o), wv, acc[r]);
        }
    }
#pragma unroll
    for (int r = 0; r < kRowChunk; ++r) {
        if (r < nr) dx[(r0 + r) * w.in_features + i] = acc[r];
    }
}

}  // namespace

int32_t launch_nf4_linear_forward_generic(const DeviceContext& ctx, const WeightView& w,
                                          const float* x, float* y, uint64_t rows,
                                          cudaStream_t stream) {
    const uint64_t row_chunks = (rows + kRowChunk - 1) / kRowChunk;
    const uint64_t tasks = w.out_features * row_chunks;
    uint64_t blocks = (tasks + 7) / 8;  // 8 warps per block
    const uint64_t cap = static_cast<uint64_t>(ctx.sm_count) * 8;
    if (blocks > cap) blocks = cap;
    nf4_forward_generic_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(w, x, y, rows);
    B2_CUDA_TRY(cudaGetLastError());
    return B2_STATUS_OK;
}

int32_t launch_nf4_linear_input_backward_generic(const DeviceContext&, const WeightView& w,
                                                 const float* dy, float* dx, uint64_t rows,
                                                 cudaStream_t stream) {
    const uint64_t row_chunks = (rows + kRowChunk - 1) / kRowChunk;
    if (row_chunks > 65535) {
        return fail(B2_STATUS_OVERFLOW, "generic NF4 input-backward supports at most %d rows",
                    65535 * kRowChunk);
    }
    const dim3 grid(static_cast<unsigned>((w.in_features + 127) / 128),
                    static_cast<unsigned>(row_chunks));
    nf4_input_backward_generic_kernel<<<grid, 128, 0, stream>>>(w, dy, dx, rows);
    B2_CUDA_TRY(cudaGetLastError());
    return B2_STATUS_OK;
}

}  // namespace b2
