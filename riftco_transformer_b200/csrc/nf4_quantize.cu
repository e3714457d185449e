// NF4 encoder and payload validation on the device (cold path: run once per weight).
//
// b2_nf4_quantize restates the reference encoder
//   pack_nf4                 src/core/quantization/quantized_weight.cpp:176-207
//   nearest_nf4_code         src/core/quantization/nf4.cpp:55-68 (strict <: ties go to the lower code)
//   double_quantize_scales   quantized_weight.cpp:209-254
// with the same FP32 operations in the same order per element, so its output is the reference's
// payload bit for bit: absmax per block, code = nearest level of value / absmax, a zero block keeps
// scale 0 and code 7; for the double-quantised form the block scales are centred on their mean
// (a DOUBLE sum, rounded once), each group of `scale_block_size` scales gets its absmax as FP32
// second-level scale and the scales become 128 + clamp(round_half_away(127 * (s - mean) / absmax)).
// The mean is summed per CTA and then over CTAs in index order; a double holds the sum of a few
// million FP32 values of similar magnitude exactly, so the order does not change the result.
//
// b2_nf4_validate_payload applies require_canonical_payload (quantized_weight.cpp:102-174) to a
// payload that already lies in device memory.
#include "b2_common.cuh"
#include "b2_kernels.h"

#include <cmath>
#include <vector>

namespace b2 {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ uint32_t nearest_code(float normalized) {
    uint32_t best = 0;
    float best_distance = fabsf(__fsub_rn(normalized, kNf4Codebook[0]));
#pragma unroll
    for (uint32_t c = 1; c < 16; ++c) {
        const float d = fabsf(__fsub_rn(normalized, kNf4Codebook[c]));
        if (d < best_distance) {
            best_distance = d;
            best = c;
        }
    }
    return best;
}

// One warp per block of `block_size` values: absmax by shuffle, then every lane encodes its
// values and the lanes' nibbles are packed pairwise. flags bit 0: a non-finite source value.
__global__ void __launch_bounds__(kThreads)
nf4_pack_kernel(const float* __restrict__ values, uint64_t n, uint32_t block_size, uint8_t* __restrict__ codes,
                float* __restrict__ scales, uint32_t* flags) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t warps = (static_cast<uint64_t>(gridDim.x) * blockDim.x) >> 5;
    const uint64_t blocks = (n + block_size - 1) / block_size;
    for (uint64_t b = (static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; b < blocks; b += warps) {
        const uint64_t begin = b * block_size;
        const uint64_t end = begin + block_size < n ? begin + block_size : n;
        float absmax = 0.0f;
        bool bad = false;
        for (uint64_t i = begin + lane; i < end; i += 32) {
            const float v = values[i];
            bad |= !isfinite(v);
            absmax = fmaxf(absmax, fabsf(v));
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) absmax = fmaxf(absmax, __shfl_xor_sync(0xFFFFFFFFu, absmax, off));
        if (__any_sync(0xFFFFFFFFu, bad)) {
            if (lane == 0) atomicOr(flags, 1u);
            continue;
        }
        if (lane == 0) scales[b] = absmax;
        // pairs of elements (2p, 2p+1) -> one byte; begin is even because block sizes are even
        for (uint64_t p = (begin >> 1) + lane; 2 * p < end; p += 32) {
            const uint64_t i0 = 2 * p, i1 = i0 + 1;
            const uint32_t c0 = absmax == 0.0f ? 7u : nearest_code(__fdiv_rn(values[i0], absmax));
            uint32_t c1 = 0;
            if (i1 < end) c1 = absmax == 0.0f ? 7u : nearest_code(__fdiv_rn(values[i1], absmax));
            codes[p] = static_cast<uint8_t>(c0 | (c1 << 4));
        }
    }
}

// Per-CTA double sums of the block scales (fixed order inside a CTA: thread-strided, then a tree).
__global__ void __launch_bounds__(kThreads)
scale_sum_kernel(const float* __restrict__ scales, uint64_t count, double* __restrict__ partial) {
    __shared__ double tree[kThreads];
    double sum = 0.0;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
        sum += static_cast<double>(scales[i]);
    }
    tree[threadIdx.x] = sum;
    __syncthreads();
    for (int off = kThreads / 2; off > 0; off >>= 1) {
        if (threadIdx.x < off) tree[threadIdx.x] += tree[threadIdx.x + off];
        __syncthreads();
    }
    if (threadIdx.x == 0) partial[blockIdx.x] = tree[0];
}

// One warp per group of `scale_block_size` block scales. `offset` is read from device memory.
__global__ void __launch_bounds__(kThreads)
double_quantize_kernel(const float* __restrict__ scales, uint64_t count, uint64_t scale_block_size,
                       const float* __restrict__ offset_ptr, uint8_t* __restrict__ scale_codes,
                       float* __restrict__ second) {
    const float offset = *offset_ptr;
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t warps = (static_cast<uint64_t>(gridDim.x) * blockDim.x) >> 5;
    const uint64_t groups = (count + scale_block_size - 1) / scale_block_size;
    for (uint64_t g = (static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; g < groups; g += warps) {
        const uint64_t begin = g * scale_block_size;
        const uint64_t end = begin + scale_block_size < count ? begin + scale_block_size : count;
        float absmax = 0.0f;
        for (uint64_t i = begin + lane; i < end; i += 32) absmax = fmaxf(absmax, fabsf(__fsub_rn(scales[i], offset)));
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) absmax = fmaxf(absmax, __shfl_xor_sync(0xFFFFFFFFu, absmax, off));
        if (lane == 0) second[g] = absmax;
        for (uint64_t i = begin + lane; i < end; i += 32) {
            uint32_t code = 128;
            if (absmax != 0.0f) {
                const float normalized = __fdiv_rn(__fsub_rn(scales[i], offset), absmax);
                const float scaled = __fmul_rn(normalized, 127.0f);
                const float rounded = scaled >= 0.0f ? floorf(__fadd_rn(scaled, 0.5f)) : ceilf(__fsub_rn(scaled, 0.5f));
                int centered = static_cast<int>(rounded);
                centered = centered < -127 ? -127 : (centered > 127 ? 127 : centered);
                code = static_cast<uint32_t>(centered + 128);
            }
            scale_codes[i] = static_cast<uint8_t>(code);
        }
    }
}

// require_canonical_payload: flags 1 unused high nibble, 2 second-level scale, 4 block scale,
// 8 zero-scale block with a code other than 7.
__global__ void __launch_bounds__(kThreads)
validate_kernel(WeightView w, uint64_t n, uint64_t blocks, uint64_t second_count, uint32_t* flags) {
    const uint64_t tid = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    if (tid == 0 && (n & 1u) != 0 && (w.codes[n >> 1] & 0xF0u) != 0) atomicOr(flags, 1u);
    if (w.encoding != B2_SCALES_FLOAT32) {
        for (uint64_t i = tid; i < second_count; i += stride) {
            const float s = w.second_level[i];
            if (!isfinite(s) || s < 0.0f) atomicOr(flags, 2u);
        }
    }
    for (uint64_t b = tid; b < blocks; b += stride) {
        const float scale = decode_block_scale(w, b);
        if (!isfinite(scale) || scale < 0.0f) {
            atomicOr(flags, 4u);
            continue;
        }
        if (scale != 0.0f || w.encoding != B2_SCALES_FLOAT32) continue;
        const uint64_t begin = b << w.block_shift;
        const uint64_t end = begin + w.block_size < n ? begin + w.block_size : n;
        for (uint64_t i = begin; i < end; ++i) {
            if (nf4_code_at(w.codes, i) != 7u) {
                atomicOr(flags, 8u);
                break;
            }
        }
    }
}

unsigned grid_for(const DeviceContext& ctx, uint64_t threads_needed) {
    uint64_t blocks = (threads_needed + kThreads - 1) / kThreads;
    const uint64_t cap = static_cast<uint64_t>(ctx.sm_count) * 8;
    if (blocks > cap) blocks = cap;
    return blocks == 0 ? 1u : static_cast<unsigned>(blocks);
}

}  // namespace

size_t nf4_quantize_workspace_bytes(const DeviceContext& ctx, uint64_t blocks, bool double_quantized) {
    // flags word + offset + per-CTA double sums, then (double-quantised only) the FP32 block scales
    size_t bytes = 256 + static_cast<size_t>(ctx.sm_count) * 8 * sizeof(double);
    if (double_quantized) bytes += blocks * sizeof(float);
    return bytes;
}

// Synchronous (the offset is returned to the host). `workspace` holds nf4_quantize_workspace_bytes.
int32_t run_nf4_quantize(const DeviceContext& ctx, const float* values, uint64_t out_features, uint64_t in_features,
                         uint32_t block_size, uint64_t scale_block_size, uint8_t* codes, void* primary,
                         float* secondary, float* offset_out, void* workspace, cudaStream_t stream) {
    const uint64_t n = out_features * in_features;
    const uint64_t blocks = (n + block_size - 1) / block_size;
    const bool dq = scale_block_size != 0;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    uint32_t* flags = reinterpret_cast<uint32_t*>(ws);
    float* d_offset = reinterpret_cast<float*>(ws + 64);
    double* partial = reinterpret_cast<double*>(ws + 256);
    float* scales = dq ? reinterpret_cast<float*>(ws + 256 + static_cast<size_t>(ctx.sm_count) * 8 * sizeof(double))
                       : static_cast<float*>(primary);
    B2_CUDA_TRY(cudaMemsetAsync(flags, 0, sizeof(uint32_t), stream));
    nf4_pack_kernel<<<grid_for(ctx, blocks * 32), kThreads, 0, stream>>>(values, n, block_size, codes, scales, flags);
    B2_CUDA_TRY(cudaGetLastError());
    uint32_t host_flags = 0;
    B2_CUDA_TRY(cudaMemcpyAsync(&host_flags, flags, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream));
    if (!dq) {
        B2_CUDA_TRY(cudaStreamSynchronize(stream));
        if (host_flags & 1u) return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 source values must be finite");
        if (offset_out != nullptr) *offset_out = 0.0f;
        return B2_STATUS_OK;
    }
    const unsigned sum_ctas = grid_for(ctx, blocks);
    scale_sum_kernel<<<sum_ctas, kThreads, 0, stream>>>(scales, blocks, partial);
    B2_CUDA_TRY(cudaGetLastError());
    std::vector<double> host_partial(sum_ctas);
    B2_CUDA_TRY(cudaMemcpyAsync(host_partial.data(), partial, sum_ctas * sizeof(double), cudaMemcpyDeviceToHost, stream));
    B2_CUDA_TRY(cudaStreamSynchronize(stream));
    if (host_flags & 1u) return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 source values must be finite");
    double sum = 0.0;
    for (double v : host_partial) sum += v;
    const float offset = static_cast<float>(sum / static_cast<double>(blocks));
    if (!std::isfinite(offset)) {
        return fail(B2_STATUS_OVERFLOW, "NF4 scale mean exceeds the FP32 double-quantization range");
    }
    B2_CUDA_TRY(cudaMemcpyAsync(d_offset, &offset, sizeof(float), cudaMemcpyHostToDevice, stream));
    const uint64_t groups = (blocks + scale_block_size - 1) / scale_block_size;
    double_quantize_kernel<<<grid_for(ctx, groups * 32), kThreads, 0, stream>>>(
        scales, blocks, scale_block_size, d_offset, static_cast<uint8_t*>(primary), secondary);
    B2_CUDA_TRY(cudaGetLastError());
    B2_CUDA_TRY(cudaStreamSynchronize(stream));
    if (offset_out != nullptr) *offset_out = offset;
    return B2_STATUS_OK;
}

// Synchronous. `flags_word` is a device word of scratch.
int32_t run_nf4_validate(const DeviceContext& ctx, const WeightView& w, uint64_t second_count, uint32_t* flags_word,
                         cudaStream_t stream) {
    const uint64_t n = w.out_features * w.in_features;
    const uint64_t blocks = (n + w.block_size - 1) / w.block_size;
    B2_CUDA_TRY(cudaMemsetAsync(flags_word, 0, sizeof(uint32_t), stream));
    validate_kernel<<<grid_for(ctx, blocks), kThreads, 0, stream>>>(w, n, blocks, second_count, flags_word);
    B2_CUDA_TRY(cudaGetLastError());
    uint32_t flags = 0;
    B2_CUDA_TRY(cudaMemcpyAsync(&flags, flags_word, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream));
    B2_CUDA_TRY(cudaStreamSynchronize(stream));
    if (flags & 1u) return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 unused high nibble must be zero");
    if (flags & 2u) return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 second-level scales must be finite and nonnegative");
    if (flags & 4u) return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 block scales must be finite and nonnegative");
    if (flags & 8u) return fail(B2_STATUS_INVALID_ARGUMENT, "zero-scale NF4 blocks must use canonical zero code 7");
    return B2_STATUS_OK;
}

}  // namespace b2
