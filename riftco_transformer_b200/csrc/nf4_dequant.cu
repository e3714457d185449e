// Bit-exact NF4 dequantisation: out[i] = codebook[code(i)] * scale(i / B).
// One FP32 multiply per element, scale decoded with separately rounded
// divide / multiply / add, so the result equals the reference's
// QuantizedWeight::dequantize (src/core/quantization/quantized_weight.cpp) and
// decode_nf4_block_scale (src/core/backend/nn/quantized_linear/storage.hpp:48-65)
// bit for bit.
//
// HBM-bound on the FP32 write: 0.5 B read + 4 B written per element.
#include "b2_common.cuh"
#include "b2_kernels.h"

namespace b2 {
namespace {

constexpr int kThreads = 256;

// Each thread expands one aligned group of 8 codes (one 32-bit word). A group
// never straddles a block because block sizes are multiples of 32.
__global__ void __launch_bounds__(kThreads)
nf4_dequant_kernel(WeightView w, float* __restrict__ out, uint64_t n, bool vector_ok) {
    const uint64_t groups = n >> 3;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t g = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; g < groups;
         g += stride) {
        const uint64_t flat = g << 3;
        const float scale = decode_block_scale(w, flat >> w.block_shift);
        uint32_t word;
        if (vector_ok) {
            word = __ldg(reinterpret_cast<const uint32_t*>(w.codes) + g);
        } else {
            const uint8_t* b = w.codes + (g << 2);
            word = __ldg(b) | (__ldg(b + 1) << 8) | (__ldg(b + 2) << 16) | (__ldg(b + 3) << 24);
        }
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = __fmul_rn(kNf4Codebook[(word >> (4 * e)) & 0xFu], scale);
        if (vector_ok) {
            float4* dst = reinterpret_cast<float4*>(out + flat);
            dst[0] = make_float4(v[0], v[1], v[2], v[3]);
            dst[1] = make_float4(v[4], v[5], v[6], v[7]);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) out[flat + e] = v[e];
        }
    }
    // Ragged tail (n % 8 elements) handled by the first threads of block 0.
    const uint64_t tail_begin = groups << 3;
    if (blockIdx.x == 0 && tail_begin + threadIdx.x < n) {
        const uint64_t flat = tail_begin + threadIdx.x;
        out[flat] = __fmul_rn(kNf4Codebook[nf4_code_at(w.codes, flat)],
                              decode_block_scale(w, flat >> w.block_shift));
    }
}

}  // namespace

int32_t launch_nf4_dequantize(const DeviceContext& ctx, const WeightView& w, float* out,
                              cudaStream_t stream) {
    const uint64_t n = w.out_features * w.in_features;
    const bool vector_ok = (reinterpret_cast<uintptr_t>(w.codes) & 3u) == 0 &&
                           (reinterpret_cast<uintptr_t>(out) & 15u) == 0;
    const uint64_t groups = n >> 3;
    uint64_t blocks = (groups + kThreads - 1) / kThreads;
    const uint64_t cap = static_cast<uint64_t>(ctx.sm_count) * 16;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) blocks = 1;
    nf4_dequant_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, stream>>>(w, out, n, vector_ok);
    B2_CUDA_TRY(cudaGetLastError());
    return B2_STATUS_OK;
}

}  // namespace b2
