// Small memory-bound kernels that sit between the packed-NF4 linears and the
// paged attention in a decode step of a Llama-shaped decoder: RMSNorm (with an
// optional fused residual add), split-half RoPE fused with the KV-page append,
// SiLU(gate)*up, embedding gather and greedy argmax. Each restates a reference
// primitive (cited at the kernel); none of them is on the roofline-critical
// path, they exist so a whole decode step stays on the device and in one graph.
#include "b2_common.cuh"
#include "b2_kernels.h"
#include "sm100_ptx.cuh"

#include <cuda_bf16.h>

#include <cmath>

namespace b2 {
namespace {

// Four values rounded to bf16 (nearest even) as one 8-byte store: the activation
// layout the tensor-core linears read, so their conversion pre-pass can be skipped.
__device__ __forceinline__ void store_bf16x4(__nv_bfloat16* dst, const float4& v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = packed;
}

__device__ __forceinline__ float block_sum(float v, float* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const uint32_t warps = blockDim.x >> 5;
    float total = 0.0f;
    for (uint32_t w = 0; w < warps; ++w) total += scratch[w];
    __syncthreads();
    return total;
}

// y = x * (1 / sqrt(mean(x^2) + eps)) * scale, one CTA per row
// (src/nn/rms_norm.cpp:39-73). With `delta`, first x_out = x + delta (the
// residual stream update) and the norm is taken of x_out. A decode batch has few
// rows, so a row gets up to 1024 threads, 16-byte accesses, and its values stay
// in registers between the two passes when they fit (two float4 per thread).
__global__ void __launch_bounds__(1024)
rmsnorm_kernel(const float* x, const float* __restrict__ delta, float* x_out,   // x_out may be x
               const float* __restrict__ scale, float* __restrict__ y, __nv_bfloat16* __restrict__ y16,
               uint32_t width, float eps, uint32_t vec4) {
    sm100::pdl_launch_dependents();   // a following linear kernel may start its set-up now
    __shared__ float scratch[32];
    const uint64_t row = blockIdx.x;
    const float* xr = x + row * width;
    float ss = 0.0f;
    if (vec4 != 0u) {
        const uint32_t n4 = width / 4;
        const float4* x4 = reinterpret_cast<const float4*>(xr);
        const float4* d4 = delta != nullptr ? reinterpret_cast<const float4*>(delta + row * width) : nullptr;
        float4* o4 = delta != nullptr ? reinterpret_cast<float4*>(x_out + row * width) : nullptr;
        auto fetch = [&](uint32_t c) {
            float4 v = x4[c];
            if (d4 != nullptr) {
                const float4 dv = d4[c];
                v = make_float4(v.x + dv.x, v.y + dv.y, v.z + dv.z, v.w + dv.w);
                o4[c] = v;
            }
            ss = fmaf(v.x, v.x, ss);
            ss = fmaf(v.y, v.y, ss);
            ss = fmaf(v.z, v.z, ss);
            ss = fmaf(v.w, v.w, ss);
            return v;
        };
        const uint32_t c0 = threadIdx.x, c1 = threadIdx.x + blockDim.x;
        float4 keep0 = make_float4(0.f, 0.f, 0.f, 0.f), keep1 = keep0;
        if (c0 < n4) keep0 = fetch(c0);
        if (c1 < n4) keep1 = fetch(c1);
        for (uint32_t c = c1 + blockDim.x; c < n4; c += blockDim.x) (void)fetch(c);
        const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / static_cast<float>(width) + eps);
        const float4* s4 = reinterpret_cast<const float4*>(scale);
        const float4* src4 = d4 != nullptr ? reinterpret_cast<const float4*>(x_out + row * width) : x4;
        float4* y4 = reinterpret_cast<float4*>(y + row * width);
        auto emit = [&](uint32_t c, const float4& v) {
            const float4 g = s4[c];
            const float4 o = make_float4(v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w);
            y4[c] = o;
            if (y16 != nullptr) store_bf16x4(y16 + row * width + 4ull * c, o);
        };
        if (c0 < n4) emit(c0, keep0);
        if (c1 < n4) emit(c1, keep1);
        for (uint32_t c = c1 + blockDim.x; c < n4; c += blockDim.x) emit(c, src4[c]);
        return;
    }
    for (uint32_t c = threadIdx.x; c < width; c += blockDim.x) {
        float v = xr[c];
        if (delta != nullptr) {
            v += delta[row * width + c];
            x_out[row * width + c] = v;
        }
        ss = fmaf(v, v, ss);
    }
    const float mean_square = block_sum(ss, scratch) / static_cast<float>(width);
    const float inv = 1.0f / sqrtf(mean_square + eps);
    const float* src = delta != nullptr ? x_out + row * width : xr;
    for (uint32_t c = threadIdx.x; c < width; c += blockDim.x) {
        const float o = src[c] * inv * scale[c];
        y[row * width + c] = o;
        if (y16 != nullptr) y16[row * width + c] = __float2bfloat16_rn(o);
    }
}

// Split-half rotary embedding of the new token's q and k (pairs (c, c + d/2),
// angle = position * theta^(-2c/d) evaluated in double,
// src/model/rotary_embedding.cpp:64-117), then k and v are written into their
// page slot (copy_token_to_page, src/stages/serving/cache/page_table_cache.cpp:44-77).
// Grid (sequence, slice): every CTA takes an equal slice of the sequence's (head, channel pair)
// items and of its v row, so a decode batch of a few dozen sequences still covers the SMs.
__global__ void __launch_bounds__(256)
rope_append_kernel(float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                   const uint32_t* __restrict__ positions, const uint32_t* __restrict__ token_seq,
                   const uint32_t* __restrict__ block_tables,
                   float* __restrict__ k_pages, float* __restrict__ v_pages, uint32_t q_heads,
                   uint32_t kv_heads, uint32_t d, uint32_t block_size, uint64_t physical_blocks,
                   uint32_t max_blocks, float theta, uint32_t* status) {
    sm100::pdl_launch_dependents();   // a following decode GEMV may start its set-up now
    // blockIdx.x is the token: row of q / k / v and entry of `positions`. With token_seq == nullptr
    // every sequence contributes one token (a decode step) and the token index is the sequence;
    // otherwise token_seq names the sequence - the block-table row - of each token (a prefill chunk).
    const uint32_t seq = blockIdx.x;
    const uint32_t table_row = token_seq != nullptr ? token_seq[seq] : seq;
    const uint32_t pos = positions[seq];
    const uint32_t half = d / 2;
    // A position past the sequence's table row is treated like a bad block id: nothing is read from
    // the neighbouring row and no page is written.
    const uint32_t logical = pos / block_size;
    bool bad = logical >= max_blocks;
    uint64_t phys = bad ? 0 : block_tables[static_cast<uint64_t>(table_row) * max_blocks + logical];
    if (phys >= physical_blocks) {
        bad = true;
        phys = 0;
    }
    if (bad && threadIdx.x == 0 && blockIdx.y == 0 && status != nullptr) atomicOr(status, B2_ATTN_STATUS_BAD_BLOCK);
    const uint32_t slot = pos % block_size;
    const uint32_t pairs = (q_heads + kv_heads) * half;
    const uint32_t stride = blockDim.x * gridDim.y;
    const uint32_t first = blockIdx.y * blockDim.x + threadIdx.x;
    // The v row does not depend on the angles: its loads go out first.
    if (!bad) {
        for (uint32_t i = first; i < kv_heads * d; i += stride) {
            const uint32_t kh = i / d, c = i % d;
            v_pages[((phys * kv_heads + kh) * block_size + slot) * d + c] =
                v[(static_cast<uint64_t>(seq) * kv_heads + kh) * d + c];
        }
    }
    // angle = position * theta^(-2c/d) with theta^(-2c/d) as exp2(-2c/d * log2(theta)): double
    // precision like the reference's pow, within a few ulp of it (an angle error of ~1e-13 rad at
    // position 2048, far below the FP32 result). When the stride is a multiple of d/2 a thread keeps
    // the same channel pair for all its items and evaluates its angle once.
    const double log2_theta = log2(static_cast<double>(theta));
    const bool fixed_channel = stride % half == 0;
    float cs = 0.0f, sn = 0.0f;
    auto angle_of = [&](uint32_t c) {
        const double angle = static_cast<double>(pos) *
                             exp2(-2.0 * static_cast<double>(c) / static_cast<double>(d) * log2_theta);
        double s_, c_;
        sincos(angle, &s_, &c_);
        cs = static_cast<float>(c_);
        sn = static_cast<float>(s_);
    };
    if (fixed_channel && first < pairs) angle_of(first % half);
    for (uint32_t i = first; i < pairs; i += stride) {
        const uint32_t head = i / half, c = i % half;
        if (!fixed_channel) angle_of(c);
        if (head < q_heads) {
            float* p = q + (static_cast<uint64_t>(seq) * q_heads + head) * d;
            const float a = p[c], b = p[c + half];
            p[c] = __fsub_rn(__fmul_rn(a, cs), __fmul_rn(b, sn));
            p[c + half] = __fadd_rn(__fmul_rn(b, cs), __fmul_rn(a, sn));
        } else if (!bad) {
            const uint32_t kh = head - q_heads;
            const float* p = k + (static_cast<uint64_t>(seq) * kv_heads + kh) * d;
            const float a = p[c], b = p[c + half];
            float* dst = k_pages + ((phys * kv_heads + kh) * block_size + slot) * d;
            dst[c] = __fsub_rn(__fmul_rn(a, cs), __fmul_rn(b, sn));
            dst[c + half] = __fadd_rn(__fmul_rn(b, cs), __fmul_rn(a, sn));
        }
    }
}

// value * sigmoid(value) with the numerically stable sigmoid of
// src/nn/activations.cpp:38-58, times `up` (src/model/swiglu.cpp:27-29).
__device__ __forceinline__ float silu_ref(float value) {
    if (value == -INFINITY) return -0.0f;
    float s;
    if (value >= 0.0f) {
        s = 1.0f / (1.0f + expf(-value));
    } else {
        const float e = expf(value);
        s = e / (1.0f + e);
    }
    return value * s;
}

__global__ void __launch_bounds__(256)
silu_mul_kernel(const float* gate, const float* up, float* out,   // out may be gate or up
                __nv_bfloat16* __restrict__ out16, uint64_t n, uint32_t vec4) {
    sm100::pdl_launch_dependents();   // a following decode GEMV may start its set-up now
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    const uint64_t first = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (vec4 != 0u) {   // 16-byte accesses: four elements per thread and step
        const uint64_t n4 = n / 4;
        for (uint64_t i = first; i < n4; i += stride) {
            const float4 g = reinterpret_cast<const float4*>(gate)[i];
            const float4 u = reinterpret_cast<const float4*>(up)[i];
            const float4 o = make_float4(silu_ref(g.x) * u.x, silu_ref(g.y) * u.y, silu_ref(g.z) * u.z,
                                         silu_ref(g.w) * u.w);
            reinterpret_cast<float4*>(out)[i] = o;
            if (out16 != nullptr) {
                const __nv_bfloat162 lo = __floats2bfloat162_rn(o.x, o.y), hi = __floats2bfloat162_rn(o.z, o.w);
                uint2 packed;
                packed.x = *reinterpret_cast<const uint32_t*>(&lo);
                packed.y = *reinterpret_cast<const uint32_t*>(&hi);
                reinterpret_cast<uint2*>(out16)[i] = packed;
            }
        }
        return;
    }
    for (uint64_t i = first; i < n; i += stride) {
        const float o = silu_ref(gate[i]) * up[i];
        out[i] = o;
        if (out16 != nullptr) out16[i] = __float2bfloat16_rn(o);
    }
}

__global__ void __launch_bounds__(256)
add_kernel(const float* a, const float* b, float* out, uint64_t n) {   // out may be a or b
    sm100::pdl_launch_dependents();   // a following decode GEMV may start its set-up now
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        out[i] = a[i] + b[i];
    }
}

// Embedding rows for a batch of token ids (gather_rows in the reference,
// src/core/backend/nn/reference/operations.cpp). An id >= vocab sets bit 0 of status.
__global__ void __launch_bounds__(256)
gather_rows_kernel(const float* __restrict__ table, const uint32_t* __restrict__ ids, float* __restrict__ out,
                   uint32_t width, uint32_t vocab, uint32_t* status) {
    sm100::pdl_launch_dependents();   // a following decode GEMV may start its set-up now
    const uint32_t row = blockIdx.x;
    uint32_t id = ids[row];
    if (id >= vocab) {
        if (threadIdx.x == 0 && status != nullptr) atomicOr(status, 1u);
        id = 0;
    }
    for (uint32_t c = threadIdx.x; c < width; c += blockDim.x) {
        out[static_cast<uint64_t>(row) * width + c] = table[static_cast<uint64_t>(id) * width + c];
    }
}

// Greedy sampling: index of the first maximum of each row
// (src/stages/serving/generation.cpp:100-120 keeps the lowest index on ties).
__global__ void __launch_bounds__(1024)
argmax_kernel(const float* __restrict__ logits, uint32_t* __restrict__ out, uint32_t width, uint32_t vec4) {
    __shared__ float s_val[1024];
    __shared__ uint32_t s_idx[1024];
    const float* r = logits + static_cast<uint64_t>(blockIdx.x) * width;
    float best = -INFINITY;
    uint32_t best_i = 0xFFFFFFFFu;
    auto take = [&](float v, uint32_t c) {   // columns reach a thread in increasing order
        if (v > best || best_i == 0xFFFFFFFFu) {
            best = v;
            best_i = c;
        }
    };
    if (vec4) {
        const float4* r4 = reinterpret_cast<const float4*>(r);
        for (uint32_t c = threadIdx.x; c < width / 4; c += blockDim.x) {
            const float4 v = __ldg(r4 + c);
            take(v.x, 4 * c);
            take(v.y, 4 * c + 1);
            take(v.z, 4 * c + 2);
            take(v.w, 4 * c + 3);
        }
    } else {
        for (uint32_t c = threadIdx.x; c < width; c += blockDim.x) take(r[c], c);
    }
    s_val[threadIdx.x] = best;
    s_idx[threadIdx.x] = best_i;
    __syncthreads();
    for (uint32_t s = blockDim.x / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
            const float ov = s_val[threadIdx.x + s];
            const uint32_t oi = s_idx[threadIdx.x + s];
            const float mv = s_val[threadIdx.x];
            const uint32_t mi = s_idx[threadIdx.x];
            if (oi != 0xFFFFFFFFu && (mi == 0xFFFFFFFFu || ov > mv || (ov == mv && oi < mi))) {
                s_val[threadIdx.x] = ov;
                s_idx[threadIdx.x] = oi;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) out[blockIdx.x] = s_idx[0];
}

unsigned grid_for(uint64_t n, int sm_count) {
    uint64_t blocks = (n + 255) / 256;
    const uint64_t cap = static_cast<uint64_t>(sm_count > 0 ? sm_count : 148) * 8;
    if (blocks > cap) blocks = cap;
    return static_cast<unsigned>(blocks == 0 ? 1 : blocks);
}

}  // namespace

int32_t launch_rmsnorm(const float* x, const float* delta, float* x_out, const float* scale, float* y,
                       void* y_bf16, uint64_t rows, uint32_t width, float eps, cudaStream_t stream) {
    const bool vec4 = width % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) |
                                          reinterpret_cast<uintptr_t>(y_bf16) |
                                          reinterpret_cast<uintptr_t>(scale) | reinterpret_cast<uintptr_t>(delta) |
                                          reinterpret_cast<uintptr_t>(x_out)) & 15u) == 0;
    unsigned threads = 256;
    if (vec4) {
        threads = (width / 4 + 31) / 32 * 32;
        if (threads > 1024) threads = 1024;
        if (threads < 64) threads = 64;
    }
    rmsnorm_kernel<<<static_cast<unsigned>(rows), threads, 0, stream>>>(
        x, delta, x_out, scale, y, static_cast<__nv_bfloat16*>(y_bf16), width, eps, vec4 ? 1u : 0u);
    B2_CUDA_TRY(cudaGetLastError());
    return B2_STATUS_OK;
}

int32_t launch_rope_append(float* q, const float* k, const float* v, const uint32_t* positions,
                           const uint32_t* token_seq, const uint32_t* block_tables, float* k_pages,
                           float* v_pages, uint32_t n_seq,
                           uint32_t q_heads, uint32_t kv_heads, uint32_t d, uint32_t block_size,
                           uint64_t physical_blocks, uint32_t max_blocks, float theta, uint32_t* status,
                           cudaStream_t stream) {
    // two items per thread, at most 16 slices per sequence
    const uint32_t pairs = (q_heads + kv_heads) * (d / 2);
    uint32_t slices = (pairs + 511u) / 512u;
    slices = slices == 0 ? 1u : (slices > 16u ? 16u : slices);
    rope_append_kernel<<<dim3(n_seq, slices), 256, 0, stream>>>(q, k, v, positions, token_seq, block_tables, k_pages, v_pages, q_heads,
                                                  kv_heads, d, block_size, physical_blocks, max_blocks, theta,
                                                  status);
    B2_CUDA_TRY(cudaGetLastError());
    return B2_STATUS_OK;
}

int32_t launch_silu_mul(const DeviceContext& ctx, const float* gate, const float* up, float* out, void* out_bf16,
                        uint64_t n, cudaStream_t stream) {
    const bool vec4 = n % 4 == 0 && ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) |
                                      reinterpret_cast<uintptr_t>(out)) & 15u) == 0 &&
                      (reinterpret_cast<uintptr_t>(out_bf16) & 7u) == 0;
    silu_mul_kernel<<<grid_for(vec4 ? n / 4 : n, ctx.sm_count), 256, 0, stream>>>(
        gate, up, out, static_cast<__nv_bfloat16*>(out_bf16), n, vec4 ? 1u : 0u);
    B2_CUDA_TRY(cudaGetLastError());
    return B2_STATUS_OK;
}

int32_t launch_add(const DeviceContext& ctx, const float* a, const float* b, float* out, uint64_t n,
                   cudaStream_t stream) {
    add_kernel<<<grid_for(n, ctx.sm_count), 256, 0, stream>>>(a, b, out, n);
    B2_CUDA_TRY(cudaGetLastError());
    return B2_STATUS_OK;
}

int32_t launch_gather_rows(const float* table, const uint32_t* ids, float* out, uint32_t rows, uint32_t width,
                           uint32_t vocab, uint32_t* status, cudaStream_t stream) {
    gather_rows_kernel<<<rows, 256, 0, stream>>>(table, ids, out, width, vocab, status);
    B2_CUDA_TRY(cudaGetLastError());
    return B2_STATUS_OK;
}

int32_t launch_argmax(const float* logits, uint32_t* out, uint32_t rows, uint32_t width, cudaStream_t stream) {
    const bool vec4 = width % 4 == 0 && (reinterpret_cast<uintptr_t>(logits) & 15u) == 0;
    unsigned threads = 256;   // a power of two: the tree reduction halves it
    while (threads < 1024 && static_cast<uint64_t>(threads) * (vec4 ? 8 : 2) < width) threads *= 2;
    argmax_kernel<<<rows, threads, 0, stream>>>(logits, out, width, vec4 ? 1u : 0u);
    B2_CUDA_TRY(cudaGetLastError());
    return B2_STATUS_OK;
}

}  // namespace b2
