// Shared host/device helpers of the riftco_b200 library: status handling, the
// NF4 codebook, and the bit-exact block-scale decode used by every kernel.
#pragma once

#include "riftco_b200.h"

#include <cuda_runtime.h>

#include <cfloat>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <mutex>

namespace b2 {

// ---- errors -----------------------------------------------------------------

// Records a printf-style message for b2_last_error() and returns `status`.
int32_t fail(int32_t status, const char* format, ...);
void clear_error();

// Maps a CUDA runtime error to a status (cudaErrorMemoryAllocation becomes
// OUT_OF_MEMORY, as in the reference's src/core/backend/nn/cuda/common.cuh:21-28).
int32_t fail_cuda(cudaError_t error, const char* what);

#define B2_CUDA_TRY(expr)                                       \
    do {                                                        \
        const cudaError_t b2_err_ = (expr);                     \
        if (b2_err_ != cudaSuccess) {                           \
            return ::b2::fail_cuda(b2_err_, #expr);             \
        }                                                       \
    } while (0)

#define B2_TRY(expr)                                            \
    do {                                                        \
        const int32_t b2_status_ = (expr);                      \
        if (b2_status_ != B2_STATUS_OK) return b2_status_;      \
    } while (0)

// ---- per-device state ---------------------------------------------------------

struct DeviceContext {
    int device = -1;
    int sm_count = 0;
    int cc_major = 0;
    // 256 rows of 256 bytes; row v holds, for each of 32 lanes at byte 4*lane,
    // the two fp16 codebook values of packed byte v (low nibble in the low half).
    uint32_t* gemv_lut = nullptr;
    // Same table with bf16 pairs, compact [256][32] words, for the prefill GEMM.
    uint32_t* gemm_lut = nullptr;
    // Device word the GEMM sets when a bounded barrier wait gives up.
    uint32_t* gemm_error = nullptr;
    // Library-owned scratch arena used when a caller passes no workspace.
    void* arena = nullptr;
    size_t arena_bytes = 0;
    // Scratch of the decode-batch linear: partial tiles of CTAs whose range ends inside a tile
    // (fixed size, 2 per SM) and a ring of per-tile arrival counters (zero between launches).
    void* decode_partial = nullptr;
    uint32_t* decode_counters = nullptr;
    uint32_t decode_counter_capacity = 0;
    uint32_t decode_counter_next = 0;
    // Staging buffers of the host-buffer seam.
    void* stage = nullptr;
    size_t stage_bytes = 0;
    void* pinned = nullptr;
    size_t pinned_bytes = 0;
};

// Returns the lazily created context of the current device, or nullptr after
// recording an error (no device, wrong architecture, allocation failure).
DeviceContext* device_context(int32_t* status);

// Grows (never shrinks) the arena / staging buffers. Growing allocates, so it is
// refused while `stream` is being captured; an arena that has been handed out is
// never freed (graphs that captured its address stay valid), a larger one simply
// replaces it for later calls.
int32_t reserve_arena(DeviceContext* ctx, size_t bytes, cudaStream_t stream);
// `count` zeroed arrival counters for one launch of the decode-batch linear.
int32_t take_decode_counters(DeviceContext* ctx, uint32_t count, uint32_t** out);
int32_t reserve_stage(DeviceContext* ctx, size_t device_bytes, size_t pinned_bytes);

// Attributes set with cudaFuncSetAttribute (and occupancy answers) belong to ONE device, and a
// process may drive several. `once_per_device` runs `configure` (returning a status) the first time
// a device is seen, under a once_flag, and reports its outcome on every later call.
constexpr int kMaxDevices = 64;
struct PerDeviceOnce {
    std::once_flag flag[kMaxDevices];
    int32_t status[kMaxDevices] = {};
};
template <class Configure>
inline int32_t once_per_device(PerDeviceOnce& state, int device, Configure&& configure) {
    if (device < 0 || device >= kMaxDevices) return fail(B2_STATUS_RUNTIME_ERROR, "internal: device index out of range");
    std::call_once(state.flag[device], [&] { state.status[device] = configure(); });
    if (state.status[device] != B2_STATUS_OK) {
        return fail(state.status[device], "a kernel could not be configured on device %d", device);
    }
    return B2_STATUS_OK;
}

// ---- weight view ----------------------------------------------------------------

struct WeightView {
    const uint8_t* codes;
    const float* fp32_scales;     // encoding 0
    const uint8_t* scale_codes;   // encoding 1
    const float* second_level;    // encoding 1
    uint32_t encoding;
    uint32_t block_size;
    uint32_t block_shift;         // log2(block_size)
    uint32_t scale_block_shift;   // log2(scale_block_size), encoding 1
    float offset;
    uint64_t out_features;
    uint64_t in_features;
    uint64_t flat_block_base;
};

// Validates the struct (pointers, power-of-two block sizes, overflow) the way
// require_weight_storage / require_dimensions do in the reference
// (src/core/backend/nn/quantized_linear/dispatch.cpp:203-258) and fills `view`.
int32_t make_weight_view(const b2_nf4_weight* weight, WeightView* view);

// ---- device helpers ---------------------------------------------------------------

#if defined(__CUDACC__)

// src/core/quantization/nf4.cpp:14-31. Indices are part of the stored format.
static __device__ __constant__ float kNf4Codebook[16] = {
    -1.0f,
    -0.6961928009986877f,
    -0.5250730514526367f,
    -0.39491748809814453f,
    -0.28444138169288635f,
    -0.18477343022823334f,
    -0.09105003625154495f,
    0.0f,
    0.07958029955625534f,
    0.16093020141124725f,
    0.24611230194568634f,
    0.33791524171829224f,
    0.44070982933044434f,
    0.5626170039176941f,
    0.7229568362236023f,
    1.0f,
};

// float(code - 128) / 127.0f with IEEE division, the first rounding of the
// double-quantised decode (storage.hpp:55-57).
__device__ __forceinline__ float dq_factor(uint32_t scale_code) {
    return __fdiv_rn(static_cast<float>(static_cast<int>(scale_code) - 128), 127.0f);
}

// Second and third roundings (multiply, then add) kept separate so the
// compiler cannot contract them into an FMA (storage.hpp:57-64).
__device__ __forceinline__ float dq_finish(float factor, float second, float offset) {
    const float delta = __fmul_rn(second, factor);
    if (delta > 0.0f && offset > __fsub_rn(FLT_MAX, delta)) return FLT_MAX;
    const float s = __fadd_rn(offset, delta);
    return s > 0.0f ? s : 0.0f;
}

// Decoded scale of local block `block` (index inside this view).
__device__ __forceinline__ float decode_block_scale(const WeightView& w, uint64_t block) {
    if (w.encoding == B2_SCALES_FLOAT32) return __ldg(w.fp32_scales + block);
    const uint32_t code = __ldg(w.scale_codes + block);
    const float second = __ldg(w.second_level + ((w.flat_block_base + block) >> w.scale_block_shift));
    return dq_finish(dq_factor(code), second, w.offset);
}

__device__ __forceinline__ uint32_t nf4_code_at(const uint8_t* codes, uint64_t flat) {
    const uint32_t byte = __ldg(codes + (flat >> 1));
    return (flat & 1u) ? (byte >> 4) : (byte & 0x0Fu);
}

#endif  // __CUDACC__

}  // namespace b2
