// C-ABI layer of riftco_b200: argument validation mirroring the reference's
// dispatch layer, per-device state, kernel selection, and the synchronous
// host-buffer forms that a reference BackendAdapter calls.
#include "b2_common.cuh"
#include "b2_kernels.h"

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

namespace b2 {
namespace {

thread_local std::string g_last_error;
thread_local std::string g_unavailable_reason;

DeviceContext g_contexts[kMaxDevices];
std::once_flag g_context_once[kMaxDevices];
int32_t g_context_status[kMaxDevices];
std::string g_context_error[kMaxDevices];
std::mutex g_arena_mutex;
// Arenas that were replaced by a larger one. They are kept until the process exits: a CUDA graph
// may have captured their address.
std::vector<void*> g_retired_arenas;
// The host-buffer forms share one staging buffer per device; a call holds this lock from its first
// copy to its final synchronise.
std::mutex g_host_mutex[kMaxDevices];

constexpr uint32_t kDecodeCounterCapacity = 1u << 20;

bool is_power_of_two(uint64_t v) { return v != 0 && (v & (v - 1)) == 0; }

uint32_t log2_u64(uint64_t v) {
    uint32_t s = 0;
    while ((1ull << s) < v) ++s;
    return s;
}

// nf4_block_size_supported, src/core/quantization/nf4.cpp:39-52.
bool block_size_supported(uint64_t v) { return is_power_of_two(v) && v >= 32 && v <= 4096; }

bool mul_overflows(uint64_t a, uint64_t b, uint64_t* out) {
    if (a != 0 && b > UINT64_MAX / a) return true;
    *out = a * b;
    return false;
}

}  // namespace

// The kernel family the calling thread's last linear or attention call was served by, so that a
// test can tell which path a shape took.
thread_local int32_t g_last_route = B2_ROUTE_NONE;
void note_route(int32_t route) { g_last_route = route; }

int32_t fail(int32_t status, const char* format, ...) {
    char buffer[512];
    va_list args;
    va_start(args, format);
    vsnprintf(buffer, sizeof(buffer), format, args);
    va_end(args);
    g_last_error = buffer;
    return status;
}

void clear_error() { g_last_error.clear(); }

int32_t fail_cuda(cudaError_t error, const char* what) {
    const int32_t status =
        error == cudaErrorMemoryAllocation ? B2_STATUS_OUT_OF_MEMORY : B2_STATUS_RUNTIME_ERROR;
    return fail(status, "CUDA error in %s: %s", what, cudaGetErrorString(error));
}

DeviceContext* device_context(int32_t* status) {
    int device = -1;
    const cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess || device < 0 || device >= kMaxDevices) {
        cudaGetLastError();
        *status = fail(B2_STATUS_BACKEND_UNAVAILABLE, "CUDA backend unavailable: %s",
                       err != cudaSuccess ? cudaGetErrorString(err) : "device index out of range");
        return nullptr;
    }
    std::call_once(g_context_once[device], [device] {
        DeviceContext& ctx = g_contexts[device];
        cudaDeviceProp prop;
        cudaError_t e = cudaGetDeviceProperties(&prop, device);
        if (e != cudaSuccess) {
            g_context_status[device] = B2_STATUS_BACKEND_UNAVAILABLE;
            g_context_error[device] = std::string("CUDA backend unavailable: ") + cudaGetErrorString(e);
            return;
        }
        if (prop.major != 10) {
            g_context_status[device] = B2_STATUS_BACKEND_UNAVAILABLE;
            g_context_error[device] = "CUDA backend unavailable: this library is built for sm_100a "
                                      "(compute capability 10.x) only, device reports " +
                                      std::to_string(prop.major) + "." + std::to_string(prop.minor);
            return;
        }
        ctx.device = device;
        ctx.sm_count = prop.multiProcessorCount;
        ctx.cc_major = prop.major;
        int32_t s = init_gemv_lut(&ctx);
        if (s == B2_STATUS_OK) s = init_gemm_lut(&ctx);
        if (s == B2_STATUS_OK) {
            cudaError_t ce = cudaMalloc(&ctx.decode_partial, nf4_decode_tmem_workspace_bytes(ctx));
            if (ce == cudaSuccess) ce = cudaMalloc(&ctx.decode_counters, kDecodeCounterCapacity * sizeof(uint32_t));
            if (ce == cudaSuccess) ce = cudaMemset(ctx.decode_counters, 0, kDecodeCounterCapacity * sizeof(uint32_t));
            if (ce == cudaSuccess) ce = cudaDeviceSynchronize();
            if (ce != cudaSuccess) s = fail_cuda(ce, "decode scratch allocation");
            ctx.decode_counter_capacity = kDecodeCounterCapacity;
        }
        if (s != B2_STATUS_OK) {
            g_context_status[device] = s;
            g_context_error[device] = g_last_error;
            return;
        }
        g_context_status[device] = B2_STATUS_OK;
    });
    if (g_context_status[device] != B2_STATUS_OK) {
        *status = fail(g_context_status[device], "%s", g_context_error[device].c_str());
        return nullptr;
    }
    *status = B2_STATUS_OK;
    return &g_contexts[device];
}

int32_t reserve_arena(DeviceContext* ctx, size_t bytes, cudaStream_t stream) {
    std::lock_guard<std::mutex> lock(g_arena_mutex);
    if (bytes <= ctx->arena_bytes) return B2_STATUS_OK;
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &capture) != cudaSuccess) {
        cudaGetLastError();
        capture = cudaStreamCaptureStatusNone;
    }
    if (capture != cudaStreamCaptureStatusNone) {
        return fail(B2_STATUS_INVALID_ARGUMENT,
                    "the library's scratch arena would have to grow to %zu bytes inside a stream capture: make one "
                    "call of this size outside the capture first, or pass a workspace", bytes);
    }
    const size_t rounded = (bytes + (size_t{1} << 20) - 1) & ~((size_t{1} << 20) - 1);
    void* fresh = nullptr;
    B2_CUDA_TRY(cudaMalloc(&fresh, rounded));
    if (ctx->arena != nullptr) g_retired_arenas.push_back(ctx->arena);
    ctx->arena = fresh;
    ctx->arena_bytes = rounded;
    return B2_STATUS_OK;
}

int32_t take_decode_counters(DeviceContext* ctx, uint32_t count, uint32_t** out) {
    std::lock_guard<std::mutex> lock(g_arena_mutex);
    if (count > ctx->decode_counter_capacity) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "too many weight-row tiles for one decode launch");
    }
    if (ctx->decode_counter_next + count > ctx->decode_counter_capacity) ctx->decode_counter_next = 0;
    *out = ctx->decode_counters + ctx->decode_counter_next;
    ctx->decode_counter_next += count;
    return B2_STATUS_OK;
}

int32_t reserve_stage(DeviceContext* ctx, size_t device_bytes, size_t pinned_bytes) {
    std::lock_guard<std::mutex> lock(g_arena_mutex);
    if (device_bytes > ctx->stage_bytes) {
        B2_CUDA_TRY(cudaDeviceSynchronize());
        if (ctx->stage != nullptr) B2_CUDA_TRY(cudaFree(ctx->stage));
        ctx->stage = nullptr;
        ctx->stage_bytes = 0;
        B2_CUDA_TRY(cudaMalloc(&ctx->stage, device_bytes));
        ctx->stage_bytes = device_bytes;
    }
    if (pinned_bytes > ctx->pinned_bytes) {
        B2_CUDA_TRY(cudaDeviceSynchronize());
        if (ctx->pinned != nullptr) B2_CUDA_TRY(cudaFreeHost(ctx->pinned));
        ctx->pinned = nullptr;
        ctx->pinned_bytes = 0;
        B2_CUDA_TRY(cudaMallocHost(&ctx->pinned, pinned_bytes));
        ctx->pinned_bytes = pinned_bytes;
    }
    return B2_STATUS_OK;
}

int32_t make_weight_view(const b2_nf4_weight* weight, WeightView* view) {
    if (weight == nullptr) return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 weight must not be null");
    if (weight->out_features == 0 || weight->in_features == 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 weight dimensions must be positive");
    }
    uint64_t numel = 0;
    if (mul_overflows(weight->out_features, weight->in_features, &numel)) {
        return fail(B2_STATUS_OVERFLOW, "NF4 weight element count overflows");
    }
    if (weight->block_size == 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 block size must be greater than zero");
    }
    if (!block_size_supported(weight->block_size)) {
        return fail(B2_STATUS_INVALID_ARGUMENT,
                    "NF4 block size must be a power of two between 32 and 4096");
    }
    if (weight->codes == nullptr || weight->scales_primary == nullptr) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 packed codes and scales must not be null");
    }
    if (weight->reserved != 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 weight reserved field must be zero");
    }
    view->codes = weight->codes;
    view->encoding = weight->encoding;
    view->block_size = weight->block_size;
    view->block_shift = log2_u64(weight->block_size);
    view->out_features = weight->out_features;
    view->in_features = weight->in_features;
    view->flat_block_base = weight->flat_block_base;
    view->fp32_scales = nullptr;
    view->scale_codes = nullptr;
    view->second_level = nullptr;
    view->scale_block_shift = 0;
    view->offset = 0.0f;
    if (weight->encoding == B2_SCALES_FLOAT32) {
        // require_scale_storage, dispatch.cpp:112-123: the legacy form carries
        // no second level, block size or offset.
        if (weight->scales_secondary != nullptr || weight->scale_block_size != 0 ||
            weight->scale_offset != 0.0f) {
            return fail(B2_STATUS_INVALID_ARGUMENT,
                        "legacy NF4 scale storage has an invalid representation");
        }
        if ((reinterpret_cast<uintptr_t>(weight->scales_primary) & 3u) != 0) {
            return fail(B2_STATUS_INVALID_ARGUMENT, "FP32 NF4 scales must be 4-byte aligned");
        }
        view->fp32_scales = static_cast<const float*>(weight->scales_primary);
    } else if (weight->encoding == B2_SCALES_DOUBLE_QUANTIZED_UINT8) {
        // dispatch.cpp:124-137.
        if (weight->scales_secondary == nullptr || !block_size_supported(weight->scale_block_size) ||
            !std::isfinite(weight->scale_offset) || weight->scale_offset < 0.0f) {
            return fail(B2_STATUS_INVALID_ARGUMENT,
                        "double-quantized NF4 scale storage has an invalid representation");
        }
        view->scale_codes = static_cast<const uint8_t*>(weight->scales_primary);
        view->second_level = weight->scales_secondary;
        view->scale_block_shift = log2_u64(weight->scale_block_size);
        view->offset = weight->scale_offset;
    } else {
        return fail(B2_STATUS_INVALID_ARGUMENT, "unknown NF4 scale encoding");
    }
    return B2_STATUS_OK;
}

namespace {

// require_dimensions + size products, dispatch.cpp:244-258,322-331.
int32_t check_linear_dims(const WeightView& w, uint64_t rows) {
    if (rows == 0) return fail(B2_STATUS_INVALID_ARGUMENT, "quantized linear needs at least one row");
    uint64_t tmp = 0;
    if (mul_overflows(rows, w.in_features, &tmp) || mul_overflows(tmp, w.out_features, &tmp)) {
        return fail(B2_STATUS_OVERFLOW, "quantized linear dimension product overflows");
    }
    return B2_STATUS_OK;
}

bool aliases_weight(const b2_nf4_weight* weight, const void* p) {
    return p == weight->codes || p == weight->scales_primary ||
           (weight->scales_secondary != nullptr && p == weight->scales_secondary);
}


// Which decode kernel serves a forward call of up to 32 rows: 17..32 rows go to the persistent
// tcgen05 decode kernel, fewer to the mma.sync decode kernel - except 9..16 rows on a contraction
// of 8192 or more, where the persistent kernel (fp16 form, conversion pass included) measured
// faster (16 rows, 14336 -> 4096: 20.7 against 24.9 us; on 4096-wide layers the mma.sync kernel
// wins). B2_DECODE_IMPL=tmem sends every batch of up to 32 rows to the persistent kernel.
bool decode_tmem_wanted(uint64_t rows, uint64_t in_features) {
    static const char* impl = getenv("B2_DECODE_IMPL");
    if (rows > 32) return false;
    if (impl != nullptr && strcmp(impl, "tmem") == 0) return true;
    return rows > 16 || (rows > 8 && in_features >= 8192);
}

// The kernel family the calling thread's last linear or attention call was served by
// (B2_ROUTE_* of the header), so that a test can tell which path a shape took.
size_t pad256(size_t v) { return (v + 255) & ~size_t{255}; }

// Scratch of the persistent decode kernel when the caller passes FP32 activations: their 16-bit
// copy, then the partial tiles.
size_t decode_tmem_workspace_bytes(const DeviceContext& ctx, const WeightView& w, uint64_t rows) {
    return pad256(static_cast<size_t>(rows) * w.in_features * 2) + nf4_decode_tmem_workspace_bytes(ctx);
}

// `count` weights of one input width on the persistent decode kernel. Either `x` (FP32, converted
// here: fp16 up to 16 rows, bf16 above) or `x_bf16` is given. With a caller workspace all scratch
// comes from it; without one the 16-bit copy lives in the arena and the partial tiles in the
// per-device buffer.
int32_t decode_tmem_forward(DeviceContext* ctx, const WeightView* views, float* const* ys, uint32_t count,
                            const float* x, const void* x_bf16, uint64_t rows, void* workspace,
                            size_t workspace_bytes, cudaStream_t stream) {
    const bool half = x_bf16 == nullptr && rows <= 16;
    const size_t x16_bytes = x_bf16 != nullptr ? 0 : pad256(static_cast<size_t>(rows) * views[0].in_features * 2);
    const size_t partial_bytes = nf4_decode_tmem_workspace_bytes(*ctx);
    void* x16 = const_cast<void*>(x_bf16);
    void* partial = ctx->decode_partial;
    if (workspace != nullptr) {
        if ((reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) {
            return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 GEMM workspace must be 16-byte aligned");
        }
        if (workspace_bytes < x16_bytes + partial_bytes) {
            return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 GEMM workspace too small: need %zu bytes",
                        x16_bytes + partial_bytes);
        }
        if (x_bf16 == nullptr) x16 = workspace;
        partial = static_cast<uint8_t*>(workspace) + x16_bytes;
    } else if (x_bf16 == nullptr) {
        B2_TRY(reserve_arena(ctx, x16_bytes, stream));
        x16 = ctx->arena;
    }
    if (x_bf16 == nullptr) {
        const uint64_t n = rows * views[0].in_features;
        if (half) {
            B2_TRY(launch_f32_to_f16(*ctx, x, x16, n, stream));
        } else {
            B2_TRY(launch_f32_to_bf16(*ctx, x, x16, n, stream));
        }
    }
    uint64_t tiles = 0;
    for (uint32_t i = 0; i < count; ++i) tiles += (views[i].out_features + 127) / 128;
    uint32_t* counters = nullptr;
    B2_TRY(take_decode_counters(ctx, static_cast<uint32_t>(tiles), &counters));
    return launch_nf4_decode_tmem(*ctx, views, ys, count, x16, half, rows, partial, counters, stream);
}

bool decode_tmem_takes(const WeightView* views, uint32_t count, const void* x, uint64_t rows) {
    if (!decode_tmem_wanted(rows, views[0].in_features)) return false;
    for (uint32_t i = 0; i < count; ++i) {
        if (!nf4_decode_tmem_supported(views[i], x, rows)) return false;
        if (views[i].encoding != views[0].encoding || views[i].block_size != views[0].block_size ||
            views[i].scale_block_shift != views[0].scale_block_shift ||
            views[i].in_features != views[0].in_features) {
            return false;
        }
    }
    return true;
}

int32_t linear_forward_impl(const b2_nf4_weight* weight, const float* x, float* y, uint64_t rows,
                            void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    int32_t status = B2_STATUS_OK;
    DeviceContext* ctx = device_context(&status);
    if (ctx == nullptr) return status;
    WeightView w;
    B2_TRY(make_weight_view(weight, &w));
    B2_TRY(check_linear_dims(w, rows));
    if (x == nullptr || y == nullptr) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "quantized linear input and output must not be null");
    }
    if (x == y) return fail(B2_STATUS_INVALID_ARGUMENT, "quantized linear input and output must not alias");
    if (aliases_weight(weight, y)) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "quantized linear weight and output storage must not alias");
    }
    if (decode_tmem_takes(&w, 1, x, rows)) {
        float* ys[1] = {y};
        note_route(B2_ROUTE_DECODE_TMEM);
        return decode_tmem_forward(ctx, &w, ys, 1, x, nullptr, rows, workspace, workspace_bytes, stream);
    }
    // More than 16 batch rows: the tcgen05 kernel that keeps the expanded weight tile in tensor
    // memory (speculative / chunked prefill, full prefill, and decode batches whose shape the
    // persistent decode kernel does not take).
    if (rows > 16 && nf4_gemm_tmem_supported(w, x, rows)) {
        const size_t need = nf4_gemm_tmem_workspace_bytes(w, rows);
        if (workspace == nullptr) {
            B2_TRY(reserve_arena(ctx, need, stream));
            workspace = ctx->arena;
            workspace_bytes = ctx->arena_bytes;
        }
        if (workspace_bytes < need) {
            return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 GEMM workspace too small: need %zu bytes", need);
        }
        if ((reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) {
            return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 GEMM workspace must be 16-byte aligned");
        }
        note_route(B2_ROUTE_GEMM_TMEM);
        B2_TRY(launch_f32_to_bf16(*ctx, x, workspace, rows * w.in_features, stream));
        return launch_nf4_gemm_tmem(*ctx, w, workspace, y, rows, stream);
    }
    if (nf4_gemv_supported(w, x, y, rows)) {
        // What the two tcgen05 kernels above did not take (up to 16 rows; 17..32 rows of a weight
        // whose codes are only 8-byte aligned): the TMA-fed mma.sync decode kernel, else the tiled
        // decode kernel, which takes any row count of the weight.
        uint32_t ksplit = 0, per = 0;
        if (rows <= 16 && nf4_gemv_tma_plan(*ctx, w, x, rows, &ksplit, &per)) {
            note_route(B2_ROUTE_GEMV_TMA);
            return launch_nf4_gemv_tma(*ctx, w, x, y, rows, ksplit, per, stream);
        }
        note_route(B2_ROUTE_GEMV_TILE);
        return launch_nf4_gemv(*ctx, w, x, y, rows, stream);
    }
    note_route(B2_ROUTE_GENERIC);
    return launch_nf4_linear_forward_generic(*ctx, w, x, y, rows, stream);
}

int32_t linear_backward_impl(const b2_nf4_weight* weight, const float* dy, float* dx, uint64_t rows,
                             void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    int32_t status = B2_STATUS_OK;
    DeviceContext* ctx = device_context(&status);
    if (ctx == nullptr) return status;
    WeightView w;
    B2_TRY(make_weight_view(weight, &w));
    B2_TRY(check_linear_dims(w, rows));
    if (dy == nullptr || dx == nullptr) {
        return fail(B2_STATUS_INVALID_ARGUMENT,
                    "quantized linear upstream and input gradient must not be null");
    }
    if (dy == dx) {
        return fail(B2_STATUS_INVALID_ARGUMENT,
                    "quantized linear upstream and input gradient must not alias");
    }
    if (aliases_weight(weight, dx)) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "quantized linear weight and output storage must not alias");
    }
    // From 512 rows: expand W once, transposed, into scratch and run a plain bf16 tcgen05 GEMM;
    // below that the kernel that transposes nibbles inside the SM.
    if (nf4_backward_dense_supported(w, dy, rows)) {
        const size_t need = nf4_backward_dense_workspace_bytes(w, rows);
        if (workspace == nullptr) {
            B2_TRY(reserve_arena(ctx, need, stream));
            workspace = ctx->arena;
            workspace_bytes = ctx->arena_bytes;
        }
        note_route(B2_ROUTE_BACKWARD_DENSE);
        return launch_nf4_backward_dense(*ctx, w, dy, dx, rows, workspace, workspace_bytes, stream);
    }
    if (nf4_gemm_supported(w, dy, rows, true)) {
        const size_t need = nf4_gemm_workspace_bytes(w, rows, true);
        if (workspace == nullptr) {
            B2_TRY(reserve_arena(ctx, need, stream));
            workspace = ctx->arena;
            workspace_bytes = ctx->arena_bytes;
        }
        note_route(B2_ROUTE_GEMM_SMEM);
        return launch_nf4_gemm(*ctx, w, dy, dx, rows, true, workspace, workspace_bytes, stream);
    }
    note_route(B2_ROUTE_GENERIC);
    return launch_nf4_linear_input_backward_generic(*ctx, w, dy, dx, rows, stream);
}

}  // namespace

// checked_paged_decode_query_size and the table checks of
// dispatch_paged_decode_attention_forward, attention/dispatch.cpp:179-219,440-509
// (the parts that need no host view of device data).
int32_t check_paged_dims(uint32_t n_seq, uint32_t q_heads, uint32_t kv_heads, uint32_t head_width,
                         uint32_t block_size, uint64_t physical_blocks, uint32_t max_blocks,
                         uint32_t max_seq_len) {
    if (n_seq == 0 || q_heads == 0 || kv_heads == 0 || head_width == 0 || block_size == 0 ||
        physical_blocks == 0 || max_seq_len == 0 || max_blocks == 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "paged decode attention dimensions must be positive");
    }
    if (physical_blocks - 1 > 0xFFFFFFFFull) {
        return fail(B2_STATUS_OVERFLOW, "paged decode attention physical block IDs exceed uint32_t");
    }
    if (q_heads % kv_heads != 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT,
                    "paged decode attention query heads must be a multiple of KV heads");
    }
    const uint64_t required_blocks = (static_cast<uint64_t>(max_seq_len) - 1) / block_size + 1;
    if (required_blocks > max_blocks) {
        return fail(B2_STATUS_INVALID_ARGUMENT,
                    "paged decode attention block table size does not match the sequence");
    }
    if (required_blocks > physical_blocks) {
        return fail(B2_STATUS_INVALID_ARGUMENT,
                    "paged decode attention has fewer physical than logical blocks");
    }
    uint64_t pool = 0;
    if (mul_overflows(physical_blocks, kv_heads, &pool) || mul_overflows(pool, block_size, &pool) ||
        mul_overflows(pool, head_width, &pool)) {
        return fail(B2_STATUS_OVERFLOW, "paged decode attention pool size overflows");
    }
    return B2_STATUS_OK;
}

}  // namespace b2

using namespace b2;

extern "C" {

int32_t b2_abi_version(void) { return B2_ABI_VERSION; }

const char* b2_last_error(void) { return g_last_error.c_str(); }

int32_t b2_is_available(void) {
    int32_t status = B2_STATUS_OK;
    const std::string saved = g_last_error;
    const bool ok = device_context(&status) != nullptr;
    if (!ok) g_unavailable_reason = g_last_error;
    g_last_error = saved;
    return ok ? 1 : 0;
}

const char* b2_unavailability_reason(void) {
    if (b2_is_available()) return "";
    return g_unavailable_reason.c_str();
}

int32_t b2_nf4_dequantize(const b2_nf4_weight* weight, float* out, void* stream) {
    clear_error();
    int32_t status = B2_STATUS_OK;
    DeviceContext* ctx = device_context(&status);
    if (ctx == nullptr) return status;
    WeightView w;
    B2_TRY(make_weight_view(weight, &w));
    if (out == nullptr) return fail(B2_STATUS_INVALID_ARGUMENT, "dequantize output must not be null");
    if (aliases_weight(weight, out)) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "dequantize output must not alias the packed weight");
    }
    return launch_nf4_dequantize(*ctx, w, out, static_cast<cudaStream_t>(stream));
}

size_t b2_nf4_quantize_workspace_bytes(uint64_t out_features, uint64_t in_features, uint32_t block_size,
                                       uint64_t scale_block_size) {
    int32_t status = B2_STATUS_OK;
    DeviceContext* ctx = device_context(&status);
    clear_error();
    uint64_t n = 0;
    if (ctx == nullptr || block_size == 0 || mul_overflows(out_features, in_features, &n)) return 0;
    return nf4_quantize_workspace_bytes(*ctx, (n + block_size - 1) / block_size, scale_block_size != 0);
}

int32_t b2_nf4_quantize(const float* values, uint64_t out_features, uint64_t in_features, uint32_t block_size,
                        uint64_t scale_block_size, uint8_t* codes, void* scales_primary, float* scales_secondary,
                        float* scale_offset, void* workspace, size_t workspace_bytes, void* stream) {
    clear_error();
    int32_t status = B2_STATUS_OK;
    DeviceContext* ctx = device_context(&status);
    if (ctx == nullptr) return status;
    if (out_features == 0 || in_features == 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 quantization requires a non-empty weight");
    }
    uint64_t n = 0;
    if (mul_overflows(out_features, in_features, &n)) return fail(B2_STATUS_OVERFLOW, "NF4 weight element count overflows");
    if (!block_size_supported(block_size)) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 block size must be a power of two between 32 and 4096");
    }
    if (scale_block_size != 0 && !block_size_supported(scale_block_size)) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 block size must be a power of two between 32 and 4096");
    }
    if (values == nullptr || codes == nullptr || scales_primary == nullptr ||
        (scale_block_size != 0 && scales_secondary == nullptr)) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 quantization pointers must not be null");
    }
    const size_t need = nf4_quantize_workspace_bytes(*ctx, (n + block_size - 1) / block_size, scale_block_size != 0);
    if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 quantization needs %zu bytes of 256-byte aligned workspace", need);
    }
    return run_nf4_quantize(*ctx, values, out_features, in_features, block_size, scale_block_size, codes,
                            scales_primary, scales_secondary, scale_offset, workspace, static_cast<cudaStream_t>(stream));
}

int32_t b2_nf4_validate_payload(const b2_nf4_weight* weight, uint64_t codes_bytes, uint64_t primary_count,
                                uint64_t secondary_count, void* stream) {
    clear_error();
    int32_t status = B2_STATUS_OK;
    DeviceContext* ctx = device_context(&status);
    if (ctx == nullptr) return status;
    WeightView w;
    B2_TRY(make_weight_view(weight, &w));
    const uint64_t n = w.out_features * w.in_features;
    const uint64_t blocks = (n + w.block_size - 1) / w.block_size;
    if (codes_bytes != (n + 1) / 2) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 packed byte count does not match the weight shape");
    }
    uint64_t second_needed = 0;
    if (w.encoding == B2_SCALES_FLOAT32) {
        if (primary_count != blocks) {
            return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 scale count does not match the weight shape and block size");
        }
    } else {
        if (primary_count != blocks) {
            return fail(B2_STATUS_INVALID_ARGUMENT, "double-quantized NF4 scale-code count does not match the weight");
        }
        // a whole weight has exactly ceil(blocks / group) second-level scales; a row shard shares its
        // parent's array and needs it to reach the shard's last block
        second_needed = ((w.flat_block_base + blocks - 1) >> w.scale_block_shift) + 1;
        if (w.flat_block_base == 0 ? secondary_count != second_needed : secondary_count < second_needed) {
            return fail(B2_STATUS_INVALID_ARGUMENT, "double-quantized NF4 second-level scale count is invalid");
        }
    }
    uint32_t* flags = nullptr;
    B2_CUDA_TRY(cudaMalloc(&flags, 256));
    const int32_t result = run_nf4_validate(*ctx, w, second_needed, flags, static_cast<cudaStream_t>(stream));
    cudaFree(flags);
    return result;
}

int32_t b2_nf4_linear_forward(const b2_nf4_weight* weight, const float* x, float* y, uint64_t rows,
                              void* workspace, size_t workspace_bytes, void* stream) {
    clear_error();
    return linear_forward_impl(weight, x, y, rows, workspace, workspace_bytes,
                               static_cast<cudaStream_t>(stream));
}

size_t b2_nf4_linear_lora_workspace_bytes(const b2_nf4_weight* weight, uint64_t rows, uint32_t rank) {
    return pad256(b2_nf4_linear_workspace_bytes(weight, rows, 0)) + lora_workspace_bytes(rows, rank);
}

int32_t b2_nf4_linear_forward_lora(const b2_nf4_weight* weight, const float* x, const float* lora_a,
                                   const float* lora_b, uint32_t rank, float scale, float* y, uint64_t rows,
                                   void* workspace, size_t workspace_bytes, void* stream_ptr) {
    clear_error();
    cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
    int32_t status = B2_STATUS_OK;
    DeviceContext* ctx = device_context(&status);
    if (ctx == nullptr) return status;
    if (lora_a == nullptr || lora_b == nullptr) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "LoRA factors must not be null");
    }
    if (weight == nullptr) return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 weight must not be null");
    // checked_rank / checked_alpha, src/nn/low_rank_adapter.cpp:20-62
    if (rank == 0 || rank > weight->in_features || rank > weight->out_features) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "LoRA rank must be positive and no larger than either width");
    }
    if (!lora_rank_supported(rank)) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "LoRA rank above 64 is not supported by this backend");
    }
    if (!std::isfinite(scale)) return fail(B2_STATUS_INVALID_ARGUMENT, "LoRA scale must be finite");
    if (y == lora_a || y == lora_b) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "quantized linear weight and output storage must not alias");
    }
    // scratch: the base kernel's part first, then the [rows, rank] reduction
    const size_t base_need = pad256(b2_nf4_linear_workspace_bytes(weight, rows, 0));
    const size_t lora_need = lora_workspace_bytes(rows, rank);
    clear_error();
    uint8_t* scratch = static_cast<uint8_t*>(workspace);
    if (workspace == nullptr) {
        B2_TRY(reserve_arena(ctx, base_need + lora_need, stream));
        scratch = static_cast<uint8_t*>(ctx->arena);
        workspace_bytes = ctx->arena_bytes;
    }
    if (workspace_bytes < base_need + lora_need) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 LoRA workspace too small: need %zu bytes", base_need + lora_need);
    }
    if ((reinterpret_cast<uintptr_t>(scratch) & 15u) != 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 GEMM workspace must be 16-byte aligned");
    }
    B2_TRY(linear_forward_impl(weight, x, y, rows, base_need != 0 ? scratch : nullptr, base_need, stream));
    return launch_lora_branch(*ctx, x, lora_a, lora_b, y, rows, weight->in_features, weight->out_features, rank, scale,
                              reinterpret_cast<float*>(scratch + base_need), stream);
}

int32_t b2_nf4_linear_forward_multi(const b2_nf4_weight* weights, uint32_t count, const float* x, float* const* ys,
                                    uint64_t rows, void* workspace, size_t workspace_bytes, void* stream_ptr) {
    clear_error();
    cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
    if (weights == nullptr || ys == nullptr || count == 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "quantized linear needs at least one weight and its output");
    }
    for (uint32_t i = 0; i < count; ++i) {
        for (uint32_t j = 0; j < i; ++j) {
            if (ys[i] != nullptr && ys[i] == ys[j]) {
                return fail(B2_STATUS_INVALID_ARGUMENT, "quantized linear outputs of one call must not alias");
            }
        }
    }
    int32_t status = B2_STATUS_OK;
    DeviceContext* ctx = device_context(&status);
    if (ctx == nullptr) return status;
    // One launch when every weight can take the tensor-memory kernel on the same activations;
    // otherwise the calls are simply made one after the other.
    bool fused = (rows > 16 || decode_tmem_wanted(rows, weights[0].in_features)) && count <= 4 && count > 1 && x != nullptr;
    WeightView views[4];
    for (uint32_t i = 0; fused && i < count; ++i) {
        if (ys[i] == nullptr || x == ys[i] || aliases_weight(&weights[i], ys[i]) ||
            make_weight_view(&weights[i], &views[i]) != B2_STATUS_OK ||
            check_linear_dims(views[i], rows) != B2_STATUS_OK ||
            views[i].in_features != views[0].in_features || !nf4_gemm_tmem_supported(views[i], x, rows)) {
            fused = false;   // let the single-weight path produce the precise error
        }
    }
    clear_error();
    if (!fused) {
        for (uint32_t i = 0; i < count; ++i) {
            B2_TRY(linear_forward_impl(&weights[i], x, ys[i], rows, workspace, workspace_bytes, stream));
        }
        return B2_STATUS_OK;
    }
    if (decode_tmem_takes(views, count, x, rows)) {
        note_route(B2_ROUTE_DECODE_TMEM);
        return decode_tmem_forward(ctx, views, ys, count, x, nullptr, rows, workspace, workspace_bytes, stream);
    }
    if (rows <= 16) {   // the prefill kernel is not used for so few rows: one call per weight
        for (uint32_t i = 0; i < count; ++i) {
            B2_TRY(linear_forward_impl(&weights[i], x, ys[i], rows, workspace, workspace_bytes, stream));
        }
        return B2_STATUS_OK;
    }
    const size_t need = nf4_gemm_tmem_workspace_bytes(views[0], rows);
    if (workspace == nullptr) {
        B2_TRY(reserve_arena(ctx, need, stream));
        workspace = ctx->arena;
        workspace_bytes = ctx->arena_bytes;
    }
    if (workspace_bytes < need) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 GEMM workspace too small: need %zu bytes", need);
    }
    if ((reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "NF4 GEMM workspace must be 16-byte aligned");
    }
    note_route(B2_ROUTE_GEMM_TMEM);
    B2_TRY(launch_f32_to_bf16(*ctx, x, workspace, rows * views[0].in_features, stream));
    return launch_nf4_gemm_tmem_multi(*ctx, views, ys, count, workspace, rows, stream);
}

int32_t b2_nf4_linear_input_backward(const b2_nf4_weight* weight, const float* dy, float* dx,
                                     uint64_t rows, void* workspace, size_t workspace_bytes,
                                     void* stream) {
    clear_error();
    return linear_backward_impl(weight, dy, dx, rows, workspace, workspace_bytes,
                                static_cast<cudaStream_t>(stream));
}

size_t b2_nf4_linear_workspace_bytes(const b2_nf4_weight* weight, uint64_t rows, int32_t backward) {
    WeightView w;
    if (make_weight_view(weight, &w) != B2_STATUS_OK) return 0;
    clear_error();
    if (backward == 0 && decode_tmem_takes(&w, 1, reinterpret_cast<const float*>(16), rows)) {
        int32_t status = B2_STATUS_OK;
        DeviceContext* ctx = device_context(&status);
        clear_error();
        if (ctx != nullptr) return decode_tmem_workspace_bytes(*ctx, w, rows);
    }
    if (backward == 0 && rows > 16 && nf4_gemm_tmem_supported(w, reinterpret_cast<const float*>(16), rows)) {
        return nf4_gemm_tmem_workspace_bytes(w, rows);
    }
    if (backward != 0 && nf4_backward_dense_supported(w, reinterpret_cast<const float*>(16), rows)) {
        return nf4_backward_dense_workspace_bytes(w, rows);
    }
    if (backward == 0 || !nf4_gemm_supported(w, reinterpret_cast<const float*>(16), rows, true)) return 0;
    return nf4_gemm_workspace_bytes(w, rows, true);
}

int32_t b2_last_route(void) { return g_last_route; }

size_t b2_paged_decode_workspace_bytes(uint32_t n_seq, uint32_t q_heads, uint32_t head_width,
                                       uint32_t block_size, uint32_t max_seq_len) {
    return paged_decode_workspace_bytes(n_seq, q_heads, head_width, block_size, max_seq_len);
}

namespace {

int32_t paged_decode_impl(const float* q, const float* k_pages, const float* v_pages,
                          const uint32_t* block_tables, const uint32_t* seq_lens, float* ctx_out,
                          void* ctx_bf16, uint32_t n_seq, uint32_t q_heads, uint32_t kv_heads,
                          uint32_t head_width, uint32_t block_size, uint64_t physical_blocks,
                          uint32_t max_blocks, uint32_t max_seq_len, void* workspace,
                          size_t workspace_bytes, uint32_t* status_word, void* stream) {
    clear_error();
    int32_t status = B2_STATUS_OK;
    DeviceContext* ctx = device_context(&status);
    if (ctx == nullptr) return status;
    B2_TRY(check_paged_dims(n_seq, q_heads, kv_heads, head_width, block_size, physical_blocks,
                            max_blocks, max_seq_len));
    if (q == nullptr || k_pages == nullptr || v_pages == nullptr || block_tables == nullptr ||
        seq_lens == nullptr || ctx_out == nullptr) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "paged decode attention pointers must not be null");
    }
    // require_distinct, attention/dispatch.cpp:504-506.
    if (ctx_out == q || ctx_out == k_pages || ctx_out == v_pages || ctx_bf16 == q || ctx_bf16 == k_pages ||
        ctx_bf16 == v_pages || ctx_bf16 == ctx_out) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "paged decode attention output must not alias an input");
    }
    if ((reinterpret_cast<uintptr_t>(ctx_bf16) & 1u) != 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "the bf16 copy must be 2-byte aligned");
    }
    PagedDecodeArgs args{q, k_pages, v_pages, block_tables, seq_lens, ctx_out,
                         n_seq, q_heads, kv_heads, head_width, block_size, max_blocks, max_seq_len,
                         physical_blocks, status_word, ctx_bf16};
    const size_t need =
        paged_decode_workspace_bytes(n_seq, q_heads, head_width, block_size, max_seq_len);
    if (workspace == nullptr && need > 0) {
        B2_TRY(reserve_arena(ctx, need, static_cast<cudaStream_t>(stream)));
        workspace = ctx->arena;
        workspace_bytes = ctx->arena_bytes;
    }
    return launch_paged_decode(*ctx, args, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

}  // namespace

int32_t b2_paged_decode_attention(const float* q, const float* k_pages, const float* v_pages,
                                  const uint32_t* block_tables, const uint32_t* seq_lens, float* ctx_out,
                                  uint32_t n_seq, uint32_t q_heads, uint32_t kv_heads,
                                  uint32_t head_width, uint32_t block_size, uint64_t physical_blocks,
                                  uint32_t max_blocks, uint32_t max_seq_len, void* workspace,
                                  size_t workspace_bytes, uint32_t* status_word, void* stream) {
    return paged_decode_impl(q, k_pages, v_pages, block_tables, seq_lens, ctx_out, nullptr, n_seq, q_heads,
                             kv_heads, head_width, block_size, physical_blocks, max_blocks, max_seq_len,
                             workspace, workspace_bytes, status_word, stream);
}

int32_t b2_paged_decode_attention_bf16(const float* q, const float* k_pages, const float* v_pages,
                                       const uint32_t* block_tables, const uint32_t* seq_lens, float* ctx_out,
                                       void* ctx_bf16, uint32_t n_seq, uint32_t q_heads, uint32_t kv_heads,
                                       uint32_t head_width, uint32_t block_size, uint64_t physical_blocks,
                                       uint32_t max_blocks, uint32_t max_seq_len, void* workspace,
                                       size_t workspace_bytes, uint32_t* status_word, void* stream) {
    if (ctx_bf16 == nullptr) {
        clear_error();
        return fail(B2_STATUS_INVALID_ARGUMENT, "paged decode attention pointers must not be null");
    }
    return paged_decode_impl(q, k_pages, v_pages, block_tables, seq_lens, ctx_out, ctx_bf16, n_seq, q_heads,
                             kv_heads, head_width, block_size, physical_blocks, max_blocks, max_seq_len,
                             workspace, workspace_bytes, status_word, stream);
}

namespace {

// Views of `count` weights that can all take the tensor-memory kernel on one bf16 activation
// matrix of `rows` rows; false when any of them cannot.
bool bf16_input_views(const b2_nf4_weight* weights, uint32_t count, const void* x_bf16, uint64_t rows,
                      WeightView* views) {
    if (weights == nullptr || count == 0 || count > 4 || rows <= 16) return false;
    for (uint32_t i = 0; i < count; ++i) {
        if (make_weight_view(&weights[i], &views[i]) != B2_STATUS_OK ||
            check_linear_dims(views[i], rows) != B2_STATUS_OK ||
            views[i].in_features != views[0].in_features ||
            !nf4_gemm_tmem_supported(views[i], static_cast<const float*>(x_bf16), rows)) {
            return false;
        }
    }
    return true;
}

}  // namespace

int32_t b2_nf4_linear_bf16_supported(const b2_nf4_weight* weights, uint32_t count, uint64_t rows) {
    clear_error();
    int32_t status = B2_STATUS_OK;
    if (device_context(&status) == nullptr) return 0;
    WeightView views[4];
    const bool ok = bf16_input_views(weights, count, nullptr, rows, views);
    clear_error();
    return ok ? 1 : 0;
}

int32_t b2_nf4_linear_forward_multi_bf16(const b2_nf4_weight* weights, uint32_t count, const void* x_bf16,
                                         float* const* ys, uint64_t rows, void* stream_ptr) {
    clear_error();
    if (weights == nullptr || ys == nullptr || count == 0 || x_bf16 == nullptr) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "quantized linear needs its weights, activations and outputs");
    }
    for (uint32_t i = 0; i < count; ++i) {
        if (ys[i] == nullptr || ys[i] == x_bf16 || aliases_weight(&weights[i], ys[i])) {
            return fail(B2_STATUS_INVALID_ARGUMENT, "quantized linear output must not be null or alias an input");
        }
        for (uint32_t j = 0; j < i; ++j) {
            if (ys[i] == ys[j]) {
                return fail(B2_STATUS_INVALID_ARGUMENT, "quantized linear outputs of one call must not alias");
            }
        }
    }
    int32_t status = B2_STATUS_OK;
    DeviceContext* ctx = device_context(&status);
    if (ctx == nullptr) return status;
    WeightView views[4];
    if (!bf16_input_views(weights, count, x_bf16, rows, views)) {
        return fail(B2_STATUS_INVALID_ARGUMENT,
                    "bf16 activations are taken only by the tensor-memory kernel (more than 16 rows, up to 4 "
                    "weights of one input width, 16-byte aligned rows); ask b2_nf4_linear_bf16_supported first");
    }
    clear_error();
    if (decode_tmem_takes(views, count, x_bf16, rows)) {
        note_route(B2_ROUTE_DECODE_TMEM);
        return decode_tmem_forward(ctx, views, ys, count, nullptr, x_bf16, rows, nullptr, 0,
                                   static_cast<cudaStream_t>(stream_ptr));
    }
    note_route(B2_ROUTE_GEMM_TMEM);
    return launch_nf4_gemm_tmem_multi(*ctx, views, ys, count, x_bf16, rows, static_cast<cudaStream_t>(stream_ptr));
}

// ---- decode-step glue ------------------------------------------------------------

int32_t b2_rmsnorm(const float* x, const float* delta, float* x_out, const float* scale, float* y,
                   uint64_t rows, uint64_t width, float eps, void* stream) {
    return b2_rmsnorm_bf16(x, delta, x_out, scale, y, nullptr, rows, width, eps, stream);
}

int32_t b2_rmsnorm_bf16(const float* x, const float* delta, float* x_out, const float* scale, float* y,
                        void* y_bf16, uint64_t rows, uint64_t width, float eps, void* stream) {
    clear_error();
    int32_t status = B2_STATUS_OK;
    if (device_context(&status) == nullptr) return status;
    if (x == nullptr || scale == nullptr || y == nullptr || (delta != nullptr && x_out == nullptr)) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "RMS normalization pointers must not be null");
    }
    if (rows == 0 || width == 0 || rows > 0x7FFFFFFFull || width > 0xFFFFFFFFull) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "RMS normalization requires positive dimensions");
    }
    if (!std::isfinite(eps) || eps <= 0.0f) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "RMS normalization epsilon must be finite and positive");
    }
    if ((reinterpret_cast<uintptr_t>(y_bf16) & 1u) != 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "the bf16 copy must be 2-byte aligned");
    }
    return launch_rmsnorm(x, delta, x_out, scale, y, y_bf16, rows, static_cast<uint32_t>(width), eps,
                          static_cast<cudaStream_t>(stream));
}

namespace {

int32_t rope_append_impl(float* q, const float* k, const float* v, const uint32_t* positions,
                         const uint32_t* token_seq, const uint32_t* block_tables, float* k_pages, float* v_pages,
                         uint32_t n_tokens, uint32_t q_heads, uint32_t kv_heads, uint32_t head_width,
                         uint32_t block_size, uint64_t physical_blocks, uint32_t max_blocks, float theta,
                         uint32_t* status_word, void* stream) {
    clear_error();
    int32_t status = B2_STATUS_OK;
    if (device_context(&status) == nullptr) return status;
    if (q == nullptr || k == nullptr || v == nullptr || positions == nullptr || block_tables == nullptr ||
        k_pages == nullptr || v_pages == nullptr) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "rotary/append pointers must not be null");
    }
    if (n_tokens == 0 || q_heads == 0 || kv_heads == 0 || head_width == 0 || block_size == 0 ||
        physical_blocks == 0 || max_blocks == 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "rotary/append dimensions must be positive");
    }
    if (head_width % 2 != 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "rotary embedding requires an even head width");
    }
    if (!std::isfinite(theta) || theta <= 0.0f) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "rotary theta must be finite and positive");
    }
    return launch_rope_append(q, k, v, positions, token_seq, block_tables, k_pages, v_pages, n_tokens, q_heads,
                              kv_heads, head_width, block_size, physical_blocks, max_blocks, theta, status_word,
                              static_cast<cudaStream_t>(stream));
}

}  // namespace

int32_t b2_rope_append_kv(float* q, const float* k, const float* v, const uint32_t* positions,
                          const uint32_t* block_tables, float* k_pages, float* v_pages, uint32_t n_seq,
                          uint32_t q_heads, uint32_t kv_heads, uint32_t head_width, uint32_t block_size,
                          uint64_t physical_blocks, uint32_t max_blocks, float theta, uint32_t* status_word,
                          void* stream) {
    return rope_append_impl(q, k, v, positions, nullptr, block_tables, k_pages, v_pages, n_seq, q_heads, kv_heads,
                            head_width, block_size, physical_blocks, max_blocks, theta, status_word, stream);
}

int32_t b2_rope_append_kv_tokens(float* q, const float* k, const float* v, const uint32_t* positions,
                                 const uint32_t* token_seq, const uint32_t* block_tables, float* k_pages,
                                 float* v_pages, uint32_t n_tokens, uint32_t q_heads, uint32_t kv_heads,
                                 uint32_t head_width, uint32_t block_size, uint64_t physical_blocks,
                                 uint32_t max_blocks, float theta, uint32_t* status_word, void* stream) {
    if (token_seq == nullptr) {
        clear_error();
        return fail(B2_STATUS_INVALID_ARGUMENT, "rotary/append pointers must not be null");
    }
    return rope_append_impl(q, k, v, positions, token_seq, block_tables, k_pages, v_pages, n_tokens, q_heads,
                            kv_heads, head_width, block_size, physical_blocks, max_blocks, theta, status_word, stream);
}

int32_t b2_silu_mul(const float* gate, const float* up, float* out, uint64_t n, void* stream) {
    return b2_silu_mul_bf16(gate, up, out, nullptr, n, stream);
}

int32_t b2_silu_mul_bf16(const float* gate, const float* up, float* out, void* out_bf16, uint64_t n,
                         void* stream) {
    clear_error();
    int32_t status = B2_STATUS_OK;
    DeviceContext* ctx = device_context(&status);
    if (ctx == nullptr) return status;
    if (gate == nullptr || up == nullptr || out == nullptr || n == 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "silu_mul needs non-null pointers and a positive size");
    }
    if ((reinterpret_cast<uintptr_t>(out_bf16) & 1u) != 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "the bf16 copy must be 2-byte aligned");
    }
    return launch_silu_mul(*ctx, gate, up, out, out_bf16, n, static_cast<cudaStream_t>(stream));
}

int32_t b2_add(const float* a, const float* b, float* out, uint64_t n, void* stream) {
    clear_error();
    int32_t status = B2_STATUS_OK;
    DeviceContext* ctx = device_context(&status);
    if (ctx == nullptr) return status;
    if (a == nullptr || b == nullptr || out == nullptr || n == 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "add needs non-null pointers and a positive size");
    }
    return launch_add(*ctx, a, b, out, n, static_cast<cudaStream_t>(stream));
}

int32_t b2_gather_rows(const float* table, const uint32_t* ids, float* out, uint32_t rows, uint32_t width,
                       uint32_t vocab, uint32_t* status_word, void* stream) {
    clear_error();
    int32_t status = B2_STATUS_OK;
    if (device_context(&status) == nullptr) return status;
    if (table == nullptr || ids == nullptr || out == nullptr || rows == 0 || width == 0 || vocab == 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "gather_rows needs non-null pointers and positive sizes");
    }
    return launch_gather_rows(table, ids, out, rows, width, vocab, status_word,
                              static_cast<cudaStream_t>(stream));
}

int32_t b2_argmax(const float* logits, uint32_t* out, uint32_t rows, uint32_t width, void* stream) {
    clear_error();
    int32_t status = B2_STATUS_OK;
    if (device_context(&status) == nullptr) return status;
    if (logits == nullptr || out == nullptr || rows == 0 || width == 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "argmax needs non-null pointers and positive sizes");
    }
    return launch_argmax(logits, out, rows, width, static_cast<cudaStream_t>(stream));
}

int32_t b2_peer_all_gather_columns(const float* local, uint64_t rows, uint64_t cols, const uint64_t* peer_full,
                                   const uint64_t* peer_flags, uint32_t rank, uint32_t world, uint32_t* state,
                                   uint32_t* status_word, void* stream) {
    return b2_peer_all_gather_columns_bf16(local, rows, cols, peer_full, nullptr, peer_flags, rank, world, state,
                                           status_word, stream);
}

int32_t b2_peer_all_gather_columns_bf16(const float* local, uint64_t rows, uint64_t cols, const uint64_t* peer_full,
                                        const uint64_t* peer_full_bf16, const uint64_t* peer_flags, uint32_t rank,
                                        uint32_t world, uint32_t* state, uint32_t* status_word, void* stream) {
    clear_error();
    int32_t status = B2_STATUS_OK;
    DeviceContext* ctx = device_context(&status);
    if (ctx == nullptr) return status;
    if (local == nullptr || peer_full == nullptr || peer_flags == nullptr || state == nullptr ||
        status_word == nullptr) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "peer all-gather needs non-null pointers");
    }
    if (rows == 0 || cols == 0 || cols % 4 != 0 || world == 0 || world > 64 || rank >= world) {
        return fail(B2_STATUS_INVALID_ARGUMENT,
                    "peer all-gather needs positive sizes, cols a multiple of 4 and rank < world <= 64");
    }
    if ((reinterpret_cast<uintptr_t>(local) & 15u) != 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "peer all-gather shard must be 16-byte aligned");
    }
    if (rows * cols * world > 0xFFFFFFFFull || rows > 0xFFFFFFFFull || cols > 0xFFFFFFFFull) {
        return fail(B2_STATUS_OVERFLOW, "peer all-gather activation too large");
    }
    return launch_peer_gather(*ctx, local, rows, cols, peer_full, peer_full_bf16, peer_flags, rank, world, state,
                              status_word, static_cast<cudaStream_t>(stream));
}

// ---- host-buffer seam ---------------------------------------------------------

int32_t b2_attention_status_result(uint32_t bits) {
    clear_error();
    if (bits & B2_ATTN_STATUS_BAD_BLOCK) {
        return fail(B2_STATUS_OUT_OF_RANGE, "paged decode attention block table contains an invalid block");
    }
    if (bits & B2_ATTN_STATUS_NAN_OR_POS_INF) {
        return fail(B2_STATUS_DOMAIN_ERROR, "softmax rejects NaN and positive infinity");
    }
    if (bits & B2_ATTN_STATUS_ALL_NEG_INF) {
        return fail(B2_STATUS_DOMAIN_ERROR, "softmax requires one finite value per slice");
    }
    if (bits != 0) {
        // B2_ATTN_STATUS_TIMEOUT, or a bit this version does not know: either way the context is not valid
        return fail(B2_STATUS_RUNTIME_ERROR,
                    "paged decode attention did not complete (status 0x%x: a bounded wait for a page copy gave up); "
                    "its output is invalid", bits);
    }
    return B2_STATUS_OK;
}

int32_t b2_check_device_errors(void) {
    int32_t status = B2_STATUS_OK;
    DeviceContext* ctx = device_context(&status);
    if (ctx == nullptr) return status;
    uint32_t word = 0;
    B2_CUDA_TRY(cudaMemcpy(&word, ctx->gemm_error, sizeof(word), cudaMemcpyDeviceToHost));
    if (word != 0) {
        B2_CUDA_TRY(cudaMemset(ctx->gemm_error, 0, sizeof(word)));
        return fail(B2_STATUS_RUNTIME_ERROR,
                    "a device-side check of an earlier NF4 kernel failed (flags 0x%x: 1 GEMM barrier timeout, 2 decode kernel "
                    "shared-memory layout, 4 decode kernel barrier timeout); that call's output is invalid",
                    word);
    }
    return B2_STATUS_OK;
}

static int32_t host_linear(const b2_nf4_weight* weight, const float* src_host, float* dst_host,
                           uint64_t rows, bool backward, cudaStream_t stream) {
    int32_t status = B2_STATUS_OK;
    DeviceContext* ctx = device_context(&status);
    if (ctx == nullptr) return status;
    WeightView w;
    B2_TRY(make_weight_view(weight, &w));
    B2_TRY(check_linear_dims(w, rows));
    // one staging buffer per device: held from the first copy to the final synchronise
    std::lock_guard<std::mutex> host_lock(g_host_mutex[ctx->device]);
    if (src_host == nullptr || dst_host == nullptr) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "quantized linear host buffers must not be null");
    }
    if (src_host == dst_host) {
        return fail(B2_STATUS_INVALID_ARGUMENT, backward
                        ? "quantized linear upstream and input gradient must not alias"
                        : "quantized linear input and output must not alias");
    }
    const uint64_t src_width = backward ? w.out_features : w.in_features;
    const uint64_t dst_width = backward ? w.in_features : w.out_features;
    const size_t src_bytes = rows * src_width * sizeof(float);
    const size_t dst_bytes = rows * dst_width * sizeof(float);
    const size_t src_padded = (src_bytes + 255) & ~size_t{255};
    B2_TRY(reserve_stage(ctx, src_padded + dst_bytes, 0));
    float* d_src = static_cast<float*>(ctx->stage);
    float* d_dst = reinterpret_cast<float*>(static_cast<uint8_t*>(ctx->stage) + src_padded);
    B2_CUDA_TRY(cudaMemcpyAsync(d_src, src_host, src_bytes, cudaMemcpyHostToDevice, stream));
    if (backward) {
        B2_TRY(linear_backward_impl(weight, d_src, d_dst, rows, nullptr, 0, stream));
    } else {
        B2_TRY(linear_forward_impl(weight, d_src, d_dst, rows, nullptr, 0, stream));
    }
    B2_CUDA_TRY(cudaMemcpyAsync(dst_host, d_dst, dst_bytes, cudaMemcpyDeviceToHost, stream));
    B2_CUDA_TRY(cudaStreamSynchronize(stream));
    return b2_check_device_errors();
}

int32_t b2_host_nf4_linear_forward(const b2_nf4_weight* weight, const float* x_host, float* y_host,
                                   uint64_t rows, void* stream) {
    clear_error();
    return host_linear(weight, x_host, y_host, rows, false, static_cast<cudaStream_t>(stream));
}

int32_t b2_host_nf4_linear_input_backward(const b2_nf4_weight* weight, const float* dy_host,
                                          float* dx_host, uint64_t rows, void* stream) {
    clear_error();
    return host_linear(weight, dy_host, dx_host, rows, true, static_cast<cudaStream_t>(stream));
}

int32_t b2_host_paged_decode_attention(const float* q_host, const float* k_pages, const float* v_pages,
                                       const uint32_t* block_tables_host,
                                       const uint32_t* seq_lens_host, float* ctx_host, uint32_t n_seq,
                                       uint32_t q_heads, uint32_t kv_heads, uint32_t head_width,
                                       uint32_t block_size, uint64_t physical_blocks,
                                       uint32_t max_blocks, void* stream_ptr) {
    clear_error();
    cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
    int32_t status = B2_STATUS_OK;
    DeviceContext* ctx = device_context(&status);
    if (ctx == nullptr) return status;
    if (q_host == nullptr || k_pages == nullptr || v_pages == nullptr || block_tables_host == nullptr ||
        seq_lens_host == nullptr || ctx_host == nullptr) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "paged decode attention pointers must not be null");
    }
    if (n_seq == 0 || block_size == 0) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "paged decode attention dimensions must be positive");
    }
    if (q_host == ctx_host) {
        return fail(B2_STATUS_INVALID_ARGUMENT, "paged decode attention output must not alias an input");
    }
    uint32_t max_seq_len = 0;
    for (uint32_t s = 0; s < n_seq; ++s) {
        if (seq_lens_host[s] == 0) {
            return fail(B2_STATUS_INVALID_ARGUMENT, "paged decode attention dimensions must be positive");
        }
        if (seq_lens_host[s] > max_seq_len) max_seq_len = seq_lens_host[s];
    }
    B2_TRY(check_paged_dims(n_seq, q_heads, kv_heads, head_width, block_size, physical_blocks,
                            max_blocks, max_seq_len));
    for (uint32_t s = 0; s < n_seq; ++s) {
        const uint32_t blocks = (seq_lens_host[s] - 1) / block_size + 1;
        for (uint32_t b = 0; b < blocks; ++b) {
            if (block_tables_host[static_cast<uint64_t>(s) * max_blocks + b] >= physical_blocks) {
                return fail(B2_STATUS_OUT_OF_RANGE,
                            "paged decode attention block table contains an invalid block");
            }
        }
    }
    std::lock_guard<std::mutex> host_lock(g_host_mutex[ctx->device]);
    const size_t q_bytes = static_cast<size_t>(n_seq) * q_heads * head_width * sizeof(float);
    const size_t table_bytes = static_cast<size_t>(n_seq) * max_blocks * sizeof(uint32_t);
    const size_t len_bytes = static_cast<size_t>(n_seq) * sizeof(uint32_t);
    auto pad = [](size_t v) { return (v + 255) & ~size_t{255}; };
    const size_t off_ctx = pad(q_bytes), off_table = off_ctx + pad(q_bytes),
                 off_len = off_table + pad(table_bytes), off_status = off_len + pad(len_bytes),
                 off_ws = off_status + 256;
    const size_t ws_bytes =
        paged_decode_workspace_bytes(n_seq, q_heads, head_width, block_size, max_seq_len);
    B2_TRY(reserve_stage(ctx, off_ws + ws_bytes, 0));
    uint8_t* base = static_cast<uint8_t*>(ctx->stage);
    float* d_q = reinterpret_cast<float*>(base);
    float* d_ctx = reinterpret_cast<float*>(base + off_ctx);
    uint32_t* d_table = reinterpret_cast<uint32_t*>(base + off_table);
    uint32_t* d_len = reinterpret_cast<uint32_t*>(base + off_len);
    uint32_t* d_status = reinterpret_cast<uint32_t*>(base + off_status);
    B2_CUDA_TRY(cudaMemcpyAsync(d_q, q_host, q_bytes, cudaMemcpyHostToDevice, stream));
    B2_CUDA_TRY(cudaMemcpyAsync(d_table, block_tables_host, table_bytes, cudaMemcpyHostToDevice, stream));
    B2_CUDA_TRY(cudaMemcpyAsync(d_len, seq_lens_host, len_bytes, cudaMemcpyHostToDevice, stream));
    B2_CUDA_TRY(cudaMemsetAsync(d_status, 0, sizeof(uint32_t), stream));
    PagedDecodeArgs args{d_q, k_pages, v_pages, d_table, d_len, d_ctx,
                         n_seq, q_heads, kv_heads, head_width, block_size, max_blocks, max_seq_len,
                         physical_blocks, d_status};
    B2_TRY(launch_paged_decode(*ctx, args, base + off_ws, ws_bytes, stream));
    uint32_t host_status = 0;
    B2_CUDA_TRY(cudaMemcpyAsync(ctx_host, d_ctx, q_bytes, cudaMemcpyDeviceToHost, stream));
    B2_CUDA_TRY(cudaMemcpyAsync(&host_status, d_status, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream));
    B2_CUDA_TRY(cudaStreamSynchronize(stream));
    return b2_attention_status_result(host_status);
}

}  // extern "C"
