// Bridge that exposes the UNMODIFIED reference CPU implementation through a
// small C interface, so Python tests and the CPU-baseline leg of the benchmark
// can call the reference's own code. TEST INFRASTRUCTURE ONLY: the product
// library never links or loads this.
//
// It is compiled together with the reference's core sources where they lie in
// a checkout of quangng2000/riftco-transformer (see oracle/build.py); only the
// resulting shared library is kept, under oracle/_ref/. The calls below go
// through the reference's public/private C++ entry points:
//   QuantizedWeight::quantize_nf4 / quantize_nf4_double_quantized /
//   from_packed_nf4 / dequantize   (src/core/quantization/quantized_weight.cpp)
//   dispatch_quantized_linear_forward / _input_backward
//                                  (src/core/backend/nn/quantized_linear/dispatch.cpp:317-370)
//   dispatch_paged_decode_attention_forward
//                                  (src/core/backend/attention/dispatch.cpp:440-509)
//   dispatch_materialized_causal_attention_forward (used by the reference's own
//   paged-decode test as its expected value, tests/core/backend/test_nn_backend.cpp:2079-2216)
// on ExecutionBackend::Cpu unless ref_set_backend() selected another one (the
// library variant linked with riftco_transformer_b200/adapter/cuda_b200_adapter.cpp
// uses it to drive the reference's dispatch layer on ExecutionBackend::Cuda).
#include "core/backend/attention/dispatch.hpp"
#include "core/backend/nn/quantized_linear/dispatch.hpp"
#include "core/quantization/nf4.hpp"
#include "riftco_transformer/core/backend.hpp"
#include "riftco_transformer/core/quantized_weight.hpp"
#include "riftco_transformer/core/tensor.hpp"

#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <new>
#include <stdexcept>
#include <string>
#include <vector>

namespace {

using riftco_transformer::ExecutionBackend;
using riftco_transformer::Nf4DoubleQuantizedScales;
using riftco_transformer::Nf4Payload;
using riftco_transformer::QuantizedWeight;
using riftco_transformer::Tensor;
namespace backend = riftco_transformer::backend_detail;

thread_local std::string g_error;
ExecutionBackend g_backend = ExecutionBackend::Cpu;

// Quantisation and dequantisation are host algorithms: they always run on the CPU backend.
struct CpuScope {
    ExecutionBackend saved = g_backend;
    CpuScope() { g_backend = ExecutionBackend::Cpu; }
    ~CpuScope() { g_backend = saved; }
};

// Same numeric codes as rt_status (include/riftco_transformer/c_api.h:41-49)
// with the mapping of src/c_api/internal/error.hpp; domain_error gets its own
// code so the tests can tell the non-finite-score rejection apart.
template <typename F> int guarded(F&& f) {
    try {
        f();
        g_error.clear();
        return 0;
    } catch (const std::domain_error& e) {
        g_error = e.what();
        return 7;
    } catch (const std::invalid_argument& e) {
        g_error = e.what();
        return 1;
    } catch (const std::out_of_range& e) {
        g_error = e.what();
        return 2;
    } catch (const std::overflow_error& e) {
        g_error = e.what();
        return 3;
    } catch (const std::bad_alloc& e) {
        g_error = e.what();
        return 5;
    } catch (const std::exception& e) {
        g_error = e.what();
        return 6;
    }
}

// Adds the lifetime of the object, i.e. the operator call alone without the
// copies into and out of reference tensors, to *seconds when it is non-null.
class Stopwatch {
public:
    explicit Stopwatch(double* sink)
        : sink_(sink), start_(std::chrono::steady_clock::now()) {}
    ~Stopwatch() {
        if (sink_ != nullptr) {
            *sink_ += std::chrono::duration<double>(
                          std::chrono::steady_clock::now() - start_)
                          .count();
        }
    }
    Stopwatch(const Stopwatch&) = delete;
    Stopwatch& operator=(const Stopwatch&) = delete;

private:
    double* sink_;
    std::chrono::steady_clock::time_point start_;
};

Tensor tensor_from(const float* p, std::size_t rows, std::size_t cols) {
    return Tensor({rows, cols}, std::vector<float>(p, p + rows * cols),
                  g_backend);
}

QuantizedWeight weight_from(const std::uint8_t* codes, const float* fp32_scales,
                            const std::uint8_t* scale_codes, const float* second,
                            std::uint64_t scale_block, float offset,
                            std::uint32_t encoding, std::uint64_t block,
                            std::uint64_t out, std::uint64_t in) {
    const std::size_t n = out * in;
    const std::size_t blocks = (n + block - 1) / block;
    Nf4Payload payload;
    payload.packed_codes.assign(codes, codes + (n + 1) / 2);
    if (encoding == 0) {
        payload.block_scales.assign(fp32_scales, fp32_scales + blocks);
    } else {
        Nf4DoubleQuantizedScales nested;
        nested.scale_codes.assign(scale_codes, scale_codes + blocks);
        nested.second_level_scales.assign(
            second, second + (blocks + scale_block - 1) / scale_block);
        nested.scale_block_size = scale_block;
        nested.offset = offset;
        payload.double_quantized_scales = std::move(nested);
    }
    return QuantizedWeight::from_packed_nf4({out, in}, block, std::move(payload),
                                            g_backend);
}

}  // namespace

extern "C" {

const char* ref_last_error() { return g_error.c_str(); }

// 0 = Cpu (default), 2 = Cuda; returns 1 when the backend is not available in this build.
int ref_set_backend(int backend) {
    const ExecutionBackend b = static_cast<ExecutionBackend>(backend);
    if (!riftco_transformer::execution_backend_available(b)) return 1;
    g_backend = b;
    return 0;
}

void ref_codebook(float* out16) {
    const auto cb = riftco_transformer::quantization::nf4_codebook();
    std::copy(cb.begin(), cb.end(), out16);
}

std::uint8_t ref_nearest_nf4_code(float v) {
    return riftco_transformer::quantization::detail::nearest_nf4_code(v);
}

// FP32-scale quantisation of a [out, in] matrix; codes: ceil(n/2) bytes,
// scales: ceil(n/block) floats.
int ref_quantize_nf4(const float* values, std::uint64_t out, std::uint64_t in,
                     std::uint64_t block, std::uint8_t* codes, float* scales) {
    const CpuScope cpu_only;
    return guarded([&] {
        const auto payload =
            QuantizedWeight::quantize_nf4(tensor_from(values, out, in), block)
                .copy_payload_to_host();
        std::copy(payload.packed_codes.begin(), payload.packed_codes.end(), codes);
        std::copy(payload.block_scales.begin(), payload.block_scales.end(), scales);
    });
}

int ref_quantize_nf4_double_quantized(const float* values, std::uint64_t out,
                                      std::uint64_t in, std::uint64_t block,
                                      std::uint64_t scale_block,
                                      std::uint8_t* codes,
                                      std::uint8_t* scale_codes, float* second,
                                      float* offset) {
    const CpuScope cpu_only;
    return guarded([&] {
        const auto payload = QuantizedWeight::quantize_nf4_double_quantized(
                                 tensor_from(values, out, in), block, scale_block)
                                 .copy_payload_to_host();
        const auto& nested = payload.double_quantized_scales.value();
        std::copy(payload.packed_codes.begin(), payload.packed_codes.end(), codes);
        std::copy(nested.scale_codes.begin(), nested.scale_codes.end(), scale_codes);
        std::copy(nested.second_level_scales.begin(),
                  nested.second_level_scales.end(), second);
        *offset = nested.offset;
    });
}

int ref_dequantize(const std::uint8_t* codes, const float* fp32_scales,
                   const std::uint8_t* scale_codes, const float* second,
                   std::uint64_t scale_block, float offset, std::uint32_t encoding,
                   std::uint64_t block, std::uint64_t out, std::uint64_t in,
                   float* values) {
    const CpuScope cpu_only;
    return guarded([&] {
        const Tensor dense = weight_from(codes, fp32_scales, scale_codes, second,
                                         scale_block, offset, encoding, block,
                                         out, in)
                                 .dequantize();
        const auto data = dense.data();
        std::copy(data.begin(), data.end(), values);
    });
}

int ref_linear_forward(const std::uint8_t* codes, const float* fp32_scales,
                       const std::uint8_t* scale_codes, const float* second,
                       std::uint64_t scale_block, float offset,
                       std::uint32_t encoding, std::uint64_t block,
                       std::uint64_t out, std::uint64_t in, const float* x,
                       float* y, std::uint64_t rows, double* seconds) {
    return guarded([&] {
        const QuantizedWeight w = weight_from(codes, fp32_scales, scale_codes,
                                              second, scale_block, offset,
                                              encoding, block, out, in);
        const Tensor input = tensor_from(x, rows, in);
        Tensor output({rows, out}, g_backend);
        const Stopwatch watch(seconds);
        backend::dispatch_quantized_linear_forward(
            g_backend,
            {backend::tensor_storage(input), backend::quantized_weight_storage(w),
             backend::tensor_storage(output), {rows, in, out, block}});
        const auto data = output.data();
        std::copy(data.begin(), data.end(), y);
    });
}

int ref_linear_input_backward(const std::uint8_t* codes, const float* fp32_scales,
                              const std::uint8_t* scale_codes, const float* second,
                              std::uint64_t scale_block, float offset,
                              std::uint32_t encoding, std::uint64_t block,
                              std::uint64_t out, std::uint64_t in,
                              const float* dy, float* dx, std::uint64_t rows,
                              double* seconds) {
    return guarded([&] {
        const QuantizedWeight w = weight_from(codes, fp32_scales, scale_codes,
                                              second, scale_block, offset,
                                              encoding, block, out, in);
        const Tensor upstream = tensor_from(dy, rows, out);
        Tensor gradient({rows, in}, g_backend);
        const Stopwatch watch(seconds);
        backend::dispatch_quantized_linear_input_backward(
            g_backend,
            {backend::tensor_storage(upstream),
             backend::quantized_weight_storage(w),
             backend::tensor_storage(gradient), {rows, in, out, block}});
        const auto data = gradient.data();
        std::copy(data.begin(), data.end(), dx);
    });
}

// One sequence, all heads: exactly the reference operator. Pages are
// [physical_blocks, heads, block_size, width].
int ref_paged_decode(const float* q, const float* key_pages,
                     const float* value_pages, const std::uint32_t* table,
                     std::uint64_t table_len, float* ctx, std::uint64_t heads,
                     std::uint64_t width, std::uint64_t block_size,
                     std::uint64_t physical_blocks, std::uint64_t seq_len,
                     double* seconds) {
    return guarded([&] {
        const std::size_t pool = physical_blocks * heads * block_size * width;
        const Tensor queries({heads, width},
                             std::vector<float>(q, q + heads * width),
                             g_backend);
        const Tensor keys({physical_blocks, heads, block_size, width},
                          std::vector<float>(key_pages, key_pages + pool),
                          g_backend);
        const Tensor values({physical_blocks, heads, block_size, width},
                            std::vector<float>(value_pages, value_pages + pool),
                            g_backend);
        Tensor context({heads, width}, g_backend);
        const Stopwatch watch(seconds);
        backend::dispatch_paged_decode_attention_forward(
            g_backend,
            {backend::tensor_storage(queries), backend::tensor_storage(keys),
             backend::tensor_storage(values),
             std::span<const std::uint32_t>(table, table_len),
             backend::tensor_storage(context),
             {heads, width, block_size, physical_blocks, seq_len}});
        const auto data = context.data();
        std::copy(data.begin(), data.end(), ctx);
    });
}

// Full causal attention on [batch, heads, time, width]; the reference's paged
// decode test takes the last time row of this as its expected value.
int ref_materialized_causal_forward(const float* q, const float* k, const float* v,
                                    float* probabilities, float* context,
                                    std::uint64_t batch, std::uint64_t heads,
                                    std::uint64_t time, std::uint64_t width) {
    return guarded([&] {
        const std::size_t n = batch * heads * time * width;
        const Tensor::Shape shape{batch, heads, time, width};
        const Tensor tq(shape, std::vector<float>(q, q + n), ExecutionBackend::Cpu);
        const Tensor tk(shape, std::vector<float>(k, k + n), ExecutionBackend::Cpu);
        const Tensor tv(shape, std::vector<float>(v, v + n), ExecutionBackend::Cpu);
        Tensor probs({batch, heads, time, time}, ExecutionBackend::Cpu);
        Tensor ctx(shape, ExecutionBackend::Cpu);
        backend::dispatch_materialized_causal_attention_forward(
            ExecutionBackend::Cpu,
            {backend::tensor_storage(tq), backend::tensor_storage(tk),
             backend::tensor_storage(tv), backend::tensor_storage(probs),
             backend::tensor_storage(ctx), {batch, heads, time, width}});
        if (probabilities != nullptr) {
            const auto p = probs.data();
            std::copy(p.begin(), p.end(), probabilities);
        }
        const auto c = ctx.data();
        std::copy(c.begin(), c.end(), context);
    });
}

}  // extern "C"
