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

// ---- decode-step primitives and the packed model state -------------------------------------
//
// The operators either side of the hot path in one decode step, called through the reference's
// own public C++ entry points, so the CUDA glue kernels and the numpy restatement in
// oracle/decode_ref.py can be held to the reference's results:
//   rms_norm                          (src/nn/rms_norm.cpp:39-73)
//   apply_rotary_position_embedding   (src/model/rotary_embedding.cpp:64-117, 142-193)
//   silu and silu(gate) * up          (src/nn/activations.cpp:38-58, src/model/swiglu.cpp:27-29)
//   GreedySampler::sample             (src/stages/serving/generation.cpp:100-110)
//   PagedKvCachePool / DecoderKeyValueCache::append_and_attend
//                                     (src/stages/serving/cache/page_table_cache.cpp:44-77,165-233)
// and the canonical RTNF4S1 stream of a quantised DecoderOnlyTransformer
//   packed_model_state_bytes          (src/c_api/model_state.cpp:27-113).
#include "c_api/internal/model_state.hpp"
#include "riftco_transformer/model/decoder_only_transformer.hpp"
#include "riftco_transformer/model/rotary_embedding.hpp"
#include "riftco_transformer/nn/activations.hpp"
#include "riftco_transformer/nn/rms_norm.hpp"
#include "riftco_transformer/stages/serving/generation.hpp"
#include "riftco_transformer/stages/serving/kv_cache.hpp"

#include <random>

namespace {

using riftco_transformer::Variable;

void copy_out(const Tensor& t, float* out) {
    const auto values = t.data();
    std::copy(values.begin(), values.end(), out);
}

void put_u64(std::vector<std::uint8_t>& out, std::uint64_t v) {
    for (int s = 0; s < 64; s += 8) out.push_back(static_cast<std::uint8_t>(v >> s));
}

}  // namespace

extern "C" {

int ref_rms_norm(const float* x, const float* scale, std::uint64_t rows, std::uint64_t width,
                 float epsilon, float* out) {
    return guarded([&] {
        CpuScope cpu;
        const Variable input(Tensor({rows, width}, std::vector<float>(x, x + rows * width), g_backend), false);
        const Variable gain(Tensor({width}, std::vector<float>(scale, scale + width), g_backend), false);
        copy_out(riftco_transformer::rms_norm(input, gain, epsilon).value(), out);
    });
}

// x, out: [batch, heads, time, width]; token t of the time axis sits at position offset + t.
int ref_rope(const float* x, std::uint64_t batch, std::uint64_t heads, std::uint64_t time,
             std::uint64_t width, std::uint64_t position_offset, float theta, float* out) {
    return guarded([&] {
        CpuScope cpu;
        const std::size_t n = batch * heads * time * width;
        const Variable input(Tensor({batch, heads, time, width}, std::vector<float>(x, x + n), g_backend), false);
        copy_out(riftco_transformer::apply_rotary_position_embedding(input, position_offset, theta).value(), out);
    });
}

// out = silu(gate) (up == nullptr) or silu(gate) * up.
int ref_silu_mul(const float* gate, const float* up, std::uint64_t n, float* out) {
    return guarded([&] {
        CpuScope cpu;
        const Variable g(Tensor({n}, std::vector<float>(gate, gate + n), g_backend), false);
        Variable result = riftco_transformer::silu(g);
        if (up != nullptr) {
            const Variable u(Tensor({n}, std::vector<float>(up, up + n), g_backend), false);
            result = result * u;
        }
        copy_out(result.value(), out);
    });
}

int ref_greedy(const float* logits, std::uint64_t n, std::uint32_t* token) {
    return guarded([&] {
        riftco_transformer::stages::serving::GreedySampler sampler;
        *token = static_cast<std::uint32_t>(sampler.sample(std::span<const float>(logits, n)));
    });
}

// Feeds `steps` tokens of one sequence through a paged KV cache of the reference (one layer):
// q, k, v: [steps, heads, width] (k already rotated by the caller); ctx: [steps, heads, width] gets
// the attention context after each append. block_count pages of block_size slots.
int ref_paged_cache_decode(const float* q, const float* k, const float* v, std::uint64_t steps,
                           std::uint64_t heads, std::uint64_t width, std::uint64_t block_size,
                           std::uint64_t block_count, float* ctx) {
    return guarded([&] {
        CpuScope cpu;
        riftco_transformer::TransformerDimensions dims;
        dims.vocabulary_size = 8;
        dims.maximum_context = block_size * block_count;
        dims.model_width = heads * width;
        dims.head_count = heads;
        dims.block_count = 1;
        dims.feed_forward_width = 4 * heads * width;
        riftco_transformer::stages::serving::PagedKvCachePool pool(dims, ExecutionBackend::Cpu, block_size, block_count);
        auto cache = pool.create();
        const std::size_t n = heads * width;
        for (std::uint64_t t = 0; t < steps; ++t) {
            const Tensor tq({1, heads, 1, width}, std::vector<float>(q + t * n, q + (t + 1) * n), ExecutionBackend::Cpu);
            const Tensor tk({1, heads, 1, width}, std::vector<float>(k + t * n, k + (t + 1) * n), ExecutionBackend::Cpu);
            const Tensor tv({1, heads, 1, width}, std::vector<float>(v + t * n, v + (t + 1) * n), ExecutionBackend::Cpu);
            cache->begin_token();
            const Tensor context = cache->append_and_attend(0, tq, tk, tv);
            cache->commit_token();
            copy_out(context, ctx + t * n);
        }
    });
}

// Builds a small DecoderOnlyTransformer (seeded), quantises every Linear base weight to NF4
// (scale_block_size == 0: FP32 scales, else double-quantised) and writes
//   stream: packed_model_state_bytes(model), the canonical RTNF4S1 stream
//   dump:   the same weights field by field straight from packed_linear_weight_state(), as
//           u64 count, then per weight u64 {out, in, block, n_codes, n_fp32, n_scale_codes, n_second,
//           scale_block}, f32 offset, u32 pad, codes, f32 scales, scale codes, f32 second level
// (*_size receive the byte counts; a too-small capacity only reports the size).
int ref_packed_model_fixture(std::uint64_t vocabulary, std::uint64_t context, std::uint64_t width,
                             std::uint64_t heads, std::uint64_t blocks, std::uint64_t feed_forward,
                             std::uint64_t block_size, std::uint64_t scale_block_size, std::uint32_t seed,
                             std::uint8_t* stream, std::uint64_t stream_capacity, std::uint64_t* stream_size,
                             std::uint8_t* dump, std::uint64_t dump_capacity, std::uint64_t* dump_size) {
    return guarded([&] {
        CpuScope cpu;
        riftco_transformer::TransformerDimensions dims;
        dims.vocabulary_size = vocabulary;
        dims.maximum_context = context;
        dims.model_width = width;
        dims.head_count = heads;
        dims.block_count = blocks;
        dims.feed_forward_width = feed_forward;
        std::mt19937 random(seed);
        riftco_transformer::DecoderOnlyTransformer model(dims, random);
        if (scale_block_size == 0) {
            model.quantize_linear_weights_nf4(block_size);
        } else {
            model.quantize_linear_weights_nf4_double_quantized(block_size, scale_block_size);
        }
        const std::vector<std::uint8_t> bytes = riftco_transformer::c_api::detail::packed_model_state_bytes(model);
        *stream_size = bytes.size();
        if (stream != nullptr && stream_capacity >= bytes.size()) std::copy(bytes.begin(), bytes.end(), stream);
        std::vector<std::uint8_t> raw;
        const auto weights = model.packed_linear_weight_state();
        put_u64(raw, weights.size());
        for (const auto& w : weights) {
            const auto& p = w.payload;
            const bool dq = p.double_quantized_scales.has_value();
            put_u64(raw, w.shape.at(0));
            put_u64(raw, w.shape.at(1));
            put_u64(raw, w.block_size);
            put_u64(raw, p.packed_codes.size());
            put_u64(raw, p.block_scales.size());
            put_u64(raw, dq ? p.double_quantized_scales->scale_codes.size() : 0);
            put_u64(raw, dq ? p.double_quantized_scales->second_level_scales.size() : 0);
            put_u64(raw, dq ? p.double_quantized_scales->scale_block_size : 0);
            const float offset = dq ? p.double_quantized_scales->offset : 0.0F;
            std::uint32_t bits;
            std::memcpy(&bits, &offset, 4);
            put_u64(raw, bits);   // offset bits in the low half, zero padding above
            raw.insert(raw.end(), p.packed_codes.begin(), p.packed_codes.end());
            const auto* f = reinterpret_cast<const std::uint8_t*>(p.block_scales.data());
            raw.insert(raw.end(), f, f + 4 * p.block_scales.size());
            if (dq) {
                const auto& n = *p.double_quantized_scales;
                raw.insert(raw.end(), n.scale_codes.begin(), n.scale_codes.end());
                const auto* s = reinterpret_cast<const std::uint8_t*>(n.second_level_scales.data());
                raw.insert(raw.end(), s, s + 4 * n.second_level_scales.size());
            }
        }
        *dump_size = raw.size();
        if (dump != nullptr && dump_capacity >= raw.size()) std::copy(raw.begin(), raw.end(), dump);
    });
}

// The LoRA branch with the reference's own operators, in the order of LowRankAdapter::forward
// (src/nn/low_rank_adapter.cpp:132-158): matmul(matmul(x, A^T), B^T) * scale. x [rows, in],
// a [rank, in], b [out, rank] -> out [rows, out].
int ref_lora_forward(const float* x, const float* a, const float* b, std::uint64_t rows,
                     std::uint64_t in_features, std::uint64_t out_features, std::uint64_t rank, float scale,
                     float* out) {
    return guarded([&] {
        CpuScope cpu;
        using riftco_transformer::matmul;
        using riftco_transformer::transpose_2d;
        const Variable input(Tensor({rows, in_features}, std::vector<float>(x, x + rows * in_features), g_backend), false);
        const Variable lora_a(Tensor({rank, in_features}, std::vector<float>(a, a + rank * in_features), g_backend), false);
        const Variable lora_b(Tensor({out_features, rank}, std::vector<float>(b, b + out_features * rank), g_backend), false);
        const Variable reduced = matmul(input, transpose_2d(lora_a));
        const Variable expanded = matmul(reduced, transpose_2d(lora_b));
        copy_out((expanded * scale).value(), out);
    });
}

}  // extern "C"
