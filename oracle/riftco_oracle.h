/*
 * CPU oracle for the packed-NF4 linear operator and paged-KV decode attention.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing under this directory is part of the
 * product: the CUDA library never links, loads or calls it. It exists so the
 * GPU results can be checked against a plain restatement of the reference
 * algorithm, and so a CPU baseline can be timed beside the GPU numbers.
 *
 * Every function restates, in plain C, one function of
 * quangng2000/riftco-transformer; the citation beside each declaration is the
 * file:line inside that project that it follows. Parity of this restatement is
 * pinned two ways: against the golden vectors the reference's own tests hold
 * (tests/core/test_quantization.cpp, tests/core/backend/
 * test_quantized_linear_backend.cpp, tests/core/backend/test_nn_backend.cpp)
 * and against the reference's own sources compiled in place (ref_bridge.cpp).
 *
 * Build with -ffp-contract=off: the reference's bits depend on the multiply
 * and the add of every accumulation step being rounded separately.
 */
#ifndef RIFTCO_ORACLE_H
#define RIFTCO_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Scale encodings: src/core/backend/nn/quantized_linear/storage.hpp:13-16. */
#define ORC_SCALES_FLOAT32 0u
#define ORC_SCALES_DOUBLE_QUANTIZED_UINT8 1u

/* One packed weight, flat row-major [out_features, in_features]; mirrors
 * Nf4ScaleStorageView (storage.hpp:31-46) plus the packed-code span. */
typedef struct orc_nf4_weight {
    const uint8_t* codes;          /* ceil(out*in/2) bytes, even index = low nibble */
    const float* fp32_scales;      /* [blocks] when encoding == FLOAT32, else NULL   */
    const uint8_t* scale_codes;    /* [blocks] when DOUBLE_QUANTIZED, else NULL      */
    const float* second_level;     /* [ceil(blocks/scale_block_size)] or NULL        */
    uint64_t scale_block_size;     /* 0 for FLOAT32                                  */
    float offset;                  /* shared mean of the first-level scales          */
    uint32_t encoding;
    uint64_t block_size;
    uint64_t out_features;
    uint64_t in_features;
} orc_nf4_weight;

/* src/core/quantization/nf4.cpp:14-31 (same literals in
 * src/core/backend/nn/quantized_linear/reference/operations.cpp:13-30). */
const float* orc_nf4_codebook(void);

/* src/core/quantization/nf4.cpp:55-68: strict '<' keeps the lower index on ties. */
uint8_t orc_nearest_nf4_code(float normalized_value);

/* src/core/quantization/quantized_weight.cpp:176-207 (pack_nf4): per-block
 * absmax scale, zero block -> scale 0 and code 7, low nibble first. codes must
 * hold ceil(n/2) bytes, scales ceil(n/block_size) floats. Returns 0, or 1 when
 * a source value is not finite. */
int orc_pack_nf4(const float* values, size_t n, size_t block_size,
                 uint8_t* codes, float* scales);

/* src/core/quantization/quantized_weight.cpp:209-254 (double_quantize_scales).
 * scale_codes holds n_scales bytes, second_level ceil(n_scales/scale_block). */
int orc_double_quantize_scales(const float* scales, size_t n_scales,
                               size_t scale_block_size, uint8_t* scale_codes,
                               float* second_level, float* offset);

/* src/core/backend/nn/quantized_linear/storage.hpp:48-65. */
float orc_decode_block_scale(const orc_nf4_weight* w, size_t scale_index);

/* QuantizedWeight::dequantize, src/core/quantization/quantized_weight.cpp
 * (values[i] = codebook[code(i)] * decoded_scale(i / block)); the bit-exact
 * reference for dequantised weights. out holds out*in floats. */
void orc_nf4_dequantize(const orc_nf4_weight* w, float* out);

/* src/core/backend/nn/quantized_linear/reference/operations.cpp:49-81.
 * y[r,o] = sum_i x[r,i] * (cb[code] * scale), accumulated in FP32 in i order.
 * threads <= 1 runs the loop as shipped (one thread); threads > 1 splits the
 * (row, output) pairs over OpenMP threads, which leaves every output's own
 * summation order, and so its bits, unchanged. */
void orc_nf4_linear_forward(const orc_nf4_weight* w, const float* x, float* y,
                            size_t rows, int threads);

/* src/core/backend/nn/quantized_linear/reference/operations.cpp:83-115.
 * dx[r,i] = sum_o dy[r,o] * deq(W[o,i]), accumulated in FP32 in o order. */
void orc_nf4_linear_input_backward(const orc_nf4_weight* w, const float* dy,
                                   float* dx, size_t rows, int threads);

/* src/core/backend/attention/reference/paged_decode.cpp:37-132: one sequence,
 * `heads` heads, pages [physical_block, head, block_offset, head_width].
 * Returns 0, 1 for a NaN or +inf score, 2 when every score of a head is -inf
 * (the two std::domain_error cases). */
int orc_paged_decode(const float* queries, const float* key_pages,
                     const float* value_pages, const uint32_t* block_table,
                     float* context, size_t heads, size_t head_width,
                     size_t block_size, size_t sequence_length);

/* Batched grouped-query form of the same loop: query head h of sequence s reads
 * KV head h / (q_heads / kv_heads) (contiguous repetition, as in
 * src/model/grouped_query_attention.cpp:61-94). It is the loop above run once
 * per (sequence, query head) with the page tensor's head count = kv_heads, so
 * each output equals the unmodified single-sequence function called with the
 * matching head subset. block_tables is [n_seq, max_blocks]. */
int orc_paged_decode_gqa(const float* queries, const float* key_pages,
                         const float* value_pages, const uint32_t* block_tables,
                         const uint32_t* seq_lens, float* context, size_t n_seq,
                         size_t q_heads, size_t kv_heads, size_t head_width,
                         size_t block_size, size_t max_blocks, int threads);

/* Decode-step primitives (rms_norm, SiLU / SwiGLU hidden state, greedy choice); see the .c file
 * for the reference lines each one follows. `up` may be NULL. */
void orc_rms_norm(const float* x, const float* scale, size_t rows, size_t width,
                  float epsilon, float* out);
void orc_silu_mul(const float* gate, const float* up, size_t n, float* out);
size_t orc_greedy(const float* logits, size_t n);

/* ((x * A^T) * B^T) * scale, the LoRA branch of a Linear; `reduced` is scratch [rows, rank]. */
void orc_lora_forward(const float* x, const float* a, const float* b, size_t rows,
                      size_t in_features, size_t out_features, size_t rank, float scale,
                      float* reduced, float* out);

#ifdef __cplusplus
}
#endif
#endif
