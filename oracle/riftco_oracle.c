/*
 * CPU oracle (test infrastructure, never part of the product path): a plain C
 * restatement of the reference's NF4 encoder, dequantiser, packed linear loops
 * and single-query paged attention. See riftco_oracle.h for the reference
 * file:line each function follows. Build with -ffp-contract=off.
 */
#include "riftco_oracle.h"

#include <float.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

static const float kCodebook[16] = {
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

const float* orc_nf4_codebook(void) { return kCodebook; }

uint8_t orc_nearest_nf4_code(float v) {
    uint8_t best = 0;
    float best_d = fabsf(v - kCodebook[0]);
    for (uint8_t c = 1; c < 16; ++c) {
        const float d = fabsf(v - kCodebook[c]);
        if (d < best_d) {
            best_d = d;
            best = c;
        }
    }
    return best;
}

static inline uint8_t code_at(const uint8_t* codes, size_t i) {
    const uint8_t b = codes[i >> 1];
    return (i & 1u) ? (uint8_t)(b >> 4) : (uint8_t)(b & 0x0Fu);
}

int orc_pack_nf4(const float* values, size_t n, size_t block_size,
                 uint8_t* codes, float* scales) {
    const size_t n_blocks = (n + block_size - 1) / block_size;
    memset(codes, 0, (n + 1) / 2);
    for (size_t b = 0; b < n_blocks; ++b) {
        const size_t lo = b * block_size;
        const size_t hi = lo + block_size < n ? lo + block_size : n;
        float absmax = 0.0f;
        for (size_t i = lo; i < hi; ++i) {
            if (!isfinite(values[i])) return 1;
            const float a = fabsf(values[i]);
            if (a > absmax) absmax = a;
        }
        scales[b] = absmax;
        for (size_t i = lo; i < hi; ++i) {
            const uint8_t c =
                absmax == 0.0f ? (uint8_t)7
                               : orc_nearest_nf4_code(values[i] / absmax);
            codes[i >> 1] |= (uint8_t)((i & 1u) ? (c << 4) : c);
        }
    }
    return 0;
}

int orc_double_quantize_scales(const float* scales, size_t n_scales,
                               size_t scale_block_size, uint8_t* scale_codes,
                               float* second_level, float* offset) {
    const size_t n_groups = (n_scales + scale_block_size - 1) / scale_block_size;
    double sum = 0.0;
    for (size_t i = 0; i < n_scales; ++i) sum += (double)scales[i];
    const float mu = (float)(sum / (double)n_scales);
    if (!isfinite(mu)) return 1;
    *offset = mu;
    for (size_t i = 0; i < n_scales; ++i) scale_codes[i] = 128;
    for (size_t g = 0; g < n_groups; ++g) {
        const size_t lo = g * scale_block_size;
        const size_t hi =
            lo + scale_block_size < n_scales ? lo + scale_block_size : n_scales;
        float absmax = 0.0f;
        for (size_t i = lo; i < hi; ++i) {
            const float a = fabsf(scales[i] - mu);
            if (a > absmax) absmax = a;
        }
        second_level[g] = absmax;
        if (absmax == 0.0f) continue;
        for (size_t i = lo; i < hi; ++i) {
            const float normalized = (scales[i] - mu) / absmax;
            const float scaled = normalized * 127.0f;
            const float rounded =
                scaled >= 0.0f ? floorf(scaled + 0.5f) : ceilf(scaled - 0.5f);
            int centered = (int)rounded;
            if (centered < -127) centered = -127;
            if (centered > 127) centered = 127;
            scale_codes[i] = (uint8_t)(centered + 128);
        }
    }
    return 0;
}

float orc_decode_block_scale(const orc_nf4_weight* w, size_t idx) {
    if (w->encoding == ORC_SCALES_FLOAT32) return w->fp32_scales[idx];
    const int centered = (int)w->scale_codes[idx] - 128;
    const float factor = (float)centered / 127.0f;
    const float delta = w->second_level[idx / w->scale_block_size] * factor;
    if (delta > 0.0f && w->offset > FLT_MAX - delta) return FLT_MAX;
    const float s = w->offset + delta;
    return s > 0.0f ? s : 0.0f;
}

void orc_nf4_dequantize(const orc_nf4_weight* w, float* out) {
    const size_t n = (size_t)(w->out_features * w->in_features);
    const size_t bs = (size_t)w->block_size;
    for (size_t b = 0, lo = 0; lo < n; ++b, lo += bs) {
        const float s = orc_decode_block_scale(w, b);
        const size_t hi = lo + bs < n ? lo + bs : n;
        for (size_t i = lo; i < hi; ++i)
            out[i] = kCodebook[code_at(w->codes, i)] * s;
    }
}

/* Decoded scale of every block, computed once: decoding is a pure function of
 * the block index, so hoisting it out of the element loop changes no bit. */
static float* decode_all_scales(const orc_nf4_weight* w, size_t* n_blocks_out) {
    const size_t n = (size_t)(w->out_features * w->in_features);
    const size_t n_blocks = (n + w->block_size - 1) / w->block_size;
    float* s = (float*)malloc(n_blocks * sizeof(float));
    for (size_t b = 0; b < n_blocks; ++b) s[b] = orc_decode_block_scale(w, b);
    if (n_blocks_out) *n_blocks_out = n_blocks;
    return s;
}

void orc_nf4_linear_forward(const orc_nf4_weight* w, const float* x, float* y,
                            size_t rows, int threads) {
    const size_t in = (size_t)w->in_features, out = (size_t)w->out_features;
    const size_t bs = (size_t)w->block_size;
    float* scales = decode_all_scales(w, NULL);
    const long long total = (long long)(rows * out);
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(threads > 1 ? threads : 1)
#else
    (void)threads;
#endif
    for (long long t = 0; t < total; ++t) {
        /* output-major order so a thread reuses one weight row across rows */
        const size_t o = (size_t)t / rows, r = (size_t)t % rows;
        const float* xr = x + r * in;
        const size_t base = o * in;
        float acc = 0.0f;
        for (size_t i = 0; i < in; ++i) {
            const size_t flat = base + i;
            const float wv = kCodebook[code_at(w->codes, flat)] * scales[flat / bs];
            acc += xr[i] * wv;
        }
        y[r * out + o] = acc;
    }
    free(scales);
}

void orc_nf4_linear_input_backward(const orc_nf4_weight* w, const float* dy,
                                   float* dx, size_t rows, int threads) {
    const size_t in = (size_t)w->in_features, out = (size_t)w->out_features;
    const size_t bs = (size_t)w->block_size;
    float* scales = decode_all_scales(w, NULL);
    const long long total = (long long)(rows * in);
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(threads > 1 ? threads : 1)
#else
    (void)threads;
#endif
    for (long long t = 0; t < total; ++t) {
        const size_t i = (size_t)t / rows, r = (size_t)t % rows;
        const float* g = dy + r * out;
        float acc = 0.0f;
        for (size_t o = 0; o < out; ++o) {
            const size_t flat = o * in + i;
            const float wv = kCodebook[code_at(w->codes, flat)] * scales[flat / bs];
            acc += g[o] * wv;
        }
        dx[r * in + i] = acc;
    }
    free(scales);
}

/* One (query vector, KV head) pair of paged_decode.cpp:52-130. `heads` is the
 * head count of the page tensor, `kv_head` the head read from it. */
static int paged_one_head(const float* q, const float* key_pages,
                          const float* value_pages, const uint32_t* table,
                          float* ctx, float* prob, size_t heads, size_t kv_head,
                          size_t width, size_t block_size, size_t seq_len) {
    const float scale = 1.0f / sqrtf((float)width);
    float maximum = -INFINITY;
    for (size_t p = 0; p < seq_len; ++p) {
        const size_t page = table[p / block_size], off = p % block_size;
        const float* k =
            key_pages + ((page * heads + kv_head) * block_size + off) * width;
        float score = 0.0f;
        for (size_t c = 0; c < width; ++c) score += q[c] * k[c];
        score *= scale;
        if (isnan(score) || score == INFINITY) return 1;
        prob[p] = score;
        if (score > maximum) maximum = score;
    }
    if (maximum == -INFINITY) return 2;

    double denom = 0.0;
    for (size_t p = 0; p < seq_len; ++p) {
        const double e = exp((double)(prob[p] - maximum));
        prob[p] = (float)e;
        denom += e;
    }
    for (size_t p = 0; p < seq_len; ++p)
        prob[p] = (float)((double)prob[p] / denom);

    for (size_t c = 0; c < width; ++c) {
        float acc = 0.0f;
        for (size_t p = 0; p < seq_len; ++p) {
            const size_t page = table[p / block_size], off = p % block_size;
            acc += prob[p] *
                   value_pages[((page * heads + kv_head) * block_size + off) *
                                   width + c];
        }
        ctx[c] = acc;
    }
    return 0;
}

int orc_paged_decode(const float* queries, const float* key_pages,
                     const float* value_pages, const uint32_t* block_table,
                     float* context, size_t heads, size_t head_width,
                     size_t block_size, size_t sequence_length) {
    memset(context, 0, heads * head_width * sizeof(float));
    float* prob = (float*)malloc(sequence_length * sizeof(float));
    int rc = 0;
    for (size_t h = 0; h < heads && rc == 0; ++h) {
        rc = paged_one_head(queries + h * head_width, key_pages, value_pages,
                            block_table, context + h * head_width, prob, heads,
                            h, head_width, block_size, sequence_length);
    }
    free(prob);
    return rc;
}

int orc_paged_decode_gqa(const float* queries, const float* key_pages,
                         const float* value_pages, const uint32_t* block_tables,
                         const uint32_t* seq_lens, float* context, size_t n_seq,
                         size_t q_heads, size_t kv_heads, size_t head_width,
                         size_t block_size, size_t max_blocks, int threads) {
    const size_t group = q_heads / kv_heads;
    const long long total = (long long)(n_seq * q_heads);
    int rc_all = 0;
    memset(context, 0, n_seq * q_heads * head_width * sizeof(float));
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads > 1 ? threads : 1)
#else
    (void)threads;
#endif
    for (long long t = 0; t < total; ++t) {
        const size_t s = (size_t)t / q_heads, h = (size_t)t % q_heads;
        const size_t len = seq_lens[s];
        float* prob = (float*)malloc((len ? len : 1) * sizeof(float));
        const int rc = paged_one_head(
            queries + (s * q_heads + h) * head_width, key_pages, value_pages,
            block_tables + s * max_blocks,
            context + (s * q_heads + h) * head_width, prob, kv_heads, h / group,
            head_width, block_size, len);
        free(prob);
        if (rc != 0) {
#ifdef _OPENMP
#pragma omp critical
#endif
            { if (rc_all == 0 || rc < rc_all) rc_all = rc; }
        }
    }
    return rc_all;
}

/* ---- decode-step primitives either side of the hot path ---------------------- */

/* rms_norm, src/nn/rms_norm.cpp:39-73: x * (1 / sqrt(mean(x * x) + eps)) * scale, where mean is
 * the reference reduction - a sequential FP32 sum followed by one division
 * (nn_reference_reduce, src/core/backend/nn/reference/operations.cpp:116-134) - and every
 * product is rounded on its own. */
void orc_rms_norm(const float* x, const float* scale, size_t rows, size_t width,
                  float epsilon, float* out) {
    for (size_t r = 0; r < rows; ++r) {
        const float* xr = x + r * width;
        float total = 0.0f;
        for (size_t c = 0; c < width; ++c) {
            const float square = xr[c] * xr[c];
            total += square;
        }
        const float mean_square = total / (float)width;
        const float inverse = 1.0f / sqrtf(mean_square + epsilon);
        for (size_t c = 0; c < width; ++c) {
            const float normalized = xr[c] * inverse;
            out[r * width + c] = normalized * scale[c];
        }
    }
}

/* stable_sigmoid / silu_forward, src/nn/activations.cpp:38-58 (libm expf, as the reference),
 * optionally times `up`: the hidden state of SwiGLU, src/model/swiglu.cpp:27-29. */
void orc_silu_mul(const float* gate, const float* up, size_t n, float* out) {
    for (size_t i = 0; i < n; ++i) {
        const float value = gate[i];
        float result;
        if (value == -INFINITY) {
            result = -0.0f;
        } else if (value >= 0.0f) {
            const float exponential = expf(-value);
            result = value * (1.0f / (1.0f + exponential));
        } else {
            const float exponential = expf(value);
            result = value * (exponential / (1.0f + exponential));
        }
        out[i] = up != NULL ? result * up[i] : result;
    }
}

/* GreedySampler::sample, src/stages/serving/generation.cpp:100-110: first maximum. */
size_t orc_greedy(const float* logits, size_t n) {
    size_t selected = 0;
    for (size_t i = 1; i < n; ++i) {
        if (logits[i] > logits[selected]) selected = i;
    }
    return selected;
}

/* LowRankAdapter::forward, src/nn/low_rank_adapter.cpp:132-158: ((x * A^T) * B^T) * scale with
 * A [rank, in], B [out, rank]; both products are the reference matmul (one FP32 accumulator per
 * output, contraction index ascending: src/core/backend/adapters/cpu/adapter.cpp:170-200). A
 * Linear with an adapter returns base + this (src/nn/linear.cpp:165-172). `reduced` is scratch
 * of rows * rank floats. */
void orc_lora_forward(const float* x, const float* a, const float* b, size_t rows,
                      size_t in_features, size_t out_features, size_t rank, float scale,
                      float* reduced, float* out) {
    for (size_t r = 0; r < rows; ++r) {
        for (size_t j = 0; j < rank; ++j) {
            float total = 0.0f;
            for (size_t i = 0; i < in_features; ++i) {
                const float product = x[r * in_features + i] * a[j * in_features + i];
                total += product;
            }
            reduced[r * rank + j] = total;
        }
    }
    for (size_t r = 0; r < rows; ++r) {
        for (size_t o = 0; o < out_features; ++o) {
            float total = 0.0f;
            for (size_t j = 0; j < rank; ++j) {
                const float product = reduced[r * rank + j] * b[o * rank + j];
                total += product;
            }
            out[r * out_features + o] = total * scale;
        }
    }
}
