/*
 * riftco_b200 - C ABI of the B200 (sm_100a) backend for Riftco's quantized
 * inference hot path: the packed-NF4 linear operator (forward and QLoRA
 * input-backward) and paged-KV single-token decode attention.
 *
 * The reference engine (quangng2000/riftco-transformer) reaches its backends
 * through a private C++ vtable; the entry points below are the function table a
 * binary CUDA plugin for that vtable binds. Each one names the reference
 * interface it replaces (paths are inside the reference project).
 *
 * Conventions
 *  - Plain pointers and sizes only. Unless a function says "host", every data
 *    pointer is a DEVICE pointer valid on the current CUDA device.
 *  - `stream` is a cudaStream_t passed as void* (NULL = the default stream).
 *    Device-pointer entry points only enqueue work: they return once the
 *    launches are queued and are ordered by the stream.
 *  - Every function returns a status with the numeric values of the
 *    reference's rt_status (include/riftco_transformer/c_api.h:41-49); the
 *    message of the last failure on the calling thread is b2_last_error().
 *  - There is no CPU fallback: without a usable CUDA device every compute entry
 *    point fails with B2_STATUS_BACKEND_UNAVAILABLE.
 */
#ifndef RIFTCO_B200_H
#define RIFTCO_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B2_ABI_VERSION 1

#if defined(__GNUC__)
#define B2_API __attribute__((visibility("default")))
#else
#define B2_API
#endif

#define B2_STATUS_OK 0
#define B2_STATUS_INVALID_ARGUMENT 1
#define B2_STATUS_OUT_OF_RANGE 2
#define B2_STATUS_OVERFLOW 3
#define B2_STATUS_BACKEND_UNAVAILABLE 4
#define B2_STATUS_OUT_OF_MEMORY 5
#define B2_STATUS_RUNTIME_ERROR 6
/* Not an rt_status value: marks the cases the reference reports by throwing
 * std::domain_error (non-finite attention scores,
 * src/core/backend/attention/reference/paged_decode.cpp:78-93). A C++ adapter
 * rethrows it as std::domain_error; the reference's C ABI then folds it into
 * RT_STATUS_INVALID_ARGUMENT (src/c_api/internal/error.hpp:25-27). */
#define B2_STATUS_DOMAIN_ERROR 7

/* Scale encodings: Nf4ScaleEncoding,
 * src/core/backend/nn/quantized_linear/storage.hpp:13-16. */
#define B2_SCALES_FLOAT32 0u
#define B2_SCALES_DOUBLE_QUANTIZED_UINT8 1u

/* Bits of the device status word written by b2_paged_decode_attention. */
#define B2_ATTN_STATUS_NAN_OR_POS_INF 1u   /* a score was NaN or +infinity      */
#define B2_ATTN_STATUS_ALL_NEG_INF 2u      /* every score of one head was -inf  */

/*
 * Borrowed view of one packed NF4 weight, flat row-major [out_features,
 * in_features]. It carries what QuantizedWeightStorage exposes
 * (src/core/backend/nn/quantized_linear/storage.hpp:81-108: packed codes,
 * primary and secondary scale handles) plus Nf4ScaleStorageView's scalars
 * (storage.hpp:31-46) and QuantizedLinearDimensions' widths and block size
 * (src/core/backend/nn/quantized_linear/contracts.hpp:10-15).
 *
 * Layout consumed unchanged: element i lives in byte i/2, even i in the low
 * nibble (src/core/quantization/nf4.cpp:70-85); block b = i / block_size over
 * the FLAT index. A row shard [r0, r1) of a larger weight is described by
 * pointing `codes` and `scales_primary` at the shard's first byte/block,
 * leaving `scales_secondary` at the parent's first second-level scale and
 * setting flat_block_base to the parent's index of the shard's first block
 * (the shard must start on a block boundary and on a whole byte).
 */
typedef struct b2_nf4_weight {
    const uint8_t* codes;           /* ceil(out*in/2) bytes                         */
    const void* scales_primary;     /* float[blocks] or uint8_t[blocks]             */
    const float* scales_secondary;  /* NULL, or float[ceil(blocks/scale_block_size)] */
    uint32_t encoding;              /* B2_SCALES_*                                  */
    uint32_t block_size;            /* 32..4096, power of two (nf4.cpp:39-52)       */
    uint64_t scale_block_size;      /* 0 for FLOAT32, else 32..4096 power of two    */
    float scale_offset;             /* shared mean of first-level scales, 0 for F32 */
    uint32_t reserved;              /* must be 0                                    */
    uint64_t out_features;
    uint64_t in_features;
    uint64_t flat_block_base;       /* 0 for a whole weight                         */
} b2_nf4_weight;

/* ---- library ----------------------------------------------------------- */

B2_API int32_t b2_abi_version(void);

/* Thread-local message of the last failed call on this thread; "" if none.
 * Counterpart of rt_last_error (include/riftco_transformer/c_api.h:339-345). */
B2_API const char* b2_last_error(void);

/* 1 when a CUDA device of compute capability 10.x is current and usable.
 * Replaces BackendAdapter::is_available (src/core/backend/adapter.hpp:74-79). */
B2_API int32_t b2_is_available(void);

/* Reason string for b2_is_available() == 0; "" otherwise. Replaces
 * BackendAdapter::unavailability_reason (adapter.hpp:76-79). */
B2_API const char* b2_unavailability_reason(void);

/* ---- packed NF4 linear ------------------------------------------------- */

/* out[i] = codebook[code(i)] * decoded_scale(i / block_size), bit-exact with
 * QuantizedWeight::dequantize (src/core/quantization/quantized_weight.cpp,
 * scale decode per storage.hpp:48-65). out: float[out*in]. */
B2_API int32_t b2_nf4_dequantize(const b2_nf4_weight* weight, float* out, void* stream);

/* The reference's NF4 encoder on a device tensor: values float[out,in] -> packed codes and block
 * scales, bit for bit what QuantizedWeight::quantize_nf4 (scale_block_size == 0: scales_primary
 * receives float[blocks]) and quantize_nf4_double_quantized (scales_primary receives uint8[blocks],
 * scales_secondary float[ceil(blocks / scale_block_size)], *scale_offset the shared mean) produce:
 * pack_nf4 / double_quantize_scales, src/core/quantization/quantized_weight.cpp:176-254, nearest
 * level with ties to the lower code (src/core/quantization/nf4.cpp:55-68), a zero block keeps scale 0
 * and code 7. codes: uint8[ceil(out*in/2)]. scale_offset is a HOST pointer; the call returns after
 * the stream is idle. Non-finite values are INVALID_ARGUMENT ("NF4 source values must be finite"),
 * a non-finite mean OVERFLOW. workspace: b2_nf4_quantize_workspace_bytes, 256-byte aligned. */
B2_API size_t b2_nf4_quantize_workspace_bytes(uint64_t out_features, uint64_t in_features,
                                              uint32_t block_size, uint64_t scale_block_size);
B2_API int32_t b2_nf4_quantize(const float* values, uint64_t out_features, uint64_t in_features,
                               uint32_t block_size, uint64_t scale_block_size, uint8_t* codes,
                               void* scales_primary, float* scales_secondary, float* scale_offset,
                               void* workspace, size_t workspace_bytes, void* stream);

/* require_canonical_payload (quantized_weight.cpp:102-174) for a payload in device memory: the
 * three array lengths against shape and block sizes, the unused high nibble of an odd element
 * count, finite non-negative second-level and decoded block scales, and code 7 throughout every
 * zero-scale block of the FP32-scale form; INVALID_ARGUMENT with the reference's message
 * otherwise. b2_nf4_weight carries no lengths, so the compute entry points cannot apply these
 * rules themselves: a loader calls this once per weight. Synchronous. */
B2_API int32_t b2_nf4_validate_payload(const b2_nf4_weight* weight, uint64_t codes_bytes,
                                       uint64_t primary_count, uint64_t secondary_count, void* stream);

/* y[r,o] = sum_i x[r,i] * W[o,i]. x: float[rows,in], y: float[rows,out].
 * Replaces QuantizedLinearCapability::quantized_linear_forward
 * (src/core/backend/nn/quantized_linear/capability.hpp:35-41; CUDA launcher
 * cuda_quantized_linear_forward, quantized_linear/cuda/launch.hpp:16-17; loop
 * reference/operations.cpp:49-81). Validation follows
 * dispatch_quantized_linear_forward (quantized_linear/dispatch.cpp:317-341):
 * zero/overflowing dimensions and aliasing x/y or weight/y are rejected.
 * workspace may be NULL: the library then uses its own per-device arena, and
 * calls that share the arena must be ordered on one stream. The arena only
 * grows and never frees or moves memory it has handed out, so an address a
 * CUDA graph captured stays valid for the life of the process; a call that
 * would have to grow the arena while its stream is being captured fails with
 * B2_STATUS_INVALID_ARGUMENT (make the first call of a shape outside capture,
 * or pass a workspace). */
B2_API int32_t b2_nf4_linear_forward(const b2_nf4_weight* weight, const float* x, float* y,
                              uint64_t rows, void* workspace, size_t workspace_bytes,
                              void* stream);

/* A packed-NF4 linear with a low-rank adapter: y = x * W^T + scale * ((x * A^T) * B^T), A [rank, in],
 * B [out, rank] FP32 device arrays, scale = alpha / rank. Replaces Linear::forward with an attached
 * adapter (src/nn/linear.cpp:165-172: base_output + lora_->forward(input)) and LowRankAdapter::forward
 * (src/nn/low_rank_adapter.cpp:132-158) on top of the packed base weight. The base projection runs
 * on the same kernels as b2_nf4_linear_forward; the branch is FP32. rank <= 64. workspace:
 * b2_nf4_linear_lora_workspace_bytes (NULL: the library's arena). */
B2_API size_t b2_nf4_linear_lora_workspace_bytes(const b2_nf4_weight* weight, uint64_t rows, uint32_t rank);
B2_API int32_t b2_nf4_linear_forward_lora(const b2_nf4_weight* weight, const float* x, const float* lora_a,
                                          const float* lora_b, uint32_t rank, float scale, float* y,
                                          uint64_t rows, void* workspace, size_t workspace_bytes, void* stream);

/* Several packed linears of the SAME input in one call: ys[i][r,o] = sum_k x[r,k] * W_i[o,k]
 * for `count` weights with equal in_features (the q / k / v projections of an attention block,
 * the gate / up projections of a SwiGLU block: src/model/grouped_query_attention.cpp:61-94,
 * src/model/swiglu.cpp:27-29 apply them one after the other to the same tensor). With more
 * than 16 rows and up to four weights the activations are converted once and one kernel launch
 * covers every weight's tiles. Results agree with `count` calls of b2_nf4_linear_forward on the
 * same arguments to FP32 summation order (the persistent decode kernel cuts the contraction of
 * a tile where its work list says, and the list depends on how many tiles one launch holds):
 * relative L2 difference <= 1e-5, and bit-for-bit from one call of this function to the next.
 * Validation, workspace and stream rules as for b2_nf4_linear_forward (the workspace need is
 * that of any single one of the calls). */
B2_API int32_t b2_nf4_linear_forward_multi(const b2_nf4_weight* weights, uint32_t count, const float* x,
                                    float* const* ys, uint64_t rows, void* workspace,
                                    size_t workspace_bytes, void* stream);

/* b2_nf4_linear_forward_multi on activations the caller already holds as bf16
 * (x_bf16: [rows, in_features], row-major, 16-byte aligned), e.g. written by
 * b2_rmsnorm_bf16 / b2_silu_mul_bf16. Results equal those of
 * b2_nf4_linear_forward_multi on the FP32 values the bf16 copy was rounded
 * from (that call rounds them the same way before its tensor-core kernel); no
 * conversion pass is launched and no workspace is needed. Only the
 * tensor-memory kernel takes this form: more than 16 rows, 1-4 weights of one
 * input width. b2_nf4_linear_bf16_supported returns 1 when a call with these
 * weights and rows would be accepted, else 0; an unsupported call fails with
 * B2_STATUS_INVALID_ARGUMENT. */
B2_API int32_t b2_nf4_linear_bf16_supported(const b2_nf4_weight* weights, uint32_t count,
                                            uint64_t rows);
B2_API int32_t b2_nf4_linear_forward_multi_bf16(const b2_nf4_weight* weights, uint32_t count,
                                                const void* x_bf16, float* const* ys,
                                                uint64_t rows, void* stream);

/* dx[r,i] = sum_o dy[r,o] * W[o,i]. dy: float[rows,out], dx: float[rows,in].
 * Replaces QuantizedLinearCapability::quantized_linear_input_backward
 * (capability.hpp:43-49; launch.hpp:19-20; loop reference/operations.cpp:83-115;
 * validation dispatch.cpp:343-370). */
B2_API int32_t b2_nf4_linear_input_backward(const b2_nf4_weight* weight, const float* dy,
                                     float* dx, uint64_t rows, void* workspace,
                                     size_t workspace_bytes, void* stream);

/* Bytes of scratch the two calls above need for `rows` rows of this weight
 * (0 when the chosen kernel needs none). `backward` selects the operator. */
B2_API size_t b2_nf4_linear_workspace_bytes(const b2_nf4_weight* weight, uint64_t rows,
                                     int32_t backward);

/* ---- paged-KV decode attention ----------------------------------------- */

/*
 * Single-token decode attention over block-addressed K/V pages for a batch of
 * sequences with grouped-query heads.
 *   q, ctx      float[n_seq, q_heads, head_width]
 *   k/v_pages   float[physical_blocks, kv_heads, block_size, head_width]
 *   block_tables uint32[n_seq, max_blocks]; row s uses its first
 *               ceil(seq_lens[s] / block_size) entries
 *   seq_lens    uint32[n_seq], each >= 1
 * Query head h reads KV head h / (q_heads / kv_heads).
 * With n_seq == 1 and q_heads == kv_heads this is exactly
 * AttentionCapability::paged_decode_attention_forward
 * (src/core/backend/attention/capability.hpp:28-30; request and page layout
 * src/core/backend/attention/contracts.hpp:88-106; loop
 * attention/reference/paged_decode.cpp:37-132; CUDA launcher
 * attention/cuda/paged_decode.cu:144-215).
 * `status` (device uint32, may be NULL) receives B2_ATTN_STATUS_* bits; the
 * caller zeroes it and reads it after synchronising, which is how the
 * reference's CUDA path reports std::domain_error (paged_decode.cu:208-214).
 * Block ids are checked on the device: an id >= physical_blocks is never
 * dereferenced and sets B2_ATTN_STATUS_BAD_BLOCK (value 4) in the status word.
 */
#define B2_ATTN_STATUS_BAD_BLOCK 4u
#define B2_ATTN_STATUS_TIMEOUT 8u          /* a bounded wait for a page copy gave up */

/* The status a synchronous caller reports for a status word read back after the
 * stream is idle, with the message in b2_last_error(): BAD_BLOCK ->
 * B2_STATUS_OUT_OF_RANGE (std::out_of_range in the reference,
 * src/core/backend/attention/dispatch.cpp:474-480), the two score bits ->
 * B2_STATUS_DOMAIN_ERROR (attention/cuda/paged_decode.cu:208-214), TIMEOUT or
 * any other bit -> B2_STATUS_RUNTIME_ERROR (the context is invalid), 0 ->
 * B2_STATUS_OK. Needs no GPU. b2_host_paged_decode_attention applies it. */
B2_API int32_t b2_attention_status_result(uint32_t status_bits);
B2_API int32_t b2_paged_decode_attention(const float* q, const float* k_pages,
                                  const float* v_pages, const uint32_t* block_tables,
                                  const uint32_t* seq_lens, float* ctx,
                                  uint32_t n_seq, uint32_t q_heads, uint32_t kv_heads,
                                  uint32_t head_width, uint32_t block_size,
                                  uint64_t physical_blocks, uint32_t max_blocks,
                                  uint32_t max_seq_len, void* workspace,
                                  size_t workspace_bytes, uint32_t* status,
                                  void* stream);

/* b2_paged_decode_attention that also writes a bf16 copy of the context
 * (ctx_bf16: [n_seq, q_heads, head_width], round to nearest even of the FP32
 * value stored in ctx), for a following output projection that reads bf16
 * activations (b2_nf4_linear_forward_multi_bf16): the projection then needs no
 * conversion pass. In the reference the projection consumes the attention
 * output directly (src/model/grouped_query_attention.cpp:254,
 * output_.forward(merge_attention_heads(attention.context))). */
B2_API int32_t b2_paged_decode_attention_bf16(const float* q, const float* k_pages,
                                  const float* v_pages, const uint32_t* block_tables,
                                  const uint32_t* seq_lens, float* ctx, void* ctx_bf16,
                                  uint32_t n_seq, uint32_t q_heads, uint32_t kv_heads,
                                  uint32_t head_width, uint32_t block_size,
                                  uint64_t physical_blocks, uint32_t max_blocks,
                                  uint32_t max_seq_len, void* workspace,
                                  size_t workspace_bytes, uint32_t* status,
                                  void* stream);

/* Scratch bytes for the calls above (split-K partial results). */
B2_API size_t b2_paged_decode_workspace_bytes(uint32_t n_seq, uint32_t q_heads,
                                       uint32_t head_width, uint32_t block_size,
                                       uint32_t max_seq_len);

/*
 * The same attention as b2_paged_decode_attention for callers that must not
 * allocate device memory: an engine whose memory is entirely owned by its own
 * pool, or a call site where cudaMalloc / cudaFree are unwelcome because they
 * synchronise the whole device. It has no counterpart in the reference. The
 * split-K scratch is a fixed B2_NOALLOC_SCRATCH_BYTES array inside the library
 * (each GPU that loads the library holds it until the process exits), and the
 * call itself performs no cudaMalloc, cudaFree or other allocating routine.
 *  - Limit: the call is rejected with B2_STATUS_INVALID_ARGUMENT when
 *    b2_paged_decode_workspace_bytes(...) for its shape exceeds
 *    B2_NOALLOC_SCRATCH_BYTES (head_width 128 / block_size 16: n_seq * q_heads *
 *    ceil(max_seq_len / 256) * 520 bytes, 0 when max_seq_len <= 256).
 *  - The first call on each device looks up the array's device address; make
 *    that first call outside any stream capture.
 *  - All calls on a device share the one array. Nothing in it has to start at
 *    zero (every partial result is written before it is read), but two calls
 *    whose kernels overlap on the GPU - different streams, or threads - race on
 *    it: order them on one stream.
 */
#define B2_NOALLOC_SCRATCH_BYTES (8u * 1024u * 1024u)
B2_API int32_t b2_paged_decode_attention_noalloc(
    const float* q, const float* k_pages, const float* v_pages, const uint32_t* block_tables,
    const uint32_t* seq_lens, float* ctx, uint32_t n_seq, uint32_t q_heads, uint32_t kv_heads,
    uint32_t head_width, uint32_t block_size, uint64_t physical_blocks, uint32_t max_blocks,
    uint32_t max_seq_len, uint32_t* status, void* stream);

/* ---- decode-step glue ---------------------------------------------------- */
/*
 * The small operators either side of the linears and the attention in one
 * decode step of a Llama-shaped decoder, so the whole step can stay on the
 * device. All pointers are device pointers; calls only enqueue.
 */

/* y[r,:] = x[r,:] * (1 / sqrt(mean(x[r,:]^2) + eps)) * scale (rms_norm,
 * src/nn/rms_norm.cpp:39-73). With delta != NULL the residual stream is
 * updated first: x_out = x + delta, and the norm is taken of x_out (x_out may
 * equal x). With delta == NULL x_out is ignored. */
B2_API int32_t b2_rmsnorm(const float* x, const float* delta, float* x_out, const float* scale,
                          float* y, uint64_t rows, uint64_t width, float eps, void* stream);

/* b2_rmsnorm that also writes y rounded to bf16 (nearest even) into y_bf16
 * [rows, width] when it is not NULL: the activation form
 * b2_nf4_linear_forward_multi_bf16 reads, so the linear that follows needs no
 * conversion pass of its own. */
B2_API int32_t b2_rmsnorm_bf16(const float* x, const float* delta, float* x_out, const float* scale,
                               float* y, void* y_bf16, uint64_t rows, uint64_t width, float eps,
                               void* stream);

/* Split-half rotary embedding of the new token of every sequence, in place on
 * q [n_seq, q_heads, d] and while copying k [n_seq, kv_heads, d] into its page
 * slot; v [n_seq, kv_heads, d] is copied unchanged. positions[s] is the token's
 * position (= its slot in the sequence's pages). RoPE: rotate_forward,
 * src/model/rotary_embedding.cpp:64-117 (pairs (c, c + d/2), angle =
 * position * theta^(-2c/d) in double). Page write: copy_token_to_page,
 * src/stages/serving/cache/page_table_cache.cpp:44-77. A block id outside the
 * pool is not written and sets B2_ATTN_STATUS_BAD_BLOCK in *status. */
B2_API int32_t b2_rope_append_kv(float* q, const float* k, const float* v, const uint32_t* positions,
                                 const uint32_t* block_tables, float* k_pages, float* v_pages,
                                 uint32_t n_seq, uint32_t q_heads, uint32_t kv_heads,
                                 uint32_t head_width, uint32_t block_size, uint64_t physical_blocks,
                                 uint32_t max_blocks, float theta, uint32_t* status, void* stream);

/* b2_rope_append_kv for a CHUNK of tokens (batched prefill): q / k / v hold n_tokens rows, token t
 * belongs to sequence token_seq[t] (its block-table row) and sits at positions[t]. Several tokens
 * of one sequence may be given in one call, in any order; each lands in slot positions[t] %
 * block_size of page block_tables[token_seq[t]][positions[t] / block_size]. The reference prefills
 * token by token through decode_token (src/stages/serving/generation.cpp:260-398) and
 * copy_token_to_page (src/stages/serving/cache/page_table_cache.cpp:44-77); this call writes what
 * that loop writes, for the whole chunk at once. */
B2_API int32_t b2_rope_append_kv_tokens(float* q, const float* k, const float* v, const uint32_t* positions,
                                        const uint32_t* token_seq, const uint32_t* block_tables,
                                        float* k_pages, float* v_pages, uint32_t n_tokens, uint32_t q_heads,
                                        uint32_t kv_heads, uint32_t head_width, uint32_t block_size,
                                        uint64_t physical_blocks, uint32_t max_blocks, float theta,
                                        uint32_t* status, void* stream);

/* out = silu(gate) * up, silu as silu_forward (src/nn/activations.cpp:38-58);
 * the product is SwiGLU's hidden state (src/model/swiglu.cpp:27-29). */
B2_API int32_t b2_silu_mul(const float* gate, const float* up, float* out, uint64_t n, void* stream);

/* b2_silu_mul that also writes the product rounded to bf16 into out_bf16 [n]
 * when it is not NULL. */
B2_API int32_t b2_silu_mul_bf16(const float* gate, const float* up, float* out, void* out_bf16,
                                uint64_t n, void* stream);

/* out = a + b (residual add). */
B2_API int32_t b2_add(const float* a, const float* b, float* out, uint64_t n, void* stream);

/* out[r,:] = table[ids[r],:] (embedding lookup; gather_rows of the reference's
 * IndexingCapability, src/core/backend/nn/capability.hpp). An id >= vocab reads
 * row 0 and sets bit 0 of *status. */
B2_API int32_t b2_gather_rows(const float* table, const uint32_t* ids, float* out, uint32_t rows,
                              uint32_t width, uint32_t vocab, uint32_t* status, void* stream);

/* All-gather of column shards over NVLink peer memory (tensor-parallel decode:
 * the reference keeps activations whole and shards nothing, so this call has no
 * reference counterpart; it joins the row-sharded outputs of b2_nf4_linear_forward,
 * src/core/backend/nn/quantized_linear/reference/operations.cpp:49-81, across GPUs).
 * local[rows, cols] holds this rank's columns rank*cols .. of the full activation;
 * the kernel stores them into full[rows, world*cols] of EVERY rank and returns
 * once every rank's columns have arrived here.
 *   peer_full   device array [world] of addresses: each rank's full buffer
 *   peer_flags  device array [world] of addresses: each rank's uint32[world] flag array
 *   state       local device uint32[2], zero before the first call (epoch, CTA counter)
 *   status      local device word; B2_PEER_STATUS_TIMEOUT is set when a peer did not
 *               arrive within two seconds (the kernel then returns, it never hangs)
 * Buffers must be peer-mapped (e.g. CUDA IPC / symmetric memory), cols a multiple
 * of 4, and consecutive gathers must not reuse the same full buffer. Every rank
 * must issue the same sequence of gathers. */
#define B2_PEER_STATUS_TIMEOUT 16u
B2_API int32_t b2_peer_all_gather_columns(const float* local, uint64_t rows, uint64_t cols,
                                          const uint64_t* peer_full, const uint64_t* peer_flags, uint32_t rank,
                                          uint32_t world, uint32_t* state, uint32_t* status, void* stream);

/* b2_peer_all_gather_columns that also stores the shard rounded to bf16 (nearest
 * even) into a second buffer of every rank: peer_full_bf16 is a device array
 * [world] of the addresses of each rank's bf16 [rows, world*cols] buffer (8-byte
 * aligned, peer-mapped like peer_full), or NULL for none. The linear that follows
 * can then take b2_nf4_linear_forward_multi_bf16. */
B2_API int32_t b2_peer_all_gather_columns_bf16(const float* local, uint64_t rows, uint64_t cols,
                                               const uint64_t* peer_full, const uint64_t* peer_full_bf16,
                                               const uint64_t* peer_flags, uint32_t rank, uint32_t world,
                                               uint32_t* state, uint32_t* status, void* stream);

/* out[r] = index of the first maximum of logits[r,:] (greedy sampling,
 * src/stages/serving/generation.cpp:100-120). */
B2_API int32_t b2_argmax(const float* logits, uint32_t* out, uint32_t rows, uint32_t width, void* stream);

/* Synchronises the device and reports (then clears) sticky device-side error
 * flags of earlier asynchronous calls: today, a bounded barrier wait inside the
 * tensor-core GEMM that gave up (B2_STATUS_RUNTIME_ERROR). Kernels never trap or
 * spin forever; this is how such a failure reaches the host. The reference
 * reads a device status word the same way after its kernels
 * (src/core/backend/attention/cuda/common.cuh:124-133). */
B2_API int32_t b2_check_device_errors(void);

/* Which kernel family served the calling thread's last linear or attention call. The library
 * picks the kernel from the request's shape and alignment alone; every family computes the
 * result the reference's dispatch_quantized_linear_forward / _input_backward
 * (src/core/backend/nn/quantized_linear/dispatch.cpp:317-370) and
 * dispatch_paged_decode_attention_forward define. This entry lets a test assert that a shape
 * reached the path it is meant to cover. Needs no GPU. */
#define B2_ROUTE_NONE 0
#define B2_ROUTE_DECODE_TMEM 1      /* persistent tcgen05 decode kernel, up to 32 rows */
#define B2_ROUTE_GEMV_TMA 2         /* TMA-fed mma.sync decode kernel, up to 16 rows per pass */
#define B2_ROUTE_GEMV_TILE 3        /* tiled mma.sync decode kernel: any out_features, in % 64 == 0 */
#define B2_ROUTE_GEMM_TMEM 4        /* tcgen05 GEMM, expanded weight tile in tensor memory */
#define B2_ROUTE_GEMM_SMEM 5        /* tcgen05 GEMM that transposes the nibbles inside the SM: input
                                     * backward of 33..511 rows */
#define B2_ROUTE_BACKWARD_DENSE 6   /* input backward: transposed bf16 expansion + tcgen05 GEMM */
#define B2_ROUTE_GENERIC 7          /* FP32 SIMT kernels, any shape */
#define B2_ROUTE_ATTENTION_BULK 8   /* head_width 128, block_size 16, rep in {1,2,4,8} */
#define B2_ROUTE_ATTENTION_GENERIC 9
B2_API int32_t b2_last_route(void);

/* ---- host-buffer seam --------------------------------------------------- */
/*
 * The reference adapter contract is synchronous over host-visible storage
 * (TensorStorage::data() is a host span, src/core/backend/storage.hpp:15-29;
 * "must finish writing output before returning", adapter.hpp:50-52). These
 * forms take HOST pointers for activations, copy them to the device, run the
 * same kernels, copy the result back and return after the stream is idle.
 * The weight / KV pools stay device-resident, as the reference's CUDA storage
 * keeps them (quantized_linear/cuda/storage.cu:72-135).
 */
B2_API int32_t b2_host_nf4_linear_forward(const b2_nf4_weight* weight, const float* x_host,
                                   float* y_host, uint64_t rows, void* stream);
B2_API int32_t b2_host_nf4_linear_input_backward(const b2_nf4_weight* weight,
                                          const float* dy_host, float* dx_host,
                                          uint64_t rows, void* stream);
/* q_host/ctx_host/block_tables_host/seq_lens_host are host pointers; pages are
 * device pointers. Block ids and lengths are validated on the host first, as
 * dispatch_paged_decode_attention_forward does
 * (src/core/backend/attention/dispatch.cpp:440-509): a short table or zero
 * dimension is INVALID_ARGUMENT, an id >= physical_blocks OUT_OF_RANGE, and a
 * non-finite score comes back as B2_STATUS_DOMAIN_ERROR. */
B2_API int32_t b2_host_paged_decode_attention(const float* q_host, const float* k_pages,
                                       const float* v_pages,
                                       const uint32_t* block_tables_host,
                                       const uint32_t* seq_lens_host, float* ctx_host,
                                       uint32_t n_seq, uint32_t q_heads,
                                       uint32_t kv_heads, uint32_t head_width,
                                       uint32_t block_size, uint64_t physical_blocks,
                                       uint32_t max_blocks, void* stream);

/* ---- packed model state (RTNF4S1) -------------------------------------------------------
 * The reference's canonical stream of packed NF4 linear weights
 * (packed_model_state_bytes / parse_packed_model_state, src/c_api/model_state.cpp:27-113,
 * 165-297): magic "RTNF4S1\0", u64 weight count, then per weight
 *   u64 rank (= 2), u64 block_size, u64 n_codes, u64 n_fp32_scales, u64 n_scale_codes,
 *   u64 n_second, u64 scale_block_size, f32 offset, u32 flags (1 = double-quantised),
 *   u64 dims[2], packed codes, f32 block scales, [u8 scale codes, f32 second-level scales],
 * everything little-endian. b2_rtnf4_index walks a stream held in host memory, applies the
 * reference parser's checks (truncation, unknown magic or flags, rank != 2, inconsistent scale
 * metadata, trailing bytes -> INVALID_ARGUMENT; sizes past the address space -> OVERFLOW) and
 * reports where each array lies, so a loader can copy row shards of codes and scales straight
 * from the stream into device memory without an FP32 detour. Writes at most `capacity`
 * entries; *count receives the number of weights in the stream. No GPU is needed. */
typedef struct b2_rtnf4_entry {
    uint64_t block_size;
    uint64_t out_features;       /* dims[0] */
    uint64_t in_features;        /* dims[1] */
    uint64_t n_codes;            /* packed bytes */
    uint64_t n_fp32_scales;      /* FP32 block scales (flags 0) */
    uint64_t n_scale_codes;      /* u8 scale codes (flags 1) */
    uint64_t n_second;           /* FP32 second-level scales (flags 1) */
    uint64_t scale_block_size;
    float offset;
    uint32_t double_quantized;   /* flags */
    uint64_t codes_offset;       /* byte offsets from the start of the stream */
    uint64_t fp32_scales_offset;
    uint64_t scale_codes_offset;
    uint64_t second_offset;
} b2_rtnf4_entry;

B2_API int32_t b2_rtnf4_index(const uint8_t* stream, uint64_t bytes, b2_rtnf4_entry* entries,
                              uint64_t capacity, uint64_t* count);

#ifdef __cplusplus
}
#endif
#endif /* RIFTCO_B200_H */
