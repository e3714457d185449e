// Internal launcher interface between the C-ABI layer (api.cu) and the kernel
// translation units. Every launcher only enqueues work on `stream`.
#pragma once

#include "b2_common.cuh"

namespace b2 {

// nf4_dequant.cu
int32_t launch_nf4_dequantize(const DeviceContext& ctx, const WeightView& w, float* out,
                              cudaStream_t stream);

// nf4_quantize.cu - the reference's NF4 encoder and payload validation on the device (both synchronous).
size_t nf4_quantize_workspace_bytes(const DeviceContext& ctx, uint64_t blocks, bool double_quantized);
int32_t run_nf4_quantize(const DeviceContext& ctx, const float* values, uint64_t out_features, uint64_t in_features,
                         uint32_t block_size, uint64_t scale_block_size, uint8_t* codes, void* primary,
                         float* secondary, float* offset_out, void* workspace, cudaStream_t stream);
int32_t run_nf4_validate(const DeviceContext& ctx, const WeightView& w, uint64_t second_count, uint32_t* flags_word,
                         cudaStream_t stream);

// nf4_lora.cu - the low-rank adapter branch added to a base projection already in y.
bool lora_rank_supported(uint64_t rank);
size_t lora_workspace_bytes(uint64_t rows, uint64_t rank);
int32_t launch_lora_branch(const DeviceContext& ctx, const float* x, const float* a, const float* b, float* y,
                           uint64_t rows, uint64_t in_features, uint64_t out_features, uint32_t rank, float scale,
                           float* reduced, cudaStream_t stream);

// nf4_linear_generic.cu - any shape, any block size, FP32 SIMT.
int32_t launch_nf4_linear_forward_generic(const DeviceContext& ctx, const WeightView& w,
                                          const float* x, float* y, uint64_t rows,
                                          cudaStream_t stream);
int32_t launch_nf4_linear_input_backward_generic(const DeviceContext& ctx, const WeightView& w,
                                                 const float* dy, float* dx, uint64_t rows,
                                                 cudaStream_t stream);

// Records the kernel family (B2_ROUTE_*) that serves the calling thread's current call.
void note_route(int32_t route);

// nf4_gemv.cu - tiled decode kernel, rows <= 32, any row count of the weight.
bool nf4_gemv_supported(const WeightView& w, const float* x, const float* y, uint64_t rows);
int32_t launch_nf4_gemv(const DeviceContext& ctx, const WeightView& w, const float* x, float* y,
                        uint64_t rows, cudaStream_t stream);
int32_t init_gemv_lut(DeviceContext* ctx);

// nf4_gemv_tma.cu - TMA-fed decode kernel, rows <= 16.
bool nf4_gemv_tma_plan(const DeviceContext& ctx, const WeightView& w, const float* x, uint64_t rows,
                       uint32_t* ksplit_out, uint32_t* steps_per_cta_out);
int32_t launch_nf4_gemv_tma(const DeviceContext& ctx, const WeightView& w, const float* x, float* y,
                            uint64_t rows, uint32_t ksplit, uint32_t steps_per_cta, cudaStream_t stream);

// nf4_gemm_sm100.cu - tcgen05 prefill GEMM, rows > 32.
int32_t init_gemm_lut(DeviceContext* ctx);
int32_t launch_f32_to_bf16(const DeviceContext& ctx, const float* src, void* dst, uint64_t count, cudaStream_t stream);
bool nf4_gemm_tmem_supported(const WeightView& w, const float* x, uint64_t rows);
size_t nf4_gemm_tmem_workspace_bytes(const WeightView& w, uint64_t rows);
int32_t launch_nf4_gemm_tmem(const DeviceContext& ctx, const WeightView& w, const void* x_bf16, float* y,
                             uint64_t rows, cudaStream_t stream);
int32_t launch_nf4_gemm_tmem_multi(const DeviceContext& ctx, const WeightView* ws, float* const* ys, uint32_t count,
                                   const void* x_bf16, uint64_t rows, cudaStream_t stream);
// nf4_decode_tmem.cu - persistent stream-K tcgen05 kernel for decode batches (1..32 rows); `x16` is the
// bf16 (half == false) or fp16 (half == true) copy of the activations.
bool nf4_decode_tmem_supported(const WeightView& w, const void* x, uint64_t rows);
size_t nf4_decode_tmem_workspace_bytes(const DeviceContext& ctx);
int32_t launch_f32_to_f16(const DeviceContext& ctx, const float* src, void* dst, uint64_t count, cudaStream_t stream);
int32_t launch_nf4_decode_tmem(const DeviceContext& ctx, const WeightView* ws, float* const* ys, uint32_t count,
                               const void* x16, bool half, uint64_t rows, void* partial, uint32_t* counters,
                               cudaStream_t stream);
// nf4_backward_dense.cu - input-backward for many rows: transposed bf16 expansion + plain tcgen05 GEMM.
bool nf4_backward_dense_supported(const WeightView& w, const float* dy, uint64_t rows);
size_t nf4_backward_dense_workspace_bytes(const WeightView& w, uint64_t rows);
int32_t launch_nf4_backward_dense(const DeviceContext& ctx, const WeightView& w, const float* dy, float* dx,
                                  uint64_t rows, void* workspace, size_t workspace_bytes, cudaStream_t stream);
bool nf4_gemm_supported(const WeightView& w, const float* x, uint64_t rows, bool backward);
size_t nf4_gemm_workspace_bytes(const WeightView& w, uint64_t rows, bool backward);
int32_t launch_nf4_gemm(const DeviceContext& ctx, const WeightView& w, const float* x, float* y, uint64_t rows,
                        bool backward, void* workspace, size_t workspace_bytes, cudaStream_t stream);

// paged_decode.cu
struct PagedDecodeArgs {
    const float* q;
    const float* k_pages;
    const float* v_pages;
    const uint32_t* block_tables;
    const uint32_t* seq_lens;
    float* ctx;
    uint32_t n_seq, q_heads, kv_heads, head_width, block_size, max_blocks, max_seq_len;
    uint64_t physical_blocks;
    uint32_t* status;  // may be null
    void* ctx16 = nullptr;   // optional bf16 copy of ctx (round to nearest even), written with it
};
// Dimension rules of dispatch_paged_decode_attention_forward that need no view of device data
// (src/core/backend/attention/dispatch.cpp:179-219,440-509); defined in api.cu.
int32_t check_paged_dims(uint32_t n_seq, uint32_t q_heads, uint32_t kv_heads, uint32_t head_width,
                         uint32_t block_size, uint64_t physical_blocks, uint32_t max_blocks,
                         uint32_t max_seq_len);
size_t paged_decode_workspace_bytes(uint32_t n_seq, uint32_t q_heads, uint32_t head_width,
                                    uint32_t block_size, uint32_t max_seq_len);
int32_t launch_paged_decode(const DeviceContext& ctx, const PagedDecodeArgs& args, void* workspace,
                            size_t workspace_bytes, cudaStream_t stream);


// decode_glue.cu
// y_bf16 / out_bf16 (nullable): a bf16 copy of the result, the form the tensor-core linears read.
int32_t launch_rmsnorm(const float* x, const float* delta, float* x_out, const float* scale, float* y,
                       void* y_bf16, uint64_t rows, uint32_t width, float eps, cudaStream_t stream);
// token_seq == nullptr: one token per sequence (token index = block-table row); else the row of each token.
int32_t launch_rope_append(float* q, const float* k, const float* v, const uint32_t* positions,
                           const uint32_t* token_seq, const uint32_t* block_tables, float* k_pages,
                           float* v_pages, uint32_t n_seq,
                           uint32_t q_heads, uint32_t kv_heads, uint32_t d, uint32_t block_size,
                           uint64_t physical_blocks, uint32_t max_blocks, float theta, uint32_t* status,
                           cudaStream_t stream);
int32_t launch_silu_mul(const DeviceContext& ctx, const float* gate, const float* up, float* out, void* out_bf16,
                        uint64_t n, cudaStream_t stream);
int32_t launch_add(const DeviceContext& ctx, const float* a, const float* b, float* out, uint64_t n,
                   cudaStream_t stream);
int32_t launch_gather_rows(const float* table, const uint32_t* ids, float* out, uint32_t rows, uint32_t width,
                           uint32_t vocab, uint32_t* status, cudaStream_t stream);
// peer_gather.cu - all-gather of column shards by peer stores.
int32_t launch_peer_gather(const DeviceContext& ctx, const float* local, uint64_t rows, uint64_t cols,
                           const uint64_t* peer_full, const uint64_t* peer_full_bf16, const uint64_t* peer_flags,
                           uint32_t rank, uint32_t world, uint32_t* state, uint32_t* status, cudaStream_t stream);
int32_t launch_argmax(const float* logits, uint32_t* out, uint32_t rows, uint32_t width, cudaStream_t stream);

}  // namespace b2
