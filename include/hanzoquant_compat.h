/*
 * Reference-named entry points: the `extern "C"` symbols hanzo-quant and hanzo-engine declare for this path, with
 * their argument lists unchanged, each a thin call into the hq_* entry points of hanzoquant_b200.h.  With these
 * in libhanzoquant_b200 the existing Rust `ffi.rs` files link unchanged (hanzo-quant/build.rs:63-121 links
 * `hanzoquant` + `cudart` + `stdc++`).  Conventions are the reference's: void return, device pointers, work is
 * enqueued on `stream`, nothing synchronises; an argument error is printed to stderr once per symbol and the
 * call does nothing.
 *
 * Scratch.  The reference's indexed / grouped MoE kernels take ids and build nothing; the kernels behind these
 * shims need the dispatch tables first.  The shims keep them in a fixed array inside the library (about 1 MB per
 * GPU) for calls of up to 65536 assignments and 512 experts; larger calls take stream-ordered scratch
 * (cudaMallocAsync / cudaFreeAsync on `stream`).  Calls share the fixed array, so keep them on one stream, as
 * the reference's single-stream discipline does.
 *
 * Q8_1.  The reference quantizes activations to int8 Q8_1 blocks in a scratch buffer and hands that buffer to the
 * mat-vec (hanzo-quant/src/gguf/fast_mmvq.rs:343-368).  That step costs ~1e-2 of error and is not reproduced: the
 * `..._quantize_q8_1_...` shims record which activation buffer belongs to the scratch pointer (on the host), and
 * the mat-vec shim that receives the scratch pointer reads the original activations.  Both calls must be issued
 * back to back from one thread with the activation buffer still alive, as the reference's call sites do.
 */
#ifndef HANZOQUANT_COMPAT_H
#define HANZOQUANT_COMPAT_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* hanzo-quant/src/gguf/ffi.rs:251-262.  sorted_token_ids = flat assignment index, sorted_source_ids = token
 * index, both in the stable (expert, token, slot) order; expert_counts / expert_cursors are not used. */
void launch_moe_dispatch(const int32_t* topk_ids, int32_t* expert_bounds, int32_t* sorted_token_ids,
                         int32_t* sorted_source_ids, int32_t total_assignments, int32_t num_experts, int32_t topk,
                         int32_t* expert_counts, int32_t* expert_cursors, void* stream);
/* hanzo-quant/src/gguf/ffi.rs:264-282: inputs f32 [T*k, H] in flat assignment order, weights f32 [T, k]. */
void launch_moe_weighted_reduce_flat(const float* inputs, const float* topk_weights, float* outputs,
                                     int32_t num_tokens, int32_t hidden, int32_t topk, void* stream);
void launch_moe_weighted_reduce_flat_bf16(const float* inputs, const float* topk_weights, void* outputs,
                                          int32_t num_tokens, int32_t hidden, int32_t topk, void* stream);

/* hanzo-quant/src/gguf/fast_mmvq.rs:107-148, :343-368 (declared in gguf/ffi.rs).  vy is the Q8_1 scratch. */
void launch_mmvq_gguf_quantize_q8_1_bf16(const void* x, void* vy, int32_t kx, int32_t kx_padded, int32_t num_rows,
                                         void* stream);
void launch_mmvq_gguf_quantize_q8_1_f16(const void* x, void* vy, int32_t kx, int32_t kx_padded, int32_t num_rows,
                                        void* stream);
void launch_mmvq_gguf_quantize_q8_1_f32(const void* x, void* vy, int32_t kx, int32_t kx_padded, int32_t num_rows,
                                        void* stream);
#define HQ_COMPAT_PLAIN(name)                                                                               \
  void name(const void* vx, const void* vy, void* dst, int32_t ncols_x, int32_t nrows_x, int32_t stride_col_y, \
            int32_t stride_col_dst, int32_t b_size, void* stream)
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q8_0_bf16_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q8_0_f16_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q8_0_f32_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q4_k_bf16_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q4_k_f16_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q4_k_f32_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q6_k_bf16_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q6_k_f16_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q6_k_f32_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q5_k_bf16_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q5_k_f16_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q5_k_f32_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q4_0_bf16_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q4_0_f16_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q4_0_f32_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q5_0_bf16_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q5_0_f16_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q5_0_f32_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q4_1_bf16_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q4_1_f16_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q4_1_f32_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q5_1_bf16_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q5_1_f16_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q5_1_f32_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q2_k_bf16_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q2_k_f16_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q2_k_f32_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q3_k_bf16_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q3_k_f16_plain);
HQ_COMPAT_PLAIN(launch_mmvq_gguf_q3_k_f32_plain);

/* hanzo-quant/src/gguf/ffi.rs:53-81 and the indexed MoE forward (gguf/ffi.rs:84-247; call site gguf/cuda.rs:213-440):
 * all_inputs is the Q8_1 scratch of a preceding launch_quantize_q8_1* call, outputs f32 [batch, topk, n]. */
void launch_quantize_q8_1(const float* x, void* vy, int32_t kx, int32_t kx_padded, int32_t num_blocks_x,
                          int32_t num_rows, void* stream);
void launch_quantize_q8_1_bf16(const void* x, void* vy, int32_t kx, int32_t kx_padded, int32_t num_rows, void* stream);
void launch_quantize_q8_1_f16(const void* x, void* vy, int32_t kx, int32_t kx_padded, int32_t num_rows, void* stream);
void launch_indexed_moe_forward_q4k_q8_1(const void* all_weights, const void* all_inputs, const uint32_t* indices,
                                         float* all_outputs, int32_t n, int32_t k, int32_t batch, int32_t topk,
                                         int32_t k_padded, int32_t input_dim1, void* stream);
void launch_indexed_moe_forward_q8_0_q8_1(const void* all_weights, const void* all_inputs, const uint32_t* indices,
                                          float* all_outputs, int32_t n, int32_t k, int32_t batch, int32_t topk,
                                          int32_t k_padded, int32_t input_dim1, void* stream);

/* hanzo-quant/src/blockwise_fp8/ffi.rs:88-150 (weight-only FP8: 16-bit activations, output in their dtype). */
void launch_fp8_matmul_f16(const void* input, const void* weight, const float* weight_scale, void* output, int32_t m,
                           int32_t n, int32_t k, int32_t scale_row_stride, int32_t block_size_y,
                           int32_t block_size_x, void* stream);
void launch_fp8_matmul_bf16(const void* input, const void* weight, const float* weight_scale, void* output, int32_t m,
                            int32_t n, int32_t k, int32_t scale_row_stride, int32_t block_size_y,
                            int32_t block_size_x, void* stream);
void launch_fp8_indexed_moe_gemm_f16(const void* input, const void* weights, const float* weight_scales,
                                     const uint32_t* indices, void* output, int32_t num_tokens, int32_t topk,
                                     int32_t num_experts, int32_t n, int32_t k, int32_t scale_row_stride,
                                     int32_t block_size_y, int32_t block_size_x, bool input_has_topk_dim,
                                     void* stream);
void launch_fp8_indexed_moe_gemm_bf16(const void* input, const void* weights, const float* weight_scales,
                                      const uint32_t* indices, void* output, int32_t num_tokens, int32_t topk,
                                      int32_t num_experts, int32_t n, int32_t k, int32_t scale_row_stride,
                                      int32_t block_size_y, int32_t block_size_x, bool input_has_topk_dim,
                                      void* stream);
/* hanzo-quant/src/blockwise_fp8/ffi.rs:9-86: [height, width] weights, scale grid rows of scale_stride floats. */
void launch_dequant_fp8_blockwise_kernel_f32(const void* d_weight, const float* d_scale, void* d_output,
                                             int32_t weight_height, int32_t weight_width, int32_t weight_row_stride,
                                             int32_t scale_stride, int32_t weight_block_size_y,
                                             int32_t weight_block_size_x, void* stream);
void launch_dequant_fp8_blockwise_kernel_f16(const void* d_weight, const float* d_scale, void* d_output,
                                             int32_t weight_height, int32_t weight_width, int32_t weight_row_stride,
                                             int32_t scale_stride, int32_t weight_block_size_y,
                                             int32_t weight_block_size_x, void* stream);
void launch_dequant_fp8_blockwise_kernel_bf16(const void* d_weight, const float* d_scale, void* d_output,
                                              int32_t weight_height, int32_t weight_width, int32_t weight_row_stride,
                                              int32_t scale_stride, int32_t weight_block_size_y,
                                              int32_t weight_block_size_x, void* stream);
void launch_quant_fp8_blockwise_kernel_f32(const void* d_input, void* d_weight, float* d_scale, int32_t weight_height,
                                           int32_t weight_width, int32_t weight_row_stride, int32_t scale_stride,
                                           int32_t weight_block_size_y, int32_t weight_block_size_x, void* stream);
void launch_quant_fp8_blockwise_kernel_f16(const void* d_input, void* d_weight, float* d_scale, int32_t weight_height,
                                           int32_t weight_width, int32_t weight_row_stride, int32_t scale_stride,
                                           int32_t weight_block_size_y, int32_t weight_block_size_x, void* stream);
void launch_quant_fp8_blockwise_kernel_bf16(const void* d_input, void* d_weight, float* d_scale, int32_t weight_height,
                                            int32_t weight_width, int32_t weight_row_stride, int32_t scale_stride,
                                            int32_t weight_block_size_y, int32_t weight_block_size_x, void* stream);

/* hanzo-quant/src/vector_fp8/ffi.rs:8-62 (1 x 128 groups over a flat tensor). */
void launch_dequant_fp8_vector_kernel_f32(const void* d_weight, const float* d_scale, void* d_output,
                                          size_t num_elements, void* stream);
void launch_dequant_fp8_vector_kernel_f16(const void* d_weight, const float* d_scale, void* d_output,
                                          size_t num_elements, void* stream);
void launch_dequant_fp8_vector_kernel_bf16(const void* d_weight, const float* d_scale, void* d_output,
                                           size_t num_elements, void* stream);
void launch_quant_fp8_vector_kernel_f32(const void* d_input, void* d_weight, float* d_scale, size_t num_elements,
                                        void* stream);
void launch_quant_fp8_vector_kernel_f16(const void* d_input, void* d_weight, float* d_scale, size_t num_elements,
                                        void* stream);
void launch_quant_fp8_vector_kernel_bf16(const void* d_input, void* d_weight, float* d_scale, size_t num_elements,
                                         void* stream);

/* hanzo-quant/src/mxfp4/ffi.rs:7-160.  The `wmma` names are the same computation. */
#define HQ_COMPAT_MXFP4_MATMUL(name)                                                                              \
  void name(const void* input, const uint8_t* weight, const uint8_t* weight_scale, const void* bias, void* output, \
            int32_t m, int32_t n, int32_t k, bool has_bias, void* stream)
HQ_COMPAT_MXFP4_MATMUL(launch_mxfp4_matmul_f16);
HQ_COMPAT_MXFP4_MATMUL(launch_mxfp4_matmul_bf16);
HQ_COMPAT_MXFP4_MATMUL(launch_mxfp4_matmul_wmma_f16);
HQ_COMPAT_MXFP4_MATMUL(launch_mxfp4_matmul_wmma_bf16);
#define HQ_COMPAT_MXFP4_MOE(name)                                                                              \
  void name(const void* input, const uint8_t* weights, const uint8_t* weight_scales, const void* biases,       \
            const uint32_t* indices, void* output, int32_t num_tokens, int32_t topk, int32_t num_experts,       \
            int32_t n, int32_t k, bool has_bias, bool input_has_topk_dim, void* stream)
HQ_COMPAT_MXFP4_MOE(launch_mxfp4_indexed_moe_gemm_f16);
HQ_COMPAT_MXFP4_MOE(launch_mxfp4_indexed_moe_gemm_bf16);
HQ_COMPAT_MXFP4_MOE(launch_mxfp4_moe_grouped_gemm_f16);
HQ_COMPAT_MXFP4_MOE(launch_mxfp4_moe_grouped_gemm_bf16);
HQ_COMPAT_MXFP4_MOE(launch_mxfp4_moe_grouped_gemm_wmma_f16);
HQ_COMPAT_MXFP4_MOE(launch_mxfp4_moe_grouped_gemm_wmma_bf16);
int32_t mxfp4_get_max_smem_optin(void);

/* hanzo-engine/src/cuda/ffi.rs:466-520 (kernel hanzo-engine/src/cuda/sort.cu:1048-1201): weights f32, ids u32,
 * selection_bias / expert_scale f32 [n_experts] or NULL; `stream` is the CUstream as an integer. */
#define HQ_COMPAT_ROUTER(name)                                                                                     \
  void name(const void* logits, void* weights, void* ids, const void* selection_bias, const void* expert_scale,    \
            int32_t nrows, int32_t n_experts, int32_t top_k, int32_t score_mode, int32_t weight_mode,               \
            bool renormalize, bool clamp_logits, float clamp_min, float clamp_max, float norm_min, float output_scale, \
            int64_t stream)
HQ_COMPAT_ROUTER(moe_router_topk_f32);
HQ_COMPAT_ROUTER(moe_router_topk_bf16);
HQ_COMPAT_ROUTER(moe_router_topk_f16);

/* hanzo-quant/src/utils/ffi.rs:177-232 (kernels/ops/ops.cu:335-360, :482-512). */
void gptoss_swiglu_f16(const void* gate, const void* up, void* output, uint32_t n, float alpha, float limit, void* stream);
void gptoss_swiglu_bf16(const void* gate, const void* up, void* output, uint32_t n, float alpha, float limit, void* stream);
void gptoss_swiglu_f32(const void* gate, const void* up, void* output, uint32_t n, float alpha, float limit, void* stream);
void gptoss_swiglu_interleaved_f16(const void* gate_up, void* output, uint32_t n, uint32_t intermediate_size,
                                   float alpha, float limit, void* stream);
void gptoss_swiglu_interleaved_bf16(const void* gate_up, void* output, uint32_t n, uint32_t intermediate_size,
                                    float alpha, float limit, void* stream);
void gptoss_swiglu_interleaved_f32(const void* gate_up, void* output, uint32_t n, uint32_t intermediate_size,
                                   float alpha, float limit, void* stream);
/* hanzo-quant/src/utils/ffi.rs:274-297: output = act(a) * b; activation 0 = SiLU (GluActivationType,
 * hanzo-quant/src/utils/ops.rs:2576-2584); the other activations of that enum are not on this path and are refused. */
void fused_glu_f16(const void* a, const void* b, void* output, uint32_t n, int32_t activation, void* stream);
void fused_glu_bf16(const void* a, const void* b, void* output, uint32_t n, int32_t activation, void* stream);
void fused_glu_f32(const void* a, const void* b, void* output, uint32_t n, int32_t activation, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* HANZOQUANT_COMPAT_H */
