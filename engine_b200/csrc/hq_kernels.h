// Internal launch interfaces shared by the .cu files (not part of the C ABI).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hanzoquant_b200.h"

namespace hq {

// ---- decode mat-vec (hq_gemv.cu) ----------------------------------------------
struct GemvParams {
  int format;
  int n, k, m;                 // m: dense activation rows (ignored when tiles != nullptr)
  int n_banks;                 // 1, or 2 = gate bank + up bank feeding one gated activation
  const void* w;
  const void* w_up;
  const void* scales;
  const void* scales_up;
  const void* bias;
  const void* bias_up;
  int bias_dtype;
  int64_t w_expert_stride;      // bytes between experts in w
  int64_t scale_expert_stride;  // scale elements between experts
  const void* x;
  int x_dtype;
  int64_t x_stride;             // elements
  void* y;
  int y_dtype;
  int64_t y_stride;             // elements
  // expert-indexed mode: work items of <= 8 sorted rows of one expert
  const int32_t* tiles;         // [n_items][2] = (expert, first sorted row)
  const int32_t* tile_count;    // device word holding n_items
  const int32_t* expert_bounds; // [E+1]
  const int32_t* x_rows;        // sorted row -> activation row (nullptr = identity)
  const int32_t* y_rows;        // sorted row -> output row (nullptr = identity)
  hq_act_args act;
  int32_t* status;
  void* workspace;              // optional caller scratch for split-K partial sums (Q8_0, Q4_K), zero between calls
  int64_t workspace_bytes;
};
int32_t launch_gemv(const GemvParams& p, int grid_y, cudaStream_t stream);
// scratch bytes the Q8_0 / Q4_K decode kernel wants for a dense [m, k] x [n, k] call (0 = none)
int64_t gemv_int8_workspace_bytes(int format, int64_t n, int64_t k, int64_t m);

// ---- grouped expert GEMM on tcgen05 (hq_grouped_gemm.cu) -----------------------------
struct GroupedParams {
  int format;
  int n, k, m;                 // m: dense rows (used when tiles == nullptr)
  const void* w;
  const void* w_up;            // second (up) bank for a fused gated activation, or nullptr
  const void* scales;          // MXFP4: e8m0 bytes [E, N, K/32]
  const void* scales_up;
  const void* bias;
  const void* bias_up;
  int bias_dtype;
  int64_t w_row_bytes;
  // block-FP8: per (expert, 128-row block) largest scale, and every scale relative to it
  const float* fp8_tile_scale;      // [E, NB]
  const float* fp8_tile_scale_up;
  const float* fp8_rel_scale;       // [E, NB, KB]
  const float* fp8_rel_scale_up;
  int fp8_nb, fp8_kb;
  const void* x;
  int x_dtype;
  int64_t x_stride;
  void* y;
  int y_dtype;
  int64_t y_stride;
  const int32_t* tiles;         // [n_tiles][2] = (expert, first sorted row), tiles of <= tile_rows rows
  const int32_t* tile_count;    // device word holding n_tiles
  int tile_rows;                // 128 or 256 tokens per tile
  bool weights_in_tmem;         // 128-token tiles only: take the kernel that expands the weights into tensor memory
  const int32_t* expert_bounds;
  const int32_t* x_rows;        // sorted row -> activation row (nullptr = identity)
  const int32_t* y_rows;        // sorted row -> output row (nullptr = identity)
  hq_act_args act;
  int32_t* status;
};
bool grouped_gemm_supported(int format, int64_t n, int64_t k);
int32_t launch_grouped_gemm(const GroupedParams& p, int max_tiles, cudaStream_t stream);
int32_t launch_fp8_scale_prepare(const float* scales, int64_t n_groups, int kb, float* tile_scale, float* rel_scale,
                                 cudaStream_t stream);

// ---- block-FP8 expert GEMM with FP8 activations on tcgen05 kind::f8f6f4 (hq_fp8_grouped.cu) --------------
struct Fp8GroupedParams {
  int n, k, m;                  // m: dense rows (used when expert_bounds == nullptr)
  int n_experts;
  const void* w;                // e4m3 codes [E, N, K]
  const float* w_scales;        // [E, N/128, K/128]
  const void* w_up;             // gated mode: the up bank (w is then the gate bank), same shape
  const float* w_up_scales;
  int fp8_nb, fp8_kb;
  const void* bias;
  const void* bias_up;
  int bias_dtype;
  const void* xq;               // e4m3 activation codes [n_rows, K], rows in expert-sorted order
  const float* xs;              // [n_rows, K/128] activation scales
  int64_t n_rows;               // rows of xq / xs (the tensor-map bound; rows beyond expert_bounds[E] are never used)
  void* y;                      // plain mode output
  int y_dtype;
  int64_t y_stride;
  bool y_vec_ok;                // set by the launcher: output row segments can be written with 16-byte stores
  uint8_t* hq;                  // gated mode output: e4m3 codes [n_rows, N] ...
  float* hs;                    // ... and scales [n_rows, N/128] of act(gate) * up, expert-sorted
  hq_act_args act;
  const int32_t* expert_bounds; // [E+1]; token tiles are cut from it inside the kernel
  const int32_t* y_rows;        // sorted row -> output row (nullptr = identity)
  int32_t* status;
  uint32_t spin_limit;          // polls per bounded wait (0 = default)
  int test_skip_producer;       // test hook: the TMA warp issues nothing, so every consumer wait runs out
  int load_burst;               // 128-column blocks the TMA warp requests together: 1, 2 or 4 (0 = default)
  int load_burst_prefetch_off;  // 1 = do not pull weight rows into L2 ahead of the operand copies
  int l2_prefetch;              // set by the launcher
};
bool fp8_grouped_supported(int64_t n, int64_t k);
int32_t launch_fp8_grouped(const Fp8GroupedParams& p, cudaStream_t stream);

// ---- MXFP4 expert GEMM with MXFP8 activations on tcgen05 kind::mxf8f6f4.block_scale (hq_mx_grouped.cu) ------
struct MxGroupedParams {
  int n, k, m;                  // m: dense rows (used when expert_bounds == nullptr)
  int n_experts;
  const void* w;                // packed e2m1 nibbles [E, N, K/2]
  const uint8_t* w_scales;      // e8m0 [E, N, K/32]
  const void* bias;             // [E, N] or nullptr
  int bias_dtype;
  const void* xq;               // e4m3 activation codes [n_rows, K], rows in expert-sorted order
  const uint8_t* xs;            // e8m0 [n_rows, K/32]
  int64_t n_rows;
  void* y;                      // plain mode: [rows, N]; gated mode without quantizer: [rows, N/2]
  int y_dtype;
  int64_t y_stride;
  int y_vec_ok;                 // y base and row pitch allow 16-byte stores (set by the launcher)
  uint8_t* hq;                  // gated mode with quantizer: e4m3 codes [n_rows, h_width] ...
  uint8_t* hs;                  // ... and e8m0 scales [n_rows, h_width/32] of the activated values
  int h_width;                  // N / 2 in gated mode
  hq_act_args act;              // HQ_ACT_NONE = plain; else rows interleave gate / up
  const int32_t* expert_bounds;
  const int32_t* y_rows;        // plain mode: sorted row -> output row (nullptr = identity)
  int32_t* status;
  uint32_t spin_limit;
  int test_skip_producer;
};
bool mx_grouped_supported(int64_t n, int64_t k);
int32_t launch_mx_grouped(const MxGroupedParams& p, cudaStream_t stream);
int32_t launch_mxfp8_quant_rows(const void* x, int x_dtype, int64_t x_stride, const int32_t* row_map,
                                const int32_t* n_valid, int64_t n_rows, int64_t k, uint8_t* codes, uint8_t* scales,
                                cudaStream_t stream);

// ---- dispatch tables (hq_dispatch.cu) -------------------------------------------
constexpr int kDispatchChunk = 1024;  // flat assignments per block
struct DispatchLayout {
  int64_t n_blocks;      // ceil(T*k / kDispatchChunk)
  int64_t off_counts;    // int32 words
  int64_t off_tiles8;    // int32 words, [max8][2]
  int64_t max_tiles8;
  int64_t off_tiles128;  // int32 words, [max128][2]
  int64_t max_tiles128;
  int64_t off_tiles256;  // int32 words, [max256][2]
  int64_t max_tiles256;
  int64_t total_words;
};
DispatchLayout dispatch_layout(int64_t n_tokens, int top_k, int n_experts);
int32_t launch_dispatch(const uint32_t* ids, int64_t n_tokens, int top_k, int n_experts, int32_t* bounds,
                        int32_t* sorted_assign, int32_t* sorted_token, int32_t* inv_perm, int32_t* ws,
                        cudaStream_t stream);

int32_t launch_dispatch_noalloc(const uint32_t* ids, int64_t n_tokens, int top_k, int n_experts, int32_t* bounds,
                                int32_t* sorted_assign, int32_t* sorted_token, int32_t* inv_perm,
                                cudaStream_t stream);

// ---- router (hq_router.cu) --------------------------------------------------------
int32_t launch_router(const void* logits, int dtype, int64_t n_rows, const hq_router_args& a, int n_group,
                      int topk_group, int group_mode, uint32_t* ids, float* weights, cudaStream_t stream);

// ---- elementwise / reduce (hq_elementwise.cu) --------------------------------------
int32_t launch_weighted_reduce(const void* y, int y_dtype, const float* w, const int32_t* row_map,
                               const void* addend, void* out, int out_dtype, int64_t n_tokens, int top_k,
                               int64_t hidden, cudaStream_t stream);
int32_t launch_fp8_vector_quant(const void* x, int x_dtype, int64_t n, uint8_t* codes, float* scales,
                                cudaStream_t stream);
int32_t launch_fp8_vector_dequant(const uint8_t* codes, const float* scales, int64_t n, void* out, int out_dtype,
                                  cudaStream_t stream);
int32_t launch_fp8_block_quant(const void* w, int w_dtype, int64_t rows, int64_t cols, int by, int bx,
                               uint8_t* codes, float* scales, cudaStream_t stream);
int32_t launch_fp8_block_dequant(const uint8_t* codes, const float* scales, int64_t rows, int64_t cols, int by,
                                 int bx, void* out, int out_dtype, cudaStream_t stream);
int32_t launch_fp8_quant_rows(const void* x, int x_dtype, int64_t x_stride, const int32_t* row_map,
                              const int32_t* n_valid, int64_t n_rows, int64_t k, uint8_t* codes, float* scales,
                              cudaStream_t stream);
int32_t launch_fp8_gated_quant_rows(const void* gu, int dtype, int64_t n_rows, int64_t width, const hq_act_args& act,
                                    uint8_t* codes, float* scales, cudaStream_t stream);
int32_t launch_convert(const void* src, int src_dtype, void* dst, int dst_dtype, int64_t n, int32_t* status,
                       cudaStream_t stream);
int32_t launch_gated_act(const void* gate, const void* up, int dtype, int64_t n, int interleaved,
                         const hq_act_args& act, void* out, cudaStream_t stream);


// ---- expert-parallel exchange helpers (hq_ep.cu) -------------------------------------
int32_t launch_ep_pack(const hq_ep_layout& l, const void* x, int x_dtype, const uint32_t* ids, const float* weights,
                       int64_t n_tokens, void* send, int32_t* back_map, cudaStream_t stream);
int32_t launch_ep_push(const void* send, void* const* peers, int world, int rank, int64_t slab_bytes,
                       cudaStream_t stream);
int32_t launch_ep_push_rows(const void* send, void* const* peers, int world, int rank, int rows_per_slab,
                            int64_t row_bytes, int always_from, const int32_t* back_map, int n_tokens,
                            const uint32_t* ids, int top_k, cudaStream_t stream);
int32_t launch_ep_barrier(int32_t* const* flags, int world, int rank, int32_t* seq_counter, uint32_t spin_limit,
                          int32_t* status, cudaStream_t stream);
int32_t launch_ep_unpack_meta(const hq_ep_layout& l, const void* recv, uint32_t* ids, float* weights,
                              cudaStream_t stream);
int32_t launch_fp8_gather_rows(const void* src_codes, int64_t src_code_stride, const void* src_scales,
                               int64_t src_scale_stride, const int32_t* row_map, const int32_t* n_valid,
                               int64_t n_rows, int64_t k, uint8_t* codes, float* scales, cudaStream_t stream);

// ---- unquantized decode mat-vec (hq_gemv_dense.cu) -----------------------------------
int32_t launch_dense_gemv(const void* w, int w_dtype, int64_t n, int64_t k, const void* bias, int bias_dtype,
                          const void* x, int x_dtype, int64_t x_stride, void* y, int y_dtype, int64_t y_stride, int m,
                          cudaStream_t stream);

// ---- tensor-core issue-rate probe (hq_probe.cu) ---------------------------------------
int32_t launch_probe_mma(int kind, int n_dim, int iters, int32_t* status, double* flops_out, cudaStream_t stream);

}  // namespace hq
