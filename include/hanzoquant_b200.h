/*
 * libhanzoquant_b200 -- C ABI of the B200 (sm_100a) quantized-linear and
 * sparse-MoE expert path.
 *
 * This is the boundary a host binding (Rust FFI, ctypes, cgo ...) links
 * against.  It replaces the `extern "C" launch_*` families that hanzo-quant
 * declares in hanzo-quant/src/gguf/ffi.rs, blockwise_fp8/ffi.rs,
 * vector_fp8/ffi.rs, mxfp4/ffi.rs, utils/ffi.rs and
 * hanzo-engine/src/cuda/ffi.rs:466-520; each entry point below names the
 * reference interface it stands in for.
 *
 * Conventions
 *   - plain pointers and sizes only; every pointer is a DEVICE pointer unless
 *     the parameter name ends in `_host`;
 *   - the caller owns every buffer, including scratch (`*_workspace_bytes`
 *     tells how much); nothing here allocates unless stated otherwise;
 *   - all work is enqueued on the `stream` argument (a cudaStream_t passed as
 *     void*), nothing synchronises the host;
 *   - every call returns an int32 status: 0 = enqueued, < 0 = argument error
 *     found on the host before any launch (see HQ_ERR_*).  A kernel that gave
 *     up on a bounded wait writes a code into the optional device status word
 *     (int32[4], see hq_status_*), it never spins forever.
 *   - there is no CPU fallback: without a CUDA device the calls fail with
 *     HQ_ERR_CUDA.
 */
#ifndef HANZOQUANT_B200_H
#define HANZOQUANT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* 2: adds the caller-scratch linear call, the FP8 row quantizers and FP8-activation calls, and the one-call
 * MoE layer; every version-1 entry point keeps its signature.
 * 3: adds the status-reporting conversion, the fused FP8 expert block, the expert-parallel pack / unpack calls,
 * the fused dense decode calls, more GGML types and the reference-named compatibility symbols; every version-2
 * entry point keeps its signature. */
#define HQ_ABI_VERSION 3

/* status codes */
#define HQ_OK 0
#define HQ_ERR_NULL (-1)        /* required pointer is NULL */
#define HQ_ERR_SHAPE (-2)       /* size not supported (divisibility, range) */
#define HQ_ERR_ALIGN (-3)       /* pointer or stride not 16-byte aligned */
#define HQ_ERR_FORMAT (-4)      /* unknown format / dtype / mode code */
#define HQ_ERR_CUDA (-5)        /* CUDA runtime error at launch (no device, bad config) */
#define HQ_ERR_WORKSPACE (-6)   /* workspace missing or too small */
#define HQ_ERR_TOO_LARGE (-7)   /* size beyond a stated fixed maximum */

/* codes a kernel may leave in word [0] of the device status buffer (int32[4]: code, blockIdx.x, blockIdx.y,
 * tag); the first one sticks until the caller clears the buffer */
#define HQ_DEV_OK 0
#define HQ_DEV_WAIT_TIMEOUT 1  /* a bounded wait ran out; the kernel skipped the rest of its work */
#define HQ_DEV_BAD_INDEX 2     /* an index read from a caller table was out of range and was skipped */
#define HQ_DEV_SCALE_RANGE 3   /* MXFP4 on the tensor-core path: a block scale outside 2^-14 .. 2^13 (e8m0 113 .. 140,
                                  or 0) was expanded as zero; run such banks with HQ_CFG_MOE_TENSOR_MIN_ROWS huge */
#define HQ_DEV_F16_RANGE 4     /* an activation beyond +-65504 was clamped while being converted to f16 */

/* weight formats (hanzo-quant: GgufMatMul Q8_0 / Q4_K, BlockwiseFP8Linear, MXFP4Layer) */
#define HQ_FMT_Q8_0 0       /* GGUF block_q8_0 {half d; int8 qs[32]}, 34 B / 32 weights   */
#define HQ_FMT_Q4_K 1       /* GGUF block_q4_K, 144 B / 256 weights                        */
#define HQ_FMT_FP8_BLOCK 2  /* e4m3 codes [N,K] + f32 scale[ceil(N/128), ceil(K/128)]      */
#define HQ_FMT_MXFP4 3      /* e2m1 nibbles [N,K/2] (low nibble = even k) + e8m0 [N,K/32]  */
#define HQ_FMT_Q6_K 4       /* GGUF block_q6_K, 210 B / 256 weights   (formats 4-7: plain calls, or a gate and an */
#define HQ_FMT_Q5_K 5       /* GGUF block_q5_K, 176 B / 256 weights    up bank with a gated activation; a decode   */
#define HQ_FMT_Q4_0 6       /* GGUF block_q4_0, 18 B / 32 weights      kernel up to 8 rows, the tensor-core GEMM   */
#define HQ_FMT_Q5_0 7       /* GGUF block_q5_0, 22 B / 32 weights      from HQ_CFG_*_TENSOR_MIN_ROWS rows on)      */
#define HQ_FMT_Q4_1 8       /* GGUF block_q4_1, 20 B / 32 weights     (formats 8-11: as 4-7)                      */
#define HQ_FMT_Q5_1 9       /* GGUF block_q5_1, 24 B / 32 weights                                                  */
#define HQ_FMT_Q2_K 10      /* GGUF block_q2_K, 84 B / 256 weights                                                 */
#define HQ_FMT_Q3_K 11      /* GGUF block_q3_K, 110 B / 256 weights                                                */

/* element types of activations, outputs, biases */
#define HQ_DT_F32 0
#define HQ_DT_F16 1
#define HQ_DT_BF16 2

/* router codes: hanzo-engine/src/ops.rs:194-222 */
#define HQ_SCORE_RAW 0
#define HQ_SCORE_SOFTMAX 1
#define HQ_SCORE_SIGMOID 2
#define HQ_WEIGHT_SCORE 0
#define HQ_WEIGHT_SOFTMAX 1
#define HQ_WEIGHT_SIGMOID 2

/* gated activation fused behind a gate/up projection */
#define HQ_ACT_NONE 0
#define HQ_ACT_SWIGLU 1        /* silu(gate) * up, optional clamp (hanzo-engine/src/ops.rs:3545-3556) */
#define HQ_ACT_GPTOSS 2        /* (clamp(up,+-L)+1) * g*sigmoid(alpha*g), g=min(gate,L) (models/gpt_oss.rs:116-135) */

/* A quantized weight matrix [N, K] or expert bank [E, N, K], row-major, in the
 * exact byte layout the reference keeps on the device (hanzo-quant
 * kernels/mmvq_gguf/mmvq_gguf.cu:134-170, src/blockwise_fp8/mod.rs:24-30,
 * src/mxfp4/mod.rs:29-41).  Expert e starts at data + e*N*row_bytes. */
typedef struct hq_weight {
  int32_t format;      /* HQ_FMT_* */
  int32_t n_experts;   /* 1 for a dense layer */
  int64_t n;           /* output features */
  int64_t k;           /* input features */
  const void* data;    /* block bytes / e4m3 codes / packed nibbles */
  const void* scales;  /* FP8: f32 [E, ceil(N/128), ceil(K/128)]; MXFP4: u8 [E, N, K/32]; else NULL */
  const void* bias;    /* optional [E, N] in bias_dtype, or NULL */
  int32_t bias_dtype;  /* HQ_DT_* */
  int32_t reserved;
  /* FP8 only, optional: tables written once per layer by hq_fp8_scale_prepare.  With them the
   * prefill-sized calls run on the tensor cores; without them every call takes the decode kernel. */
  const void* fp8_tile_scale;  /* f32 [E, ceil(N/128)] */
  const void* fp8_rel_scale;   /* f32 [E, ceil(N/128), ceil(K/128)] */
} hq_weight;

/* parameters of a gated activation (HQ_ACT_*) */
typedef struct hq_act_args {
  int32_t act;          /* HQ_ACT_* */
  int32_t has_limit;    /* SWIGLU: clamp gate<=limit, |up|<=limit first */
  float limit;          /* GPTOSS: L */
  float alpha;          /* GPTOSS: alpha */
} hq_act_args;

/* ---- library ------------------------------------------------------------ */
int32_t hq_abi_version(void);
const char* hq_error_string(int32_t code);
/* Reads the 4-word device status buffer after synchronising `stream`
 * (test / debug helper; the hot path never calls it). */
int32_t hq_status_read(const int32_t* status_dev, int32_t out_host[4], void* stream);

/* Tuning knobs (process-wide, read at call time).  HQ_CFG_MOE_TENSOR_MIN_ROWS: expert projections run on the
 * tensor-core grouped GEMM when n_tokens*top_k >= value * n_experts (default 8; 0 = always when the shape
 * allows, a huge value = never).  HQ_CFG_DENSE_TENSOR_MIN_ROWS: same switch for hq_linear_forward's m
 * (default 9).  Shapes the grouped GEMM does not cover (Q8_0, K % 64 != 0) always take the decode kernel. */
#define HQ_CFG_MOE_TENSOR_MIN_ROWS 0
#define HQ_CFG_DENSE_TENSOR_MIN_ROWS 1
/* HQ_CFG_SPIN_LIMIT: polls a kernel spends on one bounded wait before it gives up, leaves HQ_DEV_WAIT_TIMEOUT in
 * the status word and stops storing results (default 1 << 22; read by the FP8 expert GEMM).
 * HQ_CFG_TEST_SKIP_PRODUCER: test hook, 0 by default.  With 1 the FP8 expert GEMM's copy-issuing warp issues
 * nothing, so every wait of the other warps runs out: the way to see the time-out path return without anything
 * left in flight (no copy and no MMA is issued in that launch). */
#define HQ_CFG_SPIN_LIMIT 2
#define HQ_CFG_TEST_SKIP_PRODUCER 3
/* HQ_CFG_FP8_LOAD_BURST: 128-column blocks the FP8 expert GEMM requests from memory together (1, 2 or 4; default
 * 2): more of each weight row is read in one go, at the cost of pipeline depth. */
#define HQ_CFG_FP8_LOAD_BURST 4
/* HQ_CFG_FP8_L2_PREFETCH: 1 = the FP8 expert GEMM pulls 1 KiB of every weight row into L2 sixteen blocks ahead of
 * the operand copies; 0 (default) = off (it measured slower on the DeepSeek-V3-shaped layer). */
#define HQ_CFG_FP8_L2_PREFETCH 5
int32_t hq_config_set(int32_t key, int64_t value);
int64_t hq_config_get(int32_t key);

/* ---- dense quantized linear: QuantMethod::forward ------------------------
 * y[m, n] = sum_k x[m, k] * dequant(W)[n, k] (+ bias[n]).
 * Replaces launch_mmvq_gguf_quantize_q8_1_* + launch_mmvq_gguf_{q4_k,q8_0}_*_plain
 * (hanzo-quant/src/gguf/fast_mmvq.rs:107-148, :343-368), launch_fp8_matmul_*
 * (blockwise_fp8/ffi.rs) and launch_mxfp4_matmul_* (mxfp4/ffi.rs).  Activations
 * do not go through the reference's single int8 term (its Q8_1 step): for Q4_K,
 * FP8 and MXFP4 x is used at 16-bit precision; for Q8_0 every 128-element group
 * of x is split into two int8 terms (error below max|x| / 32000 per element) so
 * the block codes can enter the integer MMA unconverted.  Products accumulate in
 * f32.
 * x: [m, k] with row stride x_stride elements; y: [m, n] with row stride y_stride.
 * Requires K % 256 == 0 for Q8_0/Q4_K, K % 128 == 0 for FP8, K % 32 == 0 for
 * MXFP4; x rows 16-byte aligned.  Any m >= 0 (rows are processed 8 at a time
 * on the decode path). */
int32_t hq_linear_forward(const hq_weight* w, const void* x, int32_t x_dtype, int64_t x_stride, void* y,
                          int32_t y_dtype, int64_t y_stride, int64_t m, int32_t* status_dev, void* stream);

/* The same call with caller-owned scratch, the counterpart of the Q8_1 activation buffer the reference's
 * host side allocates for launch_mmvq_gguf_quantize_q8_1_* (hanzo-quant/src/gguf/fast_mmvq.rs:107-148).
 * With it the Q8_0 / Q4_K decode kernel splits K across CTAs when K is too long for a CTA to keep its
 * activations staged (partial sums meet in the scratch and are added in a fixed order: results stay
 * bit-reproducible).  hq_linear_workspace_bytes gives the size for (w, m), 0 when the call would not use
 * any.  The scratch must be 256-byte aligned and zero-filled once before its first use; every call leaves
 * its arrival counters (the first 1024 bytes) at zero again and overwrites the rest.  One scratch serves
 * one stream at a time.  workspace == NULL is allowed and equals hq_linear_forward. */
int64_t hq_linear_workspace_bytes(const hq_weight* w, int64_t m);
int32_t hq_linear_forward_ws(const hq_weight* w, const void* x, int32_t x_dtype, int64_t x_stride, void* y,
                             int32_t y_dtype, int64_t y_stride, int64_t m, void* workspace, int64_t workspace_bytes,
                             int32_t* status_dev, void* stream);

/* ---- fused dense decode set ---------------------------------------------------
 * hq_linear_glu_forward: y[m, n] = act(x . Wgate^T) * (x . Wup^T) in one launch, the two mat-vecs sharing the staged
 * activations.  Replaces launch_mmvq_gguf_{q4_k,q8_0}_*_fused_glu (QuantMethod-level try_fused_quantized_gate_up,
 * hanzo-quant/src/lib.rs:1116-1160; gguf/fast_mmvq.rs:463-700; kernel mmvq_gguf.cu:788-900).  w_up NULL = the rows
 * of w_gate interleave gate / up and y has n / 2 columns.  Any format; m >= 9 takes the tensor-core kernel when the
 * activations are f16.
 * hq_linear_qkv_forward: the three attention projections of one activation in one call (three back-to-back
 * launches; the reference's fused_qkv kernel, gguf/fast_mmvq.rs:702-925, saves the same host work).  q / k / v are
 * [m, n_q] / [m, n_k] / [m, n_v], dense.
 * hq_dense_gemv: unquantized weights W [n, k] in f16 / bf16 / f32, 1..8 activation rows: launch_gemv_{bf16,f16,f32}
 * (hanzo-quant/src/gemv/mod.rs:120-185, kernels/gemv/gemv.cu:51-282).  k % 8 == 0, W rows 16-byte aligned. */
int32_t hq_linear_glu_forward(const hq_weight* w_gate, const hq_weight* w_up, const hq_act_args* act, const void* x,
                              int32_t x_dtype, int64_t x_stride, void* y, int32_t y_dtype, int64_t y_stride, int64_t m,
                              int32_t* status_dev, void* stream);
int32_t hq_linear_qkv_forward(const hq_weight* w_q, const hq_weight* w_k, const hq_weight* w_v, const void* x,
                              int32_t x_dtype, int64_t x_stride, void* q, void* k, void* v, int32_t y_dtype,
                              int64_t m, int32_t* status_dev, void* stream);
int32_t hq_dense_gemv(const void* w, int32_t w_dtype, int64_t n, int64_t k, const void* bias, int32_t bias_dtype,
                      const void* x, int32_t x_dtype, int64_t x_stride, void* y, int32_t y_dtype, int64_t y_stride,
                      int64_t m, void* stream);

/* ---- router: moe_router_topk ---------------------------------------------
 * Replaces moe_router_topk_{f32,bf16,f16} (hanzo-engine/src/cuda/ffi.rs:466-520,
 * kernel hanzo-engine/src/cuda/sort.cu:1048-1201) with the canonical tie-break
 * (score DESC, expert id ASC; hanzo-engine/src/ops.rs:241-251) always on.
 * logits [n_rows, n_experts]; ids_out uint32 [n_rows, top_k] in descending
 * selection order; weights_out f32 [n_rows, top_k].  selection_bias /
 * expert_scale: f32 [n_experts] or NULL.  n_experts <= 1024, top_k <= 32. */
typedef struct hq_router_args {
  int32_t n_experts, top_k;
  int32_t score_mode, weight_mode;   /* HQ_SCORE_*, HQ_WEIGHT_* */
  int32_t renormalize, clamp_logits;
  float clamp_min, clamp_max;
  float norm_min, output_scale;
  const float* selection_bias;
  const float* expert_scale;
} hq_router_args;
int32_t hq_router_topk(const void* logits, int32_t logits_dtype, int64_t n_rows, const hq_router_args* args,
                       uint32_t* ids_out, float* weights_out, void* stream);
/* Group-limited selection of the DeepSeek routers (hanzo-engine/src/models/deepseek3.rs:623-690): the experts form
 * n_group contiguous groups; a group's score is the sum of its two best selection scores (group_score_mode 0,
 * "noaux_tc") or its best one (1, "group_limited_greedy"); only the topk_group best groups stay selectable (the
 * selection score of every other expert becomes 0, as the reference's mask multiply does), then the usual top-k.
 * Ties between groups go to the lower group.  n_group <= 32, n_experts % n_group == 0. */
int32_t hq_router_topk_grouped(const void* logits, int32_t logits_dtype, int64_t n_rows, const hq_router_args* args,
                               int32_t n_group, int32_t topk_group, int32_t group_score_mode, uint32_t* ids_out,
                               float* weights_out, void* stream);

/* ---- dispatch tables: moe_dispatch_build ----------------------------------
 * Replaces launch_moe_dispatch (hanzo-quant/src/gguf/ffi.rs:251-262; kernels
 * moe_grouped.cu:632-676) with a deterministic, stable permutation: flat
 * assignment indices t*top_k+s sorted by expert id, ties in (t, s) order -- the
 * order of the reference's host grouping (hanzo-quant/src/mxfp4/ops.rs:237-271).
 * Outputs: expert_bounds int32 [E+1]; sorted_assign int32 [T*k] (flat index);
 * sorted_token int32 [T*k] (token index); inv_perm int32 [T*k] (flat index ->
 * sorted position).  Also fills the tile lists for the expert GEMMs in the
 * workspace (see hq_moe_dispatch_workspace_bytes).
 * An id outside [0, n_experts) -- a padding slot such as 0xFFFFFFFF -- is skipped:
 * it gets no sorted row, expert_bounds[E] counts only the routed assignments (the
 * tail of sorted_assign / sorted_token beyond it is left unwritten), and its
 * inv_perm entry is -1, which hq_moe_weighted_reduce reads as "adds nothing". */
int64_t hq_moe_dispatch_workspace_bytes(int64_t n_tokens, int32_t top_k, int32_t n_experts);
int32_t hq_moe_dispatch_build(const uint32_t* ids, int64_t n_tokens, int32_t top_k, int32_t n_experts,
                              int32_t* expert_bounds, int32_t* sorted_assign, int32_t* sorted_token,
                              int32_t* inv_perm, void* workspace, int64_t workspace_bytes, void* stream);

/* Same tables for hosts that have no device memory to spare for a workspace and may not allocate any:
 * engines whose own pool already owns all of HBM, or code that runs where the CUDA runtime must not be
 * asked for memory.  This entry point has no counterpart in the reference.  The scratch it needs sits in a
 * fixed array inside the library (about 220 KB per GPU, held until the process exits), so it only accepts
 * n_tokens*top_k <= 65536 and n_experts <= 512 and answers HQ_ERR_TOO_LARGE beyond that.  It calls no
 * allocator of any kind.  The first call on a device looks up the array's device address (with lazy module
 * loading that is also when the driver backs the array with memory, so it can fail with HQ_ERR_CUDA on a GPU
 * that is already full): make that first call at start-up, before the host's own pool claims the rest of the
 * memory, and outside any stream capture.  `stream` must belong to the device that is current when the call is
 * made (the address is looked up for the current device).  All calls share the one array: calls that run at the same time
 * on one GPU corrupt each other, so keep them on one stream or order them yourself.  (The tile lists the
 * expert projections consume stay inside that array; this variant is for callers that only need the
 * four tables.) */
int32_t hq_moe_dispatch_build_noalloc(const uint32_t* ids, int64_t n_tokens, int32_t top_k, int32_t n_experts,
                                      int32_t* expert_bounds, int32_t* sorted_assign, int32_t* sorted_token,
                                      int32_t* inv_perm, void* stream);

/* ---- expert projection: QuantMethod::gather_forward ------------------------
 * out[t, s, :] = dequant(W[ids[t,s]]) . x_row (+ bias[ids[t,s]]), out [T, k, N].
 * x_layout: HQ_ROWS_PER_TOKEN = [T, K], one row per token shared by its k slots;
 * HQ_ROWS_PER_SLOT = [T, k, K] in (token, slot) order; HQ_ROWS_SORTED = [T*k, K]
 * in expert-sorted order (the order of sorted_assign).  out_layout:
 * HQ_ROWS_PER_SLOT = [T, k, N] (what gather_forward returns) or HQ_ROWS_SORTED
 * (kept expert-sorted for a following down projection).  Replaces launch_indexed_moe_forward_{q4k,q8_0}_q8_1,
 * launch_moe_grouped_gemm_*, launch_mmq_gguf_*_moe (hanzo-quant/src/gguf/ffi.rs),
 * launch_fp8_indexed_moe_gemm_* (blockwise_fp8/ffi.rs) and
 * launch_mxfp4_indexed_moe_gemm_* / launch_mxfp4_moe_grouped_gemm_* (mxfp4/ffi.rs).
 * Needs the dispatch tables built by hq_moe_dispatch_build for the same ids
 * (`workspace` is that call's workspace).
 * act != HQ_ACT_NONE fuses the gated activation: with `w_up` given, W is the
 * gate bank and w_up the up bank (out [T,k,N]); with w_up NULL the bank rows
 * interleave gate/up (row 2i = gate_i, 2i+1 = up_i) and out is [T,k,N/2]. */
#define HQ_ROWS_PER_TOKEN 0
#define HQ_ROWS_PER_SLOT 1
#define HQ_ROWS_SORTED 2
int32_t hq_moe_gather_forward(const hq_weight* w, const hq_weight* w_up, const hq_act_args* act, const void* x,
                              int32_t x_dtype, int32_t x_layout, int64_t n_tokens, int32_t top_k,
                              const int32_t* expert_bounds, const int32_t* sorted_assign,
                              const int32_t* sorted_token, const void* workspace, void* out, int32_t out_dtype,
                              int32_t out_layout, int32_t* status_dev, void* stream);

/* ---- one MoE layer in one call ---------------------------------------------
 * router -> dispatch tables -> gate/up projection with the gated activation -> down projection -> weighted
 * sum over the slots, launched back to back from one call: the fused form of the reference's per-layer
 * sequence (hanzo-engine/src/moe/experts/backends.rs:560-605; its single-launch decode entry is
 * indexed_moe_fused_decode, hanzo-quant/src/gguf/cuda.rs:879-1056).  What it saves over the separate calls is
 * host time between launches, which is most of a decode step of a few tokens.
 * `up` NULL means `gate` holds interleaved gate/up rows.  logits [n_tokens, n_experts]; x [n_tokens, hidden];
 * shared_addend [n_tokens, hidden] in out_dtype or NULL; out [n_tokens, hidden].  All scratch (routing, tables,
 * the expert-sorted intermediate and outputs) lives in the caller's workspace, 256-byte aligned, of
 * hq_moe_layer_workspace_bytes(layer, n_tokens, x_dtype) bytes. */
typedef struct hq_moe_layer {
  const hq_weight* gate;
  const hq_weight* up;
  const hq_weight* down;
  hq_act_args act;
  hq_router_args router;
} hq_moe_layer;
int64_t hq_moe_layer_workspace_bytes(const hq_moe_layer* layer, int64_t n_tokens, int32_t x_dtype);
int32_t hq_moe_layer_forward(const hq_moe_layer* layer, const void* logits, int32_t logits_dtype, const void* x,
                             int32_t x_dtype, int64_t n_tokens, const void* shared_addend, void* out,
                             int32_t out_dtype, void* workspace, int64_t workspace_bytes, int32_t* status_dev,
                             void* stream);

/* ---- combine: moe_weighted_reduce_flat -------------------------------------
 * out[t, :] = sum_s w[t, s] * y[t, s, :] (+ addend[t, :]), f32 accumulation in
 * slot order, no atomics.  Replaces launch_moe_weighted_reduce_flat{,_bf16}
 * (hanzo-quant/src/gguf/ffi.rs:421-435, moe_grouped.cu:678-703) and
 * moe_combine_kernel (hanzo-engine/src/cuda/moe_combine.cu:38-60).
 * y [T*k, H] in y_dtype, w f32 [T, k], addend [T, H] in out_dtype or NULL.
 * row_map int32 [T*k] gives the row of y that holds assignment (t, s) -- pass
 * inv_perm from hq_moe_dispatch_build when y is expert-sorted, NULL when y is
 * already in (token, slot) order.  A negative row_map entry skips that slot. */
int32_t hq_moe_weighted_reduce(const void* y, int32_t y_dtype, const float* w, const int32_t* row_map,
                               const void* addend, void* out, int32_t out_dtype, int64_t n_tokens, int32_t top_k,
                               int64_t hidden, void* stream);

/* ---- block-FP8 layers with FP8 activations --------------------------------
 * The block-scaled form of the FP8 path: activation rows are quantized 1 x 128 with the reference's vector
 * quantizer (hanzo-quant/src/vector_fp8/ops.rs:235-287: scale = absmax / 448 or 1e-12, q = e4m3(clamp(v /
 * scale))) and the e4m3 codes of weights and activations go into the FP8 tensor-core MMA unconverted; every
 * 128-column block is scaled by weight_scale_inv[n/128, k/128] * activation_scale[row, k/128] as it is added.
 * Results equal dequantize-then-matmul over the QUANTIZED activations up to f32 summation order; against
 * unquantized activations they carry the quantizer's ~3e-2 error, which is why hq_linear_forward /
 * hq_moe_gather_forward (16-bit activations) stay the default.  Requires N % 128 == 0, K % 512 == 0, K <= 8192.
 *
 * hq_fp8_quant_rows: codes [n_rows, k] / scales [n_rows, k/128] of rows x[row_map[r]] (row_map NULL = identity;
 * pass sorted_token to produce the expert-sorted rows the expert GEMM reads).  Replaces
 * launch_quant_fp8_vector_kernel_* (vector_fp8/ops.rs) plus the row gather.
 * hq_fp8_gated_quant_rows: gate_up [n_rows, 2*width] = {gate | up} -> act(gate) * up -> the same quantizer.
 * hq_fp8_linear_forward: dense layer over quantized rows.  hq_moe_fp8_gather_forward: expert bank over
 * expert-sorted quantized rows (n_tokens * top_k of them), output rows sorted or per slot, row stride
 * out_stride elements (so two banks can write the halves of one {gate | up} matrix); `workspace` is not read
 * (the kernel cuts its token tiles from expert_bounds) and may be NULL.
 * hq_moe_fp8_gate_up_forward: gate and up projection, gated activation and the 1 x 128 quantizer of the result in
 * one launch -- the fused form of the reference's gate/up GEMMs + fused_glu + quantizer sequence
 * (hanzo-engine/src/moe/experts/backends.rs:560-605, hanzo-quant/kernels/ops/ops.cu:845-858): gate and up are
 * rounded to f16, act(gate) * up is computed in f32 and rounded to f16, then quantized; h_codes [n_tokens * top_k,
 * N] and h_scales [n_tokens * top_k, N / 128] come out expert-sorted, ready for the down projection. */
int32_t hq_fp8_quant_rows(const void* x, int32_t x_dtype, int64_t x_stride, const int32_t* row_map, int64_t n_rows,
                          int64_t k, uint8_t* codes, float* scales, void* stream);
int32_t hq_fp8_gated_quant_rows(const void* gate_up, int32_t dtype, int64_t n_rows, int64_t width,
                                const hq_act_args* act, uint8_t* codes, float* scales, void* stream);
int32_t hq_fp8_linear_forward(const hq_weight* w, const uint8_t* x_codes, const float* x_scales, int64_t m, void* y,
                              int32_t y_dtype, int64_t y_stride, int32_t* status_dev, void* stream);
int32_t hq_moe_fp8_gather_forward(const hq_weight* w, const uint8_t* x_codes, const float* x_scales,
                                  int64_t n_tokens, int32_t top_k, const int32_t* expert_bounds,
                                  const int32_t* sorted_assign, const void* workspace, void* out, int32_t out_dtype,
                                  int64_t out_stride, int32_t out_layout, int32_t* status_dev, void* stream);
int32_t hq_moe_fp8_gate_up_forward(const hq_weight* w_gate, const hq_weight* w_up, const hq_act_args* act,
                                   const uint8_t* x_codes, const float* x_scales, int64_t n_tokens, int32_t top_k,
                                   const int32_t* expert_bounds, uint8_t* h_codes, float* h_scales,
                                   int32_t* status_dev, void* stream);

/* hq_fp8_quant_rows with a row count that lives on the device: only rows r < min(*n_valid_dev, n_rows) are
 * produced.  For row maps whose tail is undefined -- sorted_token after a dispatch build that skipped padding
 * ids has expert_bounds[E] valid entries, so pass expert_bounds + E. */
int32_t hq_fp8_quant_rows_n(const void* x, int32_t x_dtype, int64_t x_stride, const int32_t* row_map,
                            const int32_t* n_valid_dev, int64_t n_rows, int64_t k, uint8_t* codes, float* scales,
                            void* stream);
/* Row gather of rows that are FP8 already (received over the wire): codes [r] = src_codes + row_map[r] *
 * src_code_stride (k bytes), scales [r] = src_scales + row_map[r] * src_scale_stride_bytes (k / 128 floats), for
 * r < min(*n_valid_dev, n_rows) (n_valid_dev NULL = all).  No counterpart in the reference. */
int32_t hq_fp8_gather_rows(const uint8_t* src_codes, int64_t src_code_stride, const float* src_scales,
                           int64_t src_scale_stride_bytes, const int32_t* row_map, const int32_t* n_valid_dev,
                           int64_t n_rows, int64_t k, uint8_t* codes, float* scales, void* stream);

/* ---- MXFP4 layers with MXFP8 activations: the block-scaled tensor-core path --------------------------------
 * The counterpart of the FP8-activation calls above for MXFP4Layer banks (hanzo-quant/src/mxfp4/mod.rs:29-174): the
 * e2m1 nibbles are never expanded, the activations are MXFP8 (e4m3 codes + one e8m0 scale per 32 elements) and
 * tcgen05.mma kind::mxf8f6f4 with block scaling applies both operands' e8m0 scales per 32-element block.  The
 * reference has no activation quantizer for this format (its MXFP4 kernels multiply bf16 / f16 activations,
 * kernels/mxfp4/mxfp4_gemm_wmma.cu:310-492); the one used here is the OCP microscaling rule for e4m3 elements:
 * shared exponent = floor(log2(amax)) - 8, biased by 127 and kept in 0..254 (127 for an all-zero block), elements
 * scaled by 2^-e and converted with saturation at +-448 (the structure of MXFP4Layer::quantize, mxfp4/mod.rs:216-300).
 * Results equal dequantize-then-matmul over the QUANTIZED activations up to f32 summation order.
 * Requires K % 64 == 0, 128 <= K <= 9728 (the scale bytes of a work item are staged in shared memory); w->data
 * 32-byte aligned with at least 64 readable bytes after the last row (the packed 4-bit tensor map reads whole
 * 128-element groups; what lies past a row's end meets zero activations); x_codes, x_scales and w->scales 16-byte
 * aligned.
 *
 * hq_mxfp8_quant_rows: codes [n_rows, k] / scales u8 [n_rows, k/32] of rows x[row_map[r]], r < min(*n_valid_dev,
 * n_rows) (row_map / n_valid_dev may be NULL).
 * hq_mx_linear_forward: dense layer over quantized rows.
 * hq_moe_mx_gather_forward: expert bank over expert-sorted quantized rows.  act NULL / HQ_ACT_NONE: plain
 * projection, out [rows, N] sorted or per slot.  Otherwise the bank's rows interleave gate / up (gpt-oss): bias,
 * gated activation, and either h_codes / h_scales (MXFP8 of the N/2 activated values per row, for the down
 * projection) when h_codes is given, or out [rows, N/2] sorted. */
int32_t hq_mxfp8_quant_rows(const void* x, int32_t x_dtype, int64_t x_stride, const int32_t* row_map,
                            const int32_t* n_valid_dev, int64_t n_rows, int64_t k, uint8_t* codes, uint8_t* scales,
                            void* stream);
int32_t hq_mx_linear_forward(const hq_weight* w, const uint8_t* x_codes, const uint8_t* x_scales, int64_t m, void* y,
                             int32_t y_dtype, int64_t y_stride, int32_t* status_dev, void* stream);
int32_t hq_moe_mx_gather_forward(const hq_weight* w, const hq_act_args* act, const uint8_t* x_codes,
                                 const uint8_t* x_scales, int64_t n_tokens, int32_t top_k, const int32_t* expert_bounds,
                                 const int32_t* sorted_assign, void* out, int32_t out_dtype, int64_t out_stride,
                                 int32_t out_layout, uint8_t* h_codes, uint8_t* h_scales, int32_t* status_dev,
                                 void* stream);

/* ---- expert parallelism: what a rank does either side of the two all-to-all exchanges --------------------
 * The reference shards quantized experts over GPUs nowhere (its MoE collective is the tensor-parallel all-reduce
 * behind hanzo-engine/src/moe/experts/mod.rs:260-263, NCCL wrapper hanzo-quant/src/distributed/mod.rs:213-274,
 * :494-617); these calls are the device side of an expert-parallel layer built on the same local kernels, so that
 * a host only adds two equal-split all-to-all calls (ncclSend / ncclRecv of message_bytes per peer).
 *
 * Experts are sharded in contiguous ranges of experts_per_rank.  A token travels ONCE to every rank that hosts at
 * least one of its top_k experts, and that rank returns ONE row for it: the router-weighted sum over the experts
 * it hosts.  Every per-peer message has the same size (capacity token rows + the meta rows), so no counts go
 * through the host.  capacity = the largest number of tokens a rank brings to one call; it must be the same on
 * every rank.
 *   message to peer d: rows [0, capacity) = token payloads (written only for tokens that go to d): hidden values
 *   in wire_dtype, or with fp8 = 1 hidden e4m3 codes + hidden / 128 f32 scales (1 x 128 quantizer, so the expert
 *   rank feeds the FP8 MMA unchanged); rows [capacity, rows_per_peer) = per token and slot (int32 local expert id
 *   or -1, f32 router weight).
 * hq_ep_pack fills `send` [world, rows_per_peer, row_bytes] and back_map int32 [n_tokens, world] (row of the
 * returned buffer that holds rank d's partial sum for token t, or -1).  After the dispatch all-to-all,
 * hq_ep_unpack_meta turns the meta rows of `recv` (same shape) into ids uint32 / weights f32 [world *
 * rows_per_peer, top_k] for the local expert block (hq_moe_dispatch_build skips the -1 slots).  The local block's
 * weighted reduce over those rows gives [world * rows_per_peer, hidden] partial sums; after the return all-to-all
 * the source rank calls hq_moe_weighted_reduce(y = returned rows, w = ones [n_tokens, world], row_map = back_map,
 * top_k = world) to add the partial sums (and the shared expert, as the addend). */
typedef struct hq_ep_layout {
  int32_t world, top_k, experts_per_rank, capacity;
  int32_t pad_rows, rows_per_peer, fp8, wire_dtype;
  int64_t hidden, row_bytes, message_bytes;
} hq_ep_layout;
int32_t hq_ep_layout_init(hq_ep_layout* layout, int32_t world, int32_t top_k, int32_t experts_per_rank,
                          int32_t capacity, int64_t hidden, int32_t wire_dtype, int32_t fp8);
int32_t hq_ep_pack(const hq_ep_layout* layout, const void* x, int32_t x_dtype, const uint32_t* ids,
                   const float* weights, int64_t n_tokens, void* send, int32_t* back_map, void* stream);
int32_t hq_ep_unpack_meta(const hq_ep_layout* layout, const void* recv, uint32_t* ids_out, float* weights_out,
                          void* stream);

/* The exchange itself over peer memory, for hosts that hold their receive buffers in a symmetric allocation (every
 * rank's buffer mapped into every other rank's address space, e.g. cuMemMap of exported handles or
 * torch.distributed._symmetric_memory): an alternative to the two all-to-all calls.
 * hq_ep_push copies slab d (slab_bytes, a multiple of 16) of the local `send` buffer into slot `rank` of peer d's
 * buffer with plain stores over NVLink (peer_slabs_dev: device array of `world` base pointers, 16-byte aligned;
 * entry `rank` is this rank's own buffer).  hq_ep_barrier then tells every peer that this rank's data has arrived
 * and waits for theirs: peer_flags_dev is a device array of `world` pointers to int32[world] flag arrays in
 * symmetric memory, zero before the first call; seq_counter_dev a local device int32, zero before the first call,
 * that counts the barriers (kept on the device so that the calls can sit in a replayed CUDA graph).  The wait is
 * bounded by HQ_CFG_SPIN_LIMIT; when it runs out HQ_DEV_WAIT_TIMEOUT (tag 950 + peer) is left in status_dev and the
 * call returns.  With two barriers per layer (after the dispatch push and after the return push) single buffers
 * are safe to reuse in the next layer: a peer can only pass a barrier after this rank has finished everything it
 * queued before its own signal. */
int32_t hq_ep_push(const void* send, void* const* peer_slabs_dev, int32_t world, int32_t rank, int64_t slab_bytes,
                   void* stream);
int32_t hq_ep_barrier(int32_t* const* peer_flags_dev, int32_t world, int32_t rank, int32_t* seq_counter_dev,
                      int32_t* status_dev, void* stream);
/* hq_ep_push row by row, without the rows nobody reads (a token goes to about 5 of 8 ranks).  Slab d has
 * rows_per_slab rows of row_bytes (a multiple of 16) bytes.  Rows at or behind always_from are always sent (the meta
 * rows of a dispatch slab); an earlier row r of slab d is sent when back_map[r * world + d] >= 0 and r < n_tokens
 * (dispatch: back_map as written by hq_ep_pack, ids NULL), or when one of its top_k ids is not 0xFFFFFFFF (return:
 * ids [world * rows_per_slab, top_k] as written by hq_ep_unpack_meta, back_map NULL).  What is left out keeps
 * whatever the peer's buffer held; the receiver never reads those rows. */
int32_t hq_ep_push_rows(const void* send, void* const* peer_slabs_dev, int32_t world, int32_t rank,
                        int32_t rows_per_slab, int64_t row_bytes, int32_t always_from, const int32_t* back_map,
                        int32_t n_tokens, const uint32_t* ids, int32_t top_k, void* stream);

/* ---- FP8 quantizers ---------------------------------------------------------
 * 1x128 groups along the last axis: scale = absmax/448 (1e-12 if zero),
 * code = e4m3(clamp(v/scale, +-448)).  Replaces launch_quant_fp8_vector_kernel_*
 * / launch_dequant_fp8_vector_kernel_* (hanzo-quant/src/vector_fp8/ffi.rs;
 * CPU twin vector_fp8/ops.rs:235-287).  n_elems % 128 == 0. */
int32_t hq_fp8_vector_quant(const void* x, int32_t x_dtype, int64_t n_elems, uint8_t* codes, float* scales,
                            void* stream);
int32_t hq_fp8_vector_dequant(const uint8_t* codes, const float* scales, int64_t n_elems, void* out,
                              int32_t out_dtype, void* stream);
/* 128x128 (by x bx) blocks over [rows, cols]: launch_{quant,dequant}_fp8_blockwise_kernel_*
 * (hanzo-quant/src/blockwise_fp8/ffi.rs; CPU twin blockwise_fp8/ops.rs:11-59, :329-411). */
int32_t hq_fp8_block_quant(const void* w, int32_t w_dtype, int64_t rows, int64_t cols, int32_t by, int32_t bx,
                           uint8_t* codes, float* scales, void* stream);
int32_t hq_fp8_block_dequant(const uint8_t* codes, const float* scales, int64_t rows, int64_t cols, int32_t by,
                             int32_t bx, void* out, int32_t out_dtype, void* stream);

/* Derives the tables hq_weight.fp8_tile_scale / fp8_rel_scale from a layer's scale grid
 * (f32 [E, ceil(N/128), ceil(K/128)]): the largest scale of every 128-row block and each scale
 * divided by it.  No counterpart in the reference (its FP8 kernels multiply by the scale per
 * element, hanzo-quant/kernels/blockwise_fp8/blockwise_fp8_gemm.cu:47-124). */
int32_t hq_fp8_scale_prepare(const float* scales, int32_t n_experts, int64_t n, int64_t k, float* tile_scale_out,
                             float* rel_scale_out, void* stream);

/* Elementwise dtype conversion (f32 / f16 / bf16).  The prefill-sized calls run on the tensor cores only
 * when the activations are f16 (their rows are copied straight into the operand tiles); a host holding
 * bf16 or f32 activations converts once with this call -- the reference's Tensor::to_dtype
 * (e.g. hanzo-quant/src/gguf/mod.rs:196-209). */
int32_t hq_convert(const void* src, int32_t src_dtype, void* dst, int32_t dst_dtype, int64_t n_elems, void* stream);
/* The same conversion with a device status word.  The tensor-core kernels multiply f16 by f16, so their inputs are
 * limited to +-65504 -- a limit the reference's bf16 / f32 activation paths do not have (it quantizes from f32,
 * hanzo-quant/kernels/mmvq_gguf/mmvq_gguf.cu:1263-1295, or multiplies bf16, blockwise_fp8_gemm.cu:131-258).  A finite
 * value beyond the range is clamped to +-65504 and HQ_DEV_F16_RANGE is left in status_dev; hq_moe_layer_forward
 * converts through this call. */
int32_t hq_convert_status(const void* src, int32_t src_dtype, void* dst, int32_t dst_dtype, int64_t n_elems,
                          int32_t* status_dev, void* stream);

/* Measurement aid, no counterpart in the reference: every SM issues iters x 4 tcgen05.mma instructions back to back
 * (M = 128, N = n, operands resident in shared memory; kind 0 = f16 x f16, K = 16 per instruction; kind 1 = e4m3 x
 * e4m3 on kind::f8f6f4, K = 32).  *flops_host receives the floating-point operations of the launch; the caller
 * times the launch with events.  Gives the FP8 tensor peak the expert GEMM's fraction is quoted against. */
int32_t hq_probe_tensor_peak(int32_t kind, int32_t n, int32_t iters, int32_t* status_dev, double* flops_host,
                             void* stream);

/* ---- gated activations as stand-alone ops -----------------------------------
 * out = act(gate, up) elementwise over n_elems; interleaved = 1 reads pairs
 * (gate, up) from `gate` ([..., I, 2]) and ignores `up`.  Replaces fused_glu_*,
 * gptoss_swiglu_* and gptoss_swiglu_interleaved_* (hanzo-quant/src/utils/ffi.rs,
 * kernels/ops/ops.cu:335-360, :482-512, :845-858).  Math in f32, one rounding
 * to `dtype` at the end. */
int32_t hq_gated_act(const void* gate, const void* up, int32_t dtype, int64_t n_elems, int32_t interleaved,
                     const hq_act_args* act, void* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* HANZOQUANT_B200_H */
