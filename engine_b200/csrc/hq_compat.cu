// Reference-named entry points (include/hanzoquant_compat.h): every symbol is a thin call into the hq_* ABI.
#include <cstdio>
#include <mutex>

#include "../../include/hanzoquant_compat.h"
#include "hq_common.cuh"
#include "hq_kernels.h"

using namespace hq;

namespace {

void complain(const char* symbol, int32_t rc) {
  static std::mutex mu;
  static const char* seen[64];
  static int n_seen = 0;
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < n_seen; ++i)
    if (seen[i] == symbol) return;
  if (n_seen < 64) seen[n_seen++] = symbol;
  std::fprintf(stderr, "libhanzoquant_b200: %s: %s (%d); the call was not launched\n", symbol, hq_error_string(rc), rc);
}

// ---- scratch for the calls that need dispatch tables -----------------------------------------------
constexpr int kCompatMaxAssign = 65536;
constexpr int kCompatMaxExperts = 512;
constexpr int64_t kCompatWsWords = 4 + (int64_t)(kCompatMaxAssign / kDispatchChunk) * kCompatMaxExperts +
                                   2 * ((int64_t)kCompatMaxAssign / 8 + kCompatMaxExperts) +
                                   2 * ((int64_t)kCompatMaxAssign / 128 + kCompatMaxExperts) +
                                   2 * ((int64_t)kCompatMaxAssign / 256 + kCompatMaxExperts);
constexpr int64_t kCompatWords = (kCompatMaxExperts + 64) + 3 * (int64_t)kCompatMaxAssign + kCompatWsWords + 64;
static __device__ __align__(256) int32_t g_compat_scratch[kCompatWords];

struct Tables {
  int32_t *bounds, *sorted_assign, *sorted_token, *inv_perm, *ws;
  int64_t ws_bytes;
  void* to_free;      // stream-ordered allocation to release after the launches, or nullptr
};

int64_t up64(int64_t words) { return (words + 63) / 64 * 64; }

// Carves the tables out of the fixed array, or out of a stream-ordered allocation when the call is larger.
int32_t get_tables(int64_t n_tokens, int top_k, int n_experts, cudaStream_t stream, Tables& t) {
  const int64_t assign = n_tokens * top_k;
  const int64_t ws_words = dispatch_layout(n_tokens, top_k, n_experts).total_words;
  const int64_t need = up64(n_experts + 1) + 3 * up64(assign) + up64(ws_words);
  int32_t* base = nullptr;
  t.to_free = nullptr;
  if (assign <= kCompatMaxAssign && n_experts <= kCompatMaxExperts && need <= kCompatWords) {
    static int32_t* dev_ptr[64] = {};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return HQ_ERR_CUDA;
    std::lock_guard<std::mutex> lock(mu);
    if (dev_ptr[dev] == nullptr) {
      void* p = nullptr;
      if (cudaGetSymbolAddress(&p, g_compat_scratch) != cudaSuccess || p == nullptr) return HQ_ERR_CUDA;
      dev_ptr[dev] = static_cast<int32_t*>(p);
    }
    base = dev_ptr[dev];
  } else {
    void* p = nullptr;
    if (cudaMallocAsync(&p, (size_t)need * 4, stream) != cudaSuccess) return HQ_ERR_CUDA;
    base = static_cast<int32_t*>(p);
    t.to_free = p;
  }
  t.bounds = base;
  t.sorted_assign = t.bounds + up64(n_experts + 1);
  t.sorted_token = t.sorted_assign + up64(assign);
  t.inv_perm = t.sorted_token + up64(assign);
  t.ws = t.inv_perm + up64(assign);
  t.ws_bytes = ws_words * 4;
  return HQ_OK;
}

void release(const Tables& t, cudaStream_t stream) {
  if (t.to_free != nullptr) cudaFreeAsync(t.to_free, stream);
}

// expert projection out of a bank through ids, no gated activation: out [T, k, N] in (token, slot) order
int32_t indexed_gemm(const hq_weight& w, const void* x, int x_dtype, bool per_slot, const uint32_t* ids,
                     int64_t n_tokens, int top_k, void* out, int out_dtype, cudaStream_t stream) {
  Tables t;
  int32_t rc = get_tables(n_tokens, top_k, w.n_experts, stream, t);
  if (rc != HQ_OK) return rc;
  rc = hq_moe_dispatch_build(ids, n_tokens, top_k, w.n_experts, t.bounds, t.sorted_assign, t.sorted_token, t.inv_perm,
                             t.ws, t.ws_bytes, stream);
  if (rc == HQ_OK)
    rc = hq_moe_gather_forward(&w, nullptr, nullptr, x, x_dtype, per_slot ? HQ_ROWS_PER_SLOT : HQ_ROWS_PER_TOKEN,
                               n_tokens, top_k, t.bounds, t.sorted_assign, t.sorted_token, t.ws, out, out_dtype,
                               HQ_ROWS_PER_SLOT, nullptr, stream);
  release(t, stream);
  return rc;
}

// ---- which activation buffer a Q8_1 scratch pointer stands for ---------------------------------------
struct Q81Record {
  const void* scratch;
  const void* x;
  int dtype, kx, rows;
};
std::mutex g_q81_mu;
Q81Record g_q81[32];
int g_q81_next = 0;

void q81_remember(const void* scratch, const void* x, int dtype, int kx, int rows) {
  std::lock_guard<std::mutex> lock(g_q81_mu);
  for (auto& r : g_q81)
    if (r.scratch == scratch) {
      r = {scratch, x, dtype, kx, rows};
      return;
    }
  g_q81[g_q81_next] = {scratch, x, dtype, kx, rows};
  g_q81_next = (g_q81_next + 1) % 32;
}
bool q81_lookup(const void* scratch, Q81Record& out) {
  std::lock_guard<std::mutex> lock(g_q81_mu);
  for (const auto& r : g_q81)
    if (r.scratch == scratch && r.x != nullptr) {
      out = r;
      return true;
    }
  return false;
}

hq_weight gguf_weight(int format, const void* data, int n_experts, int64_t n, int64_t k) {
  hq_weight w{};
  w.format = format;
  w.n_experts = n_experts;
  w.n = n;
  w.k = k;
  w.data = data;
  return w;
}

void mmvq_plain(const char* symbol, int format, int out_dtype, const void* vx, const void* vy, void* dst, int ncols_x,
                int nrows_x, int stride_col_dst, int b_size, void* stream) {
  Q81Record r;
  if (!q81_lookup(vy, r) || r.kx != ncols_x || r.rows < b_size) return complain(symbol, HQ_ERR_WORKSPACE);
  const hq_weight w = gguf_weight(format, vx, 1, nrows_x, ncols_x);
  const int32_t rc = hq_linear_forward(&w, r.x, r.dtype, ncols_x, dst, out_dtype, stride_col_dst, b_size, nullptr, stream);
  if (rc != HQ_OK) complain(symbol, rc);
}

void indexed_q81(const char* symbol, int format, const void* all_weights, const void* all_inputs,
                 const uint32_t* indices, float* all_outputs, int n, int k, int batch, int topk, int input_dim1,
                 void* stream) {
  Q81Record r;
  if (!q81_lookup(all_inputs, r) || r.kx != k) return complain(symbol, HQ_ERR_WORKSPACE);
  // the bank's expert count is not an argument of the reference call: ids are trusted to be in range, as there
  hq_weight w = gguf_weight(format, all_weights, kCompatMaxExperts, n, k);
  const int32_t rc = indexed_gemm(w, r.x, r.dtype, input_dim1 > 1, indices, batch, topk, all_outputs, HQ_DT_F32,
                                  (cudaStream_t)stream);
  if (rc != HQ_OK) complain(symbol, rc);
}

void fp8_matmul(const char* symbol, int dtype, const void* input, const void* weight, const float* scale, void* output,
                int m, int n, int k, int scale_row_stride, int by, int bx, void* stream) {
  if (by != 128 || bx != 128 || scale_row_stride != (k + 127) / 128) return complain(symbol, HQ_ERR_SHAPE);
  hq_weight w{};
  w.format = HQ_FMT_FP8_BLOCK;
  w.n_experts = 1;
  w.n = n;
  w.k = k;
  w.data = weight;
  w.scales = scale;
  const int32_t rc = hq_linear_forward(&w, input, dtype, k, output, dtype, n, m, nullptr, stream);
  if (rc != HQ_OK) complain(symbol, rc);
}

void fp8_indexed(const char* symbol, int dtype, const void* input, const void* weights, const float* scales,
                 const uint32_t* indices, void* output, int num_tokens, int topk, int num_experts, int n, int k,
                 int scale_row_stride, int by, int bx, bool per_slot, void* stream) {
  if (by != 128 || bx != 128 || scale_row_stride != (k + 127) / 128) return complain(symbol, HQ_ERR_SHAPE);
  hq_weight w{};
  w.format = HQ_FMT_FP8_BLOCK;
  w.n_experts = num_experts;
  w.n = n;
  w.k = k;
  w.data = weights;
  w.scales = scales;
  const int32_t rc = indexed_gemm(w, input, dtype, per_slot, indices, num_tokens, topk, output, dtype,
                                  (cudaStream_t)stream);
  if (rc != HQ_OK) complain(symbol, rc);
}

void mxfp4_matmul(const char* symbol, int dtype, const void* input, const uint8_t* weight, const uint8_t* scale,
                  const void* bias, void* output, int m, int n, int k, bool has_bias, void* stream) {
  hq_weight w{};
  w.format = HQ_FMT_MXFP4;
  w.n_experts = 1;
  w.n = n;
  w.k = k;
  w.data = weight;
  w.scales = scale;
  w.bias = has_bias ? bias : nullptr;
  w.bias_dtype = dtype;
  const int32_t rc = hq_linear_forward(&w, input, dtype, k, output, dtype, n, m, nullptr, stream);
  if (rc != HQ_OK) complain(symbol, rc);
}

void mxfp4_moe(const char* symbol, int dtype, const void* input, const uint8_t* weights, const uint8_t* scales,
               const void* biases, const uint32_t* indices, void* output, int num_tokens, int topk, int num_experts,
               int n, int k, bool has_bias, bool per_slot, void* stream) {
  hq_weight w{};
  w.format = HQ_FMT_MXFP4;
  w.n_experts = num_experts;
  w.n = n;
  w.k = k;
  w.data = weights;
  w.scales = scales;
  w.bias = has_bias ? biases : nullptr;
  w.bias_dtype = dtype;
  const int32_t rc = indexed_gemm(w, input, dtype, per_slot, indices, num_tokens, topk, output, dtype,
                                  (cudaStream_t)stream);
  if (rc != HQ_OK) complain(symbol, rc);
}

void router(const char* symbol, int dtype, const void* logits, void* weights, void* ids, const void* selection_bias,
            const void* expert_scale, int nrows, int n_experts, int top_k, int score_mode, int weight_mode,
            bool renormalize, bool clamp_logits, float clamp_min, float clamp_max, float norm_min, float output_scale,
            int64_t stream) {
  hq_router_args a{};
  a.n_experts = n_experts;
  a.top_k = top_k;
  a.score_mode = score_mode;
  a.weight_mode = weight_mode;
  a.renormalize = renormalize;
  a.clamp_logits = clamp_logits;
  a.clamp_min = clamp_min;
  a.clamp_max = clamp_max;
  a.norm_min = norm_min;
  a.output_scale = output_scale;
  a.selection_bias = static_cast<const float*>(selection_bias);
  a.expert_scale = static_cast<const float*>(expert_scale);
  const int32_t rc = hq_router_topk(logits, dtype, nrows, &a, static_cast<uint32_t*>(ids), static_cast<float*>(weights),
                                    reinterpret_cast<void*>(stream));
  if (rc != HQ_OK) complain(symbol, rc);
}

void gptoss(const char* symbol, int dtype, const void* gate, const void* up, void* output, uint64_t n, int interleaved,
            float alpha, float limit, void* stream) {
  hq_act_args a{HQ_ACT_GPTOSS, 1, limit, alpha};
  const int32_t rc = hq_gated_act(gate, up, dtype, n, interleaved, &a, output, stream);
  if (rc != HQ_OK) complain(symbol, rc);
}

void glu(const char* symbol, int dtype, const void* a_in, const void* b_in, void* output, uint32_t n, int activation,
         void* stream) {
  if (activation != 0) return complain(symbol, HQ_ERR_FORMAT);      // SiLU only on this path
  hq_act_args a{HQ_ACT_SWIGLU, 0, 0.f, 0.f};
  const int32_t rc = hq_gated_act(a_in, b_in, dtype, n, 0, &a, output, stream);
  if (rc != HQ_OK) complain(symbol, rc);
}

void block_quant(const char* symbol, int dtype, const void* in, void* codes, float* scales, int h, int wd,
                 int row_stride, int scale_stride, int by, int bx, void* stream) {
  if (row_stride != wd || scale_stride != (wd + bx - 1) / bx) return complain(symbol, HQ_ERR_SHAPE);
  const int32_t rc = hq_fp8_block_quant(in, dtype, h, wd, by, bx, static_cast<uint8_t*>(codes), scales, stream);
  if (rc != HQ_OK) complain(symbol, rc);
}
void block_dequant(const char* symbol, int dtype, const void* codes, const float* scales, void* out, int h, int wd,
                   int row_stride, int scale_stride, int by, int bx, void* stream) {
  if (row_stride != wd || scale_stride != (wd + bx - 1) / bx) return complain(symbol, HQ_ERR_SHAPE);
  const int32_t rc = hq_fp8_block_dequant(static_cast<const uint8_t*>(codes), scales, h, wd, by, bx, out, dtype, stream);
  if (rc != HQ_OK) complain(symbol, rc);
}

}  // namespace

extern "C" {

void launch_moe_dispatch(const int32_t* topk_ids, int32_t* expert_bounds, int32_t* sorted_token_ids,
                         int32_t* sorted_source_ids, int32_t total_assignments, int32_t num_experts, int32_t topk,
                         int32_t* expert_counts, int32_t* expert_cursors, void* stream) {
  (void)expert_counts;
  (void)expert_cursors;
  if (topk < 1 || total_assignments % topk != 0) return complain("launch_moe_dispatch", HQ_ERR_SHAPE);
  const int64_t n_tokens = total_assignments / topk;
  Tables t;
  int32_t rc = get_tables(n_tokens, topk, num_experts, (cudaStream_t)stream, t);
  if (rc == HQ_OK) {
    rc = hq_moe_dispatch_build(reinterpret_cast<const uint32_t*>(topk_ids), n_tokens, topk, num_experts, expert_bounds,
                               sorted_token_ids, sorted_source_ids, t.inv_perm, t.ws, t.ws_bytes, stream);
    release(t, (cudaStream_t)stream);
  }
  if (rc != HQ_OK) complain("launch_moe_dispatch", rc);
}

void launch_moe_weighted_reduce_flat(const float* inputs, const float* topk_weights, float* outputs,
                                     int32_t num_tokens, int32_t hidden, int32_t topk, void* stream) {
  const int32_t rc = hq_moe_weighted_reduce(inputs, HQ_DT_F32, topk_weights, nullptr, nullptr, outputs, HQ_DT_F32,
                                            num_tokens, topk, hidden, stream);
  if (rc != HQ_OK) complain("launch_moe_weighted_reduce_flat", rc);
}
void launch_moe_weighted_reduce_flat_bf16(const float* inputs, const float* topk_weights, void* outputs,
                                          int32_t num_tokens, int32_t hidden, int32_t topk, void* stream) {
  const int32_t rc = hq_moe_weighted_reduce(inputs, HQ_DT_F32, topk_weights, nullptr, nullptr, outputs, HQ_DT_BF16,
                                            num_tokens, topk, hidden, stream);
  if (rc != HQ_OK) complain("launch_moe_weighted_reduce_flat_bf16", rc);
}

#define HQ_Q81_RECORD(name, dt)                                                                             \
  void name(const void* x, void* vy, int32_t kx, int32_t kx_padded, int32_t num_rows, void* stream) {      \
    (void)kx_padded;                                                                                        \
    (void)stream;                                                                                           \
    q81_remember(vy, x, dt, kx, num_rows);                                                                  \
  }
HQ_Q81_RECORD(launch_mmvq_gguf_quantize_q8_1_bf16, HQ_DT_BF16)
HQ_Q81_RECORD(launch_mmvq_gguf_quantize_q8_1_f16, HQ_DT_F16)
HQ_Q81_RECORD(launch_mmvq_gguf_quantize_q8_1_f32, HQ_DT_F32)
HQ_Q81_RECORD(launch_quantize_q8_1_bf16, HQ_DT_BF16)
HQ_Q81_RECORD(launch_quantize_q8_1_f16, HQ_DT_F16)
void launch_quantize_q8_1(const float* x, void* vy, int32_t kx, int32_t kx_padded, int32_t num_blocks_x,
                          int32_t num_rows, void* stream) {
  (void)kx_padded;
  (void)num_blocks_x;
  (void)stream;
  q81_remember(vy, x, HQ_DT_F32, kx, num_rows);
}

#define HQ_PLAIN(name, fmt, dt)                                                                              \
  void name(const void* vx, const void* vy, void* dst, int32_t ncols_x, int32_t nrows_x, int32_t stride_col_y, \
            int32_t stride_col_dst, int32_t b_size, void* stream) {                                          \
    (void)stride_col_y;                                                                                      \
    mmvq_plain(#name, fmt, dt, vx, vy, dst, ncols_x, nrows_x, stride_col_dst, b_size, stream);               \
  }
HQ_PLAIN(launch_mmvq_gguf_q8_0_bf16_plain, HQ_FMT_Q8_0, HQ_DT_BF16)
HQ_PLAIN(launch_mmvq_gguf_q8_0_f16_plain, HQ_FMT_Q8_0, HQ_DT_F16)
HQ_PLAIN(launch_mmvq_gguf_q8_0_f32_plain, HQ_FMT_Q8_0, HQ_DT_F32)
HQ_PLAIN(launch_mmvq_gguf_q4_k_bf16_plain, HQ_FMT_Q4_K, HQ_DT_BF16)
HQ_PLAIN(launch_mmvq_gguf_q4_k_f16_plain, HQ_FMT_Q4_K, HQ_DT_F16)
HQ_PLAIN(launch_mmvq_gguf_q4_k_f32_plain, HQ_FMT_Q4_K, HQ_DT_F32)
HQ_PLAIN(launch_mmvq_gguf_q6_k_bf16_plain, HQ_FMT_Q6_K, HQ_DT_BF16)
HQ_PLAIN(launch_mmvq_gguf_q6_k_f16_plain, HQ_FMT_Q6_K, HQ_DT_F16)
HQ_PLAIN(launch_mmvq_gguf_q6_k_f32_plain, HQ_FMT_Q6_K, HQ_DT_F32)
HQ_PLAIN(launch_mmvq_gguf_q5_k_bf16_plain, HQ_FMT_Q5_K, HQ_DT_BF16)
HQ_PLAIN(launch_mmvq_gguf_q5_k_f16_plain, HQ_FMT_Q5_K, HQ_DT_F16)
HQ_PLAIN(launch_mmvq_gguf_q5_k_f32_plain, HQ_FMT_Q5_K, HQ_DT_F32)
HQ_PLAIN(launch_mmvq_gguf_q4_0_bf16_plain, HQ_FMT_Q4_0, HQ_DT_BF16)
HQ_PLAIN(launch_mmvq_gguf_q4_0_f16_plain, HQ_FMT_Q4_0, HQ_DT_F16)
HQ_PLAIN(launch_mmvq_gguf_q4_0_f32_plain, HQ_FMT_Q4_0, HQ_DT_F32)
HQ_PLAIN(launch_mmvq_gguf_q5_0_bf16_plain, HQ_FMT_Q5_0, HQ_DT_BF16)
HQ_PLAIN(launch_mmvq_gguf_q5_0_f16_plain, HQ_FMT_Q5_0, HQ_DT_F16)
HQ_PLAIN(launch_mmvq_gguf_q5_0_f32_plain, HQ_FMT_Q5_0, HQ_DT_F32)
HQ_PLAIN(launch_mmvq_gguf_q4_1_bf16_plain, HQ_FMT_Q4_1, HQ_DT_BF16)
HQ_PLAIN(launch_mmvq_gguf_q4_1_f16_plain, HQ_FMT_Q4_1, HQ_DT_F16)
HQ_PLAIN(launch_mmvq_gguf_q4_1_f32_plain, HQ_FMT_Q4_1, HQ_DT_F32)
HQ_PLAIN(launch_mmvq_gguf_q5_1_bf16_plain, HQ_FMT_Q5_1, HQ_DT_BF16)
HQ_PLAIN(launch_mmvq_gguf_q5_1_f16_plain, HQ_FMT_Q5_1, HQ_DT_F16)
HQ_PLAIN(launch_mmvq_gguf_q5_1_f32_plain, HQ_FMT_Q5_1, HQ_DT_F32)
HQ_PLAIN(launch_mmvq_gguf_q2_k_bf16_plain, HQ_FMT_Q2_K, HQ_DT_BF16)
HQ_PLAIN(launch_mmvq_gguf_q2_k_f16_plain, HQ_FMT_Q2_K, HQ_DT_F16)
HQ_PLAIN(launch_mmvq_gguf_q2_k_f32_plain, HQ_FMT_Q2_K, HQ_DT_F32)
HQ_PLAIN(launch_mmvq_gguf_q3_k_bf16_plain, HQ_FMT_Q3_K, HQ_DT_BF16)
HQ_PLAIN(launch_mmvq_gguf_q3_k_f16_plain, HQ_FMT_Q3_K, HQ_DT_F16)
HQ_PLAIN(launch_mmvq_gguf_q3_k_f32_plain, HQ_FMT_Q3_K, HQ_DT_F32)

void launch_indexed_moe_forward_q4k_q8_1(const void* all_weights, const void* all_inputs, const uint32_t* indices,
                                         float* all_outputs, int32_t n, int32_t k, int32_t batch, int32_t topk,
                                         int32_t k_padded, int32_t input_dim1, void* stream) {
  (void)k_padded;
  indexed_q81("launch_indexed_moe_forward_q4k_q8_1", HQ_FMT_Q4_K, all_weights, all_inputs, indices, all_outputs, n, k,
              batch, topk, input_dim1, stream);
}
void launch_indexed_moe_forward_q8_0_q8_1(const void* all_weights, const void* all_inputs, const uint32_t* indices,
                                          float* all_outputs, int32_t n, int32_t k, int32_t batch, int32_t topk,
                                          int32_t k_padded, int32_t input_dim1, void* stream) {
  (void)k_padded;
  indexed_q81("launch_indexed_moe_forward_q8_0_q8_1", HQ_FMT_Q8_0, all_weights, all_inputs, indices, all_outputs, n, k,
              batch, topk, input_dim1, stream);
}

void launch_fp8_matmul_f16(const void* input, const void* weight, const float* weight_scale, void* output, int32_t m,
                           int32_t n, int32_t k, int32_t scale_row_stride, int32_t by, int32_t bx, void* stream) {
  fp8_matmul("launch_fp8_matmul_f16", HQ_DT_F16, input, weight, weight_scale, output, m, n, k, scale_row_stride, by, bx,
             stream);
}
void launch_fp8_matmul_bf16(const void* input, const void* weight, const float* weight_scale, void* output, int32_t m,
                            int32_t n, int32_t k, int32_t scale_row_stride, int32_t by, int32_t bx, void* stream) {
  fp8_matmul("launch_fp8_matmul_bf16", HQ_DT_BF16, input, weight, weight_scale, output, m, n, k, scale_row_stride, by,
             bx, stream);
}
void launch_fp8_indexed_moe_gemm_f16(const void* input, const void* weights, const float* weight_scales,
                                     const uint32_t* indices, void* output, int32_t num_tokens, int32_t topk,
                                     int32_t num_experts, int32_t n, int32_t k, int32_t scale_row_stride, int32_t by,
                                     int32_t bx, bool input_has_topk_dim, void* stream) {
  fp8_indexed("launch_fp8_indexed_moe_gemm_f16", HQ_DT_F16, input, weights, weight_scales, indices, output, num_tokens,
              topk, num_experts, n, k, scale_row_stride, by, bx, input_has_topk_dim, stream);
}
void launch_fp8_indexed_moe_gemm_bf16(const void* input, const void* weights, const float* weight_scales,
                                      const uint32_t* indices, void* output, int32_t num_tokens, int32_t topk,
                                      int32_t num_experts, int32_t n, int32_t k, int32_t scale_row_stride, int32_t by,
                                      int32_t bx, bool input_has_topk_dim, void* stream) {
  fp8_indexed("launch_fp8_indexed_moe_gemm_bf16", HQ_DT_BF16, input, weights, weight_scales, indices, output,
              num_tokens, topk, num_experts, n, k, scale_row_stride, by, bx, input_has_topk_dim, stream);
}

#define HQ_BLOCK_DEQ(name, dt)                                                                                  \
  void name(const void* d_weight, const float* d_scale, void* d_output, int32_t h, int32_t w, int32_t row_stride, \
            int32_t scale_stride, int32_t by, int32_t bx, void* stream) {                                       \
    block_dequant(#name, dt, d_weight, d_scale, d_output, h, w, row_stride, scale_stride, by, bx, stream);      \
  }
#define HQ_BLOCK_Q(name, dt)                                                                                  \
  void name(const void* d_input, void* d_weight, float* d_scale, int32_t h, int32_t w, int32_t row_stride,     \
            int32_t scale_stride, int32_t by, int32_t bx, void* stream) {                                      \
    block_quant(#name, dt, d_input, d_weight, d_scale, h, w, row_stride, scale_stride, by, bx, stream);        \
  }
HQ_BLOCK_DEQ(launch_dequant_fp8_blockwise_kernel_f32, HQ_DT_F32)
HQ_BLOCK_DEQ(launch_dequant_fp8_blockwise_kernel_f16, HQ_DT_F16)
HQ_BLOCK_DEQ(launch_dequant_fp8_blockwise_kernel_bf16, HQ_DT_BF16)
HQ_BLOCK_Q(launch_quant_fp8_blockwise_kernel_f32, HQ_DT_F32)
HQ_BLOCK_Q(launch_quant_fp8_blockwise_kernel_f16, HQ_DT_F16)
HQ_BLOCK_Q(launch_quant_fp8_blockwise_kernel_bf16, HQ_DT_BF16)

#define HQ_VEC_DEQ(name, dt)                                                                                  \
  void name(const void* d_weight, const float* d_scale, void* d_output, size_t num_elements, void* stream) { \
    const int32_t rc = hq_fp8_vector_dequant(static_cast<const uint8_t*>(d_weight), d_scale, (int64_t)num_elements, \
                                             d_output, dt, stream);                                           \
    if (rc != HQ_OK) complain(#name, rc);                                                                     \
  }
#define HQ_VEC_Q(name, dt)                                                                                   \
  void name(const void* d_input, void* d_weight, float* d_scale, size_t num_elements, void* stream) {        \
    const int32_t rc = hq_fp8_vector_quant(d_input, dt, (int64_t)num_elements, static_cast<uint8_t*>(d_weight), \
                                           d_scale, stream);                                                  \
    if (rc != HQ_OK) complain(#name, rc);                                                                     \
  }
HQ_VEC_DEQ(launch_dequant_fp8_vector_kernel_f32, HQ_DT_F32)
HQ_VEC_DEQ(launch_dequant_fp8_vector_kernel_f16, HQ_DT_F16)
HQ_VEC_DEQ(launch_dequant_fp8_vector_kernel_bf16, HQ_DT_BF16)
HQ_VEC_Q(launch_quant_fp8_vector_kernel_f32, HQ_DT_F32)
HQ_VEC_Q(launch_quant_fp8_vector_kernel_f16, HQ_DT_F16)
HQ_VEC_Q(launch_quant_fp8_vector_kernel_bf16, HQ_DT_BF16)

#define HQ_MX_MATMUL(name, dt)                                                                                    \
  void name(const void* input, const uint8_t* weight, const uint8_t* weight_scale, const void* bias, void* output, \
            int32_t m, int32_t n, int32_t k, bool has_bias, void* stream) {                                       \
    mxfp4_matmul(#name, dt, input, weight, weight_scale, bias, output, m, n, k, has_bias, stream);                \
  }
HQ_MX_MATMUL(launch_mxfp4_matmul_f16, HQ_DT_F16)
HQ_MX_MATMUL(launch_mxfp4_matmul_bf16, HQ_DT_BF16)
HQ_MX_MATMUL(launch_mxfp4_matmul_wmma_f16, HQ_DT_F16)
HQ_MX_MATMUL(launch_mxfp4_matmul_wmma_bf16, HQ_DT_BF16)
#define HQ_MX_MOE(name, dt)                                                                                      \
  void name(const void* input, const uint8_t* weights, const uint8_t* weight_scales, const void* biases,         \
            const uint32_t* indices, void* output, int32_t num_tokens, int32_t topk, int32_t num_experts, int32_t n, \
            int32_t k, bool has_bias, bool input_has_topk_dim, void* stream) {                                   \
    mxfp4_moe(#name, dt, input, weights, weight_scales, biases, indices, output, num_tokens, topk, num_experts, n, k, \
              has_bias, input_has_topk_dim, stream);                                                             \
  }
HQ_MX_MOE(launch_mxfp4_indexed_moe_gemm_f16, HQ_DT_F16)
HQ_MX_MOE(launch_mxfp4_indexed_moe_gemm_bf16, HQ_DT_BF16)
HQ_MX_MOE(launch_mxfp4_moe_grouped_gemm_f16, HQ_DT_F16)
HQ_MX_MOE(launch_mxfp4_moe_grouped_gemm_bf16, HQ_DT_BF16)
HQ_MX_MOE(launch_mxfp4_moe_grouped_gemm_wmma_f16, HQ_DT_F16)
HQ_MX_MOE(launch_mxfp4_moe_grouped_gemm_wmma_bf16, HQ_DT_BF16)

int32_t mxfp4_get_max_smem_optin(void) {
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return 0;
  return v;
}

#define HQ_ROUTER(name, dt)                                                                                       \
  void name(const void* logits, void* weights, void* ids, const void* selection_bias, const void* expert_scale,   \
            int32_t nrows, int32_t n_experts, int32_t top_k, int32_t score_mode, int32_t weight_mode,              \
            bool renormalize, bool clamp_logits, float clamp_min, float clamp_max, float norm_min, float output_scale, \
            int64_t stream) {                                                                                     \
    router(#name, dt, logits, weights, ids, selection_bias, expert_scale, nrows, n_experts, top_k, score_mode,    \
           weight_mode, renormalize, clamp_logits, clamp_min, clamp_max, norm_min, output_scale, stream);         \
  }
HQ_ROUTER(moe_router_topk_f32, HQ_DT_F32)
HQ_ROUTER(moe_router_topk_bf16, HQ_DT_BF16)
HQ_ROUTER(moe_router_topk_f16, HQ_DT_F16)

void gptoss_swiglu_f16(const void* gate, const void* up, void* output, uint32_t n, float alpha, float limit, void* stream) {
  gptoss("gptoss_swiglu_f16", HQ_DT_F16, gate, up, output, n, 0, alpha, limit, stream);
}
void gptoss_swiglu_bf16(const void* gate, const void* up, void* output, uint32_t n, float alpha, float limit, void* stream) {
  gptoss("gptoss_swiglu_bf16", HQ_DT_BF16, gate, up, output, n, 0, alpha, limit, stream);
}
void gptoss_swiglu_f32(const void* gate, const void* up, void* output, uint32_t n, float alpha, float limit, void* stream) {
  gptoss("gptoss_swiglu_f32", HQ_DT_F32, gate, up, output, n, 0, alpha, limit, stream);
}
void gptoss_swiglu_interleaved_f16(const void* gate_up, void* output, uint32_t n, uint32_t intermediate_size, float alpha,
                                   float limit, void* stream) {
  gptoss("gptoss_swiglu_interleaved_f16", HQ_DT_F16, gate_up, nullptr, output, n * intermediate_size, 1, alpha, limit,
         stream);
}
void gptoss_swiglu_interleaved_bf16(const void* gate_up, void* output, uint32_t n, uint32_t intermediate_size,
                                    float alpha, float limit, void* stream) {
  gptoss("gptoss_swiglu_interleaved_bf16", HQ_DT_BF16, gate_up, nullptr, output, n * intermediate_size, 1, alpha,
         limit, stream);
}
void gptoss_swiglu_interleaved_f32(const void* gate_up, void* output, uint32_t n, uint32_t intermediate_size, float alpha,
                                   float limit, void* stream) {
  gptoss("gptoss_swiglu_interleaved_f32", HQ_DT_F32, gate_up, nullptr, output, n * intermediate_size, 1, alpha, limit,
         stream);
}
void fused_glu_f16(const void* a, const void* b, void* output, uint32_t n, int32_t activation, void* stream) {
  glu("fused_glu_f16", HQ_DT_F16, a, b, output, n, activation, stream);
}
void fused_glu_bf16(const void* a, const void* b, void* output, uint32_t n, int32_t activation, void* stream) {
  glu("fused_glu_bf16", HQ_DT_BF16, a, b, output, n, activation, stream);
}
void fused_glu_f32(const void* a, const void* b, void* output, uint32_t n, int32_t activation, void* stream) {
  glu("fused_glu_f32", HQ_DT_F32, a, b, output, n, activation, stream);
}

}  // extern "C"
