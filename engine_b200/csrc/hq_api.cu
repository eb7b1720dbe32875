// C ABI entry points: argument validation on the host, then kernel launches on
// the caller's stream.  Nothing here allocates or synchronises.
#include "hq_common.cuh"
#include "hq_kernels.h"

using namespace hq;

namespace {

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
bool valid_dtype(int d) { return d == HQ_DT_F32 || d == HQ_DT_F16 || d == HQ_DT_BF16; }

int64_t weight_row_bytes(int format, int64_t k) {
  switch (format) {
    case HQ_FMT_Q8_0: return k / 32 * 34;
    case HQ_FMT_Q4_K: return k / 256 * 144;
    case HQ_FMT_FP8_BLOCK: return k;
    case HQ_FMT_MXFP4: return k / 2;
    case HQ_FMT_Q6_K: return k / 256 * 210;
    case HQ_FMT_Q5_K: return k / 256 * 176;
    case HQ_FMT_Q4_0: return k / 32 * 18;
    case HQ_FMT_Q5_0: return k / 32 * 22;
    case HQ_FMT_Q4_1: return k / 32 * 20;
    case HQ_FMT_Q5_1: return k / 32 * 24;
    case HQ_FMT_Q2_K: return k / 256 * 84;
    case HQ_FMT_Q3_K: return k / 256 * 110;
    default: return -1;
  }
}

int32_t check_weight(const hq_weight* w) {
  if (w == nullptr || w->data == nullptr) return HQ_ERR_NULL;
  if (w->n <= 0 || w->k <= 0 || w->n_experts <= 0) return HQ_ERR_SHAPE;
  if (w->n > (1ll << 30) || w->k > (1ll << 30)) return HQ_ERR_SHAPE;
  switch (w->format) {
    case HQ_FMT_Q8_0:
    case HQ_FMT_Q4_K:
    case HQ_FMT_Q6_K:
    case HQ_FMT_Q5_K:
    case HQ_FMT_Q4_0:
    case HQ_FMT_Q5_0:
    case HQ_FMT_Q4_1:
    case HQ_FMT_Q5_1:
    case HQ_FMT_Q2_K:
    case HQ_FMT_Q3_K:
      if (w->k % 256 != 0) return HQ_ERR_SHAPE;
      break;
    case HQ_FMT_FP8_BLOCK:
      if (w->k % 128 != 0) return HQ_ERR_SHAPE;
      if (w->scales == nullptr) return HQ_ERR_NULL;
      break;
    case HQ_FMT_MXFP4:
      if (w->k % 32 != 0) return HQ_ERR_SHAPE;
      if (w->scales == nullptr) return HQ_ERR_NULL;
      break;
    default:
      return HQ_ERR_FORMAT;
  }
  if (!aligned16(w->data)) return HQ_ERR_ALIGN;
  // Q6_K, Q3_K and Q2_K rows (210, 110, 84 bytes per super-block) are only 2- or 4-byte aligned; their kernels read
  // 16-bit fields and aligned words
  const bool narrow_rows = w->format == HQ_FMT_Q6_K || w->format == HQ_FMT_Q3_K || w->format == HQ_FMT_Q2_K;
  if (!narrow_rows && weight_row_bytes(w->format, w->k) % 16 != 0) return HQ_ERR_ALIGN;
  if (w->bias != nullptr && !valid_dtype(w->bias_dtype)) return HQ_ERR_FORMAT;
  return HQ_OK;
}

int64_t g_cfg[6] = {8, 9, 1 << 22, 0, 2, 0};

void fill_grouped(GroupedParams& g, const hq_weight* w, const hq_weight* w_up) {
  g.format = w->format;
  g.n = (int)w->n;
  g.k = (int)w->k;
  g.w = w->data;
  g.scales = w->scales;
  g.bias = w->bias;
  g.bias_dtype = w->bias_dtype;
  g.w_up = w_up ? w_up->data : nullptr;
  g.scales_up = w_up ? w_up->scales : nullptr;
  g.bias_up = w_up ? w_up->bias : nullptr;
  g.w_row_bytes = weight_row_bytes(w->format, w->k);
  g.fp8_tile_scale = (const float*)w->fp8_tile_scale;
  g.fp8_rel_scale = (const float*)w->fp8_rel_scale;
  g.fp8_tile_scale_up = w_up ? (const float*)w_up->fp8_tile_scale : nullptr;
  g.fp8_rel_scale_up = w_up ? (const float*)w_up->fp8_rel_scale : nullptr;
  g.fp8_nb = (int)((w->n + 127) / 128);
  g.fp8_kb = (int)((w->k + 127) / 128);
}

// Row counts from which a call goes to the tensor-core grouped GEMM.  Q8_0's decode kernel streams at HBM speed,
// so re-reading the weights once per 8 rows stays cheaper than expanding them for longer: four times the
// configured thresholds.
int64_t dense_tensor_min_rows(int format) {
  return g_cfg[HQ_CFG_DENSE_TENSOR_MIN_ROWS] * (format == HQ_FMT_Q8_0 ? 4 : 1);
}
int64_t moe_tensor_min_rows(int format) {
  return g_cfg[HQ_CFG_MOE_TENSOR_MIN_ROWS] * (format == HQ_FMT_Q8_0 ? 4 : 1);
}

// the tensor-core kernel takes f16 activation rows (it copies them into its operand tiles); hosts holding bf16 or
// f32 activations cast once per call (cheaper than converting every gathered copy of a row)
bool tensor_path_ok(const hq_weight* w, const hq_weight* w_up, int x_dtype, int64_t x_stride) {
  if (x_dtype != HQ_DT_F16 || (x_stride % 8) != 0) return false;
  if (!grouped_gemm_supported(w->format, w->n, w->k)) return false;
  if (w->format == HQ_FMT_FP8_BLOCK) {
    if (w->fp8_tile_scale == nullptr || w->fp8_rel_scale == nullptr) return false;
    if (w_up != nullptr && (w_up->fp8_tile_scale == nullptr || w_up->fp8_rel_scale == nullptr)) return false;
  }
  return true;
}

void fill_weight(GemvParams& p, const hq_weight* w, const hq_weight* w_up) {
  p.format = w->format;
  p.n = (int)w->n;
  p.k = (int)w->k;
  p.w = w->data;
  p.scales = w->scales;
  p.bias = w->bias;
  p.bias_dtype = w->bias_dtype;
  p.w_up = w_up ? w_up->data : nullptr;
  p.scales_up = w_up ? w_up->scales : nullptr;
  p.bias_up = w_up ? w_up->bias : nullptr;
  p.n_banks = w_up ? 2 : 1;
  p.w_expert_stride = w->n * weight_row_bytes(w->format, w->k);
  if (w->format == HQ_FMT_FP8_BLOCK) p.scale_expert_stride = ((w->n + 127) / 128) * ((w->k + 127) / 128);
  else if (w->format == HQ_FMT_MXFP4) p.scale_expert_stride = w->n * (w->k / 32);
  else p.scale_expert_stride = 0;
}

}  // namespace

extern "C" {

int32_t hq_abi_version(void) { return HQ_ABI_VERSION; }

const char* hq_error_string(int32_t code) {
  switch (code) {
    case HQ_OK: return "ok";
    case HQ_ERR_NULL: return "required pointer is NULL";
    case HQ_ERR_SHAPE: return "unsupported size";
    case HQ_ERR_ALIGN: return "pointer or stride not 16-byte aligned";
    case HQ_ERR_FORMAT: return "unknown format, dtype or mode";
    case HQ_ERR_CUDA: return "CUDA launch failed";
    case HQ_ERR_WORKSPACE: return "workspace missing or too small";
    case HQ_ERR_TOO_LARGE: return "size beyond the fixed maximum of this entry point";
    default: return "unknown status";
  }
}

int32_t hq_config_set(int32_t key, int64_t value) {
  if (key < 0 || key > 5 || value < 0) return HQ_ERR_FORMAT;
  if (key == HQ_CFG_FP8_LOAD_BURST && value != 1 && value != 2 && value != 4) return HQ_ERR_FORMAT;
  if (key == HQ_CFG_SPIN_LIMIT && (value < 1 || value > (1ll << 31) - 1)) return HQ_ERR_FORMAT;
  g_cfg[key] = value;
  return HQ_OK;
}

int64_t hq_config_get(int32_t key) { return (key < 0 || key > 5) ? -1 : g_cfg[key]; }

int32_t hq_status_read(const int32_t* status_dev, int32_t out_host[4], void* stream) {
  if (status_dev == nullptr || out_host == nullptr) return HQ_ERR_NULL;
  cudaStream_t s = (cudaStream_t)stream;
  if (cudaMemcpyAsync(out_host, status_dev, 4 * sizeof(int32_t), cudaMemcpyDeviceToHost, s) != cudaSuccess)
    return HQ_ERR_CUDA;
  if (cudaStreamSynchronize(s) != cudaSuccess) return HQ_ERR_CUDA;
  return HQ_OK;
}

int64_t hq_linear_workspace_bytes(const hq_weight* w, int64_t m) {
  if (check_weight(w) != HQ_OK || m <= 0) return 0;
  if (w->n_experts != 1) return 0;
  if ((w->format == HQ_FMT_Q4_K || w->format == HQ_FMT_FP8_BLOCK || w->format == HQ_FMT_Q8_0) &&
      m >= dense_tensor_min_rows(w->format))
    return 0;   // tensor-core path
  return gemv_int8_workspace_bytes(w->format, w->n, w->k, m);
}

int32_t hq_linear_forward_ws(const hq_weight* w, const void* x, int32_t x_dtype, int64_t x_stride, void* y,
                             int32_t y_dtype, int64_t y_stride, int64_t m, void* workspace, int64_t workspace_bytes,
                             int32_t* status_dev, void* stream) {
  int32_t rc = check_weight(w);
  if (rc != HQ_OK) return rc;
  if (m < 0 || m > (1 << 24)) return HQ_ERR_SHAPE;
  if (m == 0) return HQ_OK;
  if (x == nullptr || y == nullptr) return HQ_ERR_NULL;
  if (!valid_dtype(x_dtype) || !valid_dtype(y_dtype)) return HQ_ERR_FORMAT;
  if (!aligned16(x) || (x_stride * dtype_size(x_dtype)) % 16 != 0) return HQ_ERR_ALIGN;
  if (x_stride < w->k || y_stride < w->n) return HQ_ERR_SHAPE;
  if (workspace != nullptr && (workspace_bytes < 0 || ((uintptr_t)workspace & 255u) != 0)) return HQ_ERR_ALIGN;
  if (m >= dense_tensor_min_rows(w->format) && w->n_experts == 1 && tensor_path_ok(w, nullptr, x_dtype, x_stride)) {
    GroupedParams g{};
    fill_grouped(g, w, nullptr);
    g.m = (int)m;
    g.x = x; g.x_dtype = x_dtype; g.x_stride = x_stride;
    g.y = y; g.y_dtype = y_dtype; g.y_stride = y_stride;
    g.act.act = HQ_ACT_NONE;
    g.status = status_dev;
    g.tile_rows = m >= 512 ? 256 : 128;
    g.weights_in_tmem = w->format != HQ_FMT_FP8_BLOCK && w->format != HQ_FMT_Q8_0;
    return launch_grouped_gemm(g, (int)((m + g.tile_rows - 1) / g.tile_rows), (cudaStream_t)stream);
  }
  GemvParams p{};
  fill_weight(p, w, nullptr);
  p.m = (int)m;
  p.x = x; p.x_dtype = x_dtype; p.x_stride = x_stride;
  p.y = y; p.y_dtype = y_dtype; p.y_stride = y_stride;
  p.act.act = HQ_ACT_NONE;
  p.status = status_dev;
  p.workspace = workspace;
  p.workspace_bytes = workspace != nullptr ? workspace_bytes : 0;
  return launch_gemv(p, (int)((m + 7) / 8), (cudaStream_t)stream);
}

int32_t hq_linear_forward(const hq_weight* w, const void* x, int32_t x_dtype, int64_t x_stride, void* y,
                          int32_t y_dtype, int64_t y_stride, int64_t m, int32_t* status_dev, void* stream) {
  return hq_linear_forward_ws(w, x, x_dtype, x_stride, y, y_dtype, y_stride, m, nullptr, 0, status_dev, stream);
}

// ---- fused dense decode set ----------------------------------------------------------------------------
int32_t hq_linear_glu_forward(const hq_weight* w_gate, const hq_weight* w_up, const hq_act_args* act, const void* x,
                              int32_t x_dtype, int64_t x_stride, void* y, int32_t y_dtype, int64_t y_stride, int64_t m,
                              int32_t* status_dev, void* stream) {
  int32_t rc = check_weight(w_gate);
  if (rc != HQ_OK) return rc;
  if (w_up != nullptr) {
    rc = check_weight(w_up);
    if (rc != HQ_OK) return rc;
    if (w_up->format != w_gate->format || w_up->n != w_gate->n || w_up->k != w_gate->k) return HQ_ERR_SHAPE;
  } else if (w_gate->n % 2 != 0) {
    return HQ_ERR_SHAPE;
  }
  if (w_gate->n_experts != 1 || (w_up != nullptr && w_up->n_experts != 1)) return HQ_ERR_SHAPE;
  if (act == nullptr) return HQ_ERR_NULL;
  if (act->act != HQ_ACT_SWIGLU && act->act != HQ_ACT_GPTOSS) return HQ_ERR_FORMAT;
  if (m < 0 || m > (1 << 24)) return HQ_ERR_SHAPE;
  if (m == 0) return HQ_OK;
  if (x == nullptr || y == nullptr) return HQ_ERR_NULL;
  if (!valid_dtype(x_dtype) || !valid_dtype(y_dtype)) return HQ_ERR_FORMAT;
  if (!aligned16(x) || (x_stride * dtype_size(x_dtype)) % 16 != 0) return HQ_ERR_ALIGN;
  const int64_t n_out = w_up != nullptr ? w_gate->n : w_gate->n / 2;
  if (x_stride < w_gate->k || y_stride < n_out) return HQ_ERR_SHAPE;
  if (m >= dense_tensor_min_rows(w_gate->format) && tensor_path_ok(w_gate, w_up, x_dtype, x_stride)) {
    GroupedParams g{};
    fill_grouped(g, w_gate, w_up);
    g.m = (int)m;
    g.x = x; g.x_dtype = x_dtype; g.x_stride = x_stride;
    g.y = y; g.y_dtype = y_dtype; g.y_stride = y_stride;
    g.act = *act;
    g.status = status_dev;
    g.tile_rows = 128;
    g.weights_in_tmem = w_gate->format != HQ_FMT_FP8_BLOCK;
    return launch_grouped_gemm(g, (int)((m + 127) / 128), (cudaStream_t)stream);
  }
  GemvParams p{};
  fill_weight(p, w_gate, w_up);
  p.m = (int)m;
  p.x = x; p.x_dtype = x_dtype; p.x_stride = x_stride;
  p.y = y; p.y_dtype = y_dtype; p.y_stride = y_stride;
  p.act = *act;
  p.status = status_dev;
  return launch_gemv(p, (int)((m + 7) / 8), (cudaStream_t)stream);
}

int32_t hq_linear_qkv_forward(const hq_weight* w_q, const hq_weight* w_k, const hq_weight* w_v, const void* x,
                              int32_t x_dtype, int64_t x_stride, void* q, void* k, void* v, int32_t y_dtype,
                              int64_t m, int32_t* status_dev, void* stream) {
  if (w_q == nullptr || w_k == nullptr || w_v == nullptr) return HQ_ERR_NULL;
  if (w_q->k != w_k->k || w_q->k != w_v->k) return HQ_ERR_SHAPE;
  int32_t rc = hq_linear_forward(w_q, x, x_dtype, x_stride, q, y_dtype, w_q->n, m, status_dev, stream);
  if (rc == HQ_OK) rc = hq_linear_forward(w_k, x, x_dtype, x_stride, k, y_dtype, w_k->n, m, status_dev, stream);
  if (rc == HQ_OK) rc = hq_linear_forward(w_v, x, x_dtype, x_stride, v, y_dtype, w_v->n, m, status_dev, stream);
  return rc;
}

int32_t hq_dense_gemv(const void* w, int32_t w_dtype, int64_t n, int64_t k, const void* bias, int32_t bias_dtype,
                      const void* x, int32_t x_dtype, int64_t x_stride, void* y, int32_t y_dtype, int64_t y_stride,
                      int64_t m, void* stream) {
  if (n < 1 || k < 8 || k % 8 != 0 || m < 0 || m > 8 || x_stride < k || y_stride < n) return HQ_ERR_SHAPE;
  if (m == 0) return HQ_OK;
  if (w == nullptr || x == nullptr || y == nullptr) return HQ_ERR_NULL;
  if (!valid_dtype(w_dtype) || !valid_dtype(x_dtype) || !valid_dtype(y_dtype)) return HQ_ERR_FORMAT;
  if (bias != nullptr && !valid_dtype(bias_dtype)) return HQ_ERR_FORMAT;
  if (!aligned16(w) || (k * dtype_size(w_dtype)) % 16 != 0) return HQ_ERR_ALIGN;
  return launch_dense_gemv(w, w_dtype, n, k, bias, bias_dtype, x, x_dtype, x_stride, y, y_dtype, y_stride, (int)m,
                           (cudaStream_t)stream);
}

int32_t hq_router_topk(const void* logits, int32_t logits_dtype, int64_t n_rows, const hq_router_args* args,
                       uint32_t* ids_out, float* weights_out, void* stream) {
  if (args == nullptr) return HQ_ERR_NULL;
  if (n_rows < 0) return HQ_ERR_SHAPE;
  if (n_rows == 0) return HQ_OK;
  if (logits == nullptr || ids_out == nullptr || weights_out == nullptr) return HQ_ERR_NULL;
  if (!valid_dtype(logits_dtype)) return HQ_ERR_FORMAT;
  if (args->n_experts < 1 || args->n_experts > 1024) return HQ_ERR_SHAPE;
  if (args->top_k < 1 || args->top_k > 32 || args->top_k > args->n_experts) return HQ_ERR_SHAPE;
  if (args->score_mode < 0 || args->score_mode > 2 || args->weight_mode < 0 || args->weight_mode > 2)
    return HQ_ERR_FORMAT;
  return launch_router(logits, logits_dtype, n_rows, *args, 1, 1, 0, ids_out, weights_out, (cudaStream_t)stream);
}

int32_t hq_router_topk_grouped(const void* logits, int32_t logits_dtype, int64_t n_rows, const hq_router_args* args,
                               int32_t n_group, int32_t topk_group, int32_t group_score_mode, uint32_t* ids_out,
                               float* weights_out, void* stream) {
  if (args == nullptr) return HQ_ERR_NULL;
  if (n_group < 1 || n_group > 32 || topk_group < 1 || topk_group > n_group) return HQ_ERR_SHAPE;
  if (args->n_experts % n_group != 0) return HQ_ERR_SHAPE;
  if (group_score_mode != 0 && group_score_mode != 1) return HQ_ERR_FORMAT;
  if (group_score_mode == 0 && n_group > 1 && args->n_experts / n_group < 2) return HQ_ERR_SHAPE;
  if ((int64_t)topk_group * (args->n_experts / n_group) < args->top_k) return HQ_ERR_SHAPE;
  const int32_t rc = hq_router_topk(nullptr, logits_dtype, 0, args, ids_out, weights_out, stream);   // argument checks
  if (rc != HQ_OK) return rc;
  if (n_rows < 0) return HQ_ERR_SHAPE;
  if (n_rows == 0) return HQ_OK;
  if (logits == nullptr || ids_out == nullptr || weights_out == nullptr) return HQ_ERR_NULL;
  if (!valid_dtype(logits_dtype)) return HQ_ERR_FORMAT;
  if (args->n_experts < 1 || args->n_experts > 1024) return HQ_ERR_SHAPE;
  if (args->top_k < 1 || args->top_k > 32 || args->top_k > args->n_experts) return HQ_ERR_SHAPE;
  if (args->score_mode < 0 || args->score_mode > 2 || args->weight_mode < 0 || args->weight_mode > 2)
    return HQ_ERR_FORMAT;
  return launch_router(logits, logits_dtype, n_rows, *args, n_group, topk_group, group_score_mode, ids_out, weights_out,
                       (cudaStream_t)stream);
}

int64_t hq_moe_dispatch_workspace_bytes(int64_t n_tokens, int32_t top_k, int32_t n_experts) {
  if (n_tokens < 0 || top_k < 1 || n_experts < 1) return -1;
  return dispatch_layout(n_tokens, top_k, n_experts).total_words * 4;
}

int32_t hq_moe_dispatch_build(const uint32_t* ids, int64_t n_tokens, int32_t top_k, int32_t n_experts,
                              int32_t* expert_bounds, int32_t* sorted_assign, int32_t* sorted_token,
                              int32_t* inv_perm, void* workspace, int64_t workspace_bytes, void* stream) {
  if (n_tokens < 0 || top_k < 1 || top_k > 64 || n_experts < 1 || n_experts > 4096) return HQ_ERR_SHAPE;
  if (n_tokens * top_k > (1ll << 30)) return HQ_ERR_SHAPE;
  if (expert_bounds == nullptr || workspace == nullptr) return HQ_ERR_NULL;
  if (n_tokens > 0 && (ids == nullptr || sorted_assign == nullptr || sorted_token == nullptr || inv_perm == nullptr))
    return HQ_ERR_NULL;
  if (workspace_bytes < hq_moe_dispatch_workspace_bytes(n_tokens, top_k, n_experts)) return HQ_ERR_WORKSPACE;
  return launch_dispatch(ids, n_tokens, top_k, n_experts, expert_bounds, sorted_assign, sorted_token, inv_perm,
                         (int32_t*)workspace, (cudaStream_t)stream);
}

int32_t hq_moe_dispatch_build_noalloc(const uint32_t* ids, int64_t n_tokens, int32_t top_k, int32_t n_experts,
                                      int32_t* expert_bounds, int32_t* sorted_assign, int32_t* sorted_token,
                                      int32_t* inv_perm, void* stream) {
  if (n_tokens < 0 || top_k < 1 || top_k > 64 || n_experts < 1) return HQ_ERR_SHAPE;
  if (expert_bounds == nullptr) return HQ_ERR_NULL;
  if (n_tokens > 0 && (ids == nullptr || sorted_assign == nullptr || sorted_token == nullptr || inv_perm == nullptr))
    return HQ_ERR_NULL;
  return launch_dispatch_noalloc(ids, n_tokens, top_k, n_experts, expert_bounds, sorted_assign, sorted_token,
                                 inv_perm, (cudaStream_t)stream);
}

int32_t hq_moe_gather_forward(const hq_weight* w, const hq_weight* w_up, const hq_act_args* act, const void* x,
                              int32_t x_dtype, int32_t x_layout, int64_t n_tokens, int32_t top_k,
                              const int32_t* expert_bounds, const int32_t* sorted_assign,
                              const int32_t* sorted_token, const void* workspace, void* out, int32_t out_dtype,
                              int32_t out_layout, int32_t* status_dev, void* stream) {
  int32_t rc = check_weight(w);
  if (rc != HQ_OK) return rc;
  if (w_up != nullptr) {
    rc = check_weight(w_up);
    if (rc != HQ_OK) return rc;
    if (w_up->format != w->format || w_up->n != w->n || w_up->k != w->k || w_up->n_experts != w->n_experts)
      return HQ_ERR_SHAPE;
    if (act == nullptr || act->act == HQ_ACT_NONE) return HQ_ERR_FORMAT;
  }
  if (n_tokens < 0 || top_k < 1) return HQ_ERR_SHAPE;
  if (n_tokens == 0) return HQ_OK;
  if (x == nullptr || out == nullptr || expert_bounds == nullptr || sorted_assign == nullptr ||
      sorted_token == nullptr || workspace == nullptr)
    return HQ_ERR_NULL;
  if (!valid_dtype(x_dtype) || !valid_dtype(out_dtype)) return HQ_ERR_FORMAT;
  if (x_layout < 0 || x_layout > 2 || (out_layout != HQ_ROWS_PER_SLOT && out_layout != HQ_ROWS_SORTED))
    return HQ_ERR_FORMAT;
  if (!aligned16(x) || (w->k * dtype_size(x_dtype)) % 16 != 0) return HQ_ERR_ALIGN;
  const bool has_act = act != nullptr && act->act != HQ_ACT_NONE;
  if (has_act && w_up == nullptr && (w->n % 2) != 0) return HQ_ERR_SHAPE;
  const DispatchLayout l = dispatch_layout(n_tokens, top_k, w->n_experts);
  const int32_t* ws = (const int32_t*)workspace;
  const int32_t* x_rows =
      x_layout == HQ_ROWS_PER_TOKEN ? sorted_token : (x_layout == HQ_ROWS_PER_SLOT ? sorted_assign : nullptr);
  const int32_t* y_rows = out_layout == HQ_ROWS_PER_SLOT ? sorted_assign : nullptr;
  if (n_tokens * top_k >= moe_tensor_min_rows(w->format) * (int64_t)w->n_experts && tensor_path_ok(w, w_up, x_dtype, w->k)) {
    GroupedParams g{};
    fill_grouped(g, w, w_up);
    g.x = x; g.x_dtype = x_dtype; g.x_stride = w->k;
    g.y = out; g.y_dtype = out_dtype;
    g.y_stride = (has_act && w_up == nullptr) ? w->n / 2 : w->n;
    // 256-token tiles when experts hold enough rows on average to fill them and a single bank leaves tensor
    // memory for two accumulator buffers
    const bool many_rows = n_tokens * top_k >= 192 * (int64_t)w->n_experts;
    g.tile_rows = (w_up == nullptr && many_rows) ? 256 : 128;
    // the variant that expands the weights into tensor memory (128-token tiles): MXFP4 always, Q4_K while the
    // experts do not fill 256-token tiles; block-FP8 and Q8_0 expand into shared memory
    g.weights_in_tmem = w->format == HQ_FMT_MXFP4 || (w->format == HQ_FMT_Q4_K && !many_rows);
    if (w->format == HQ_FMT_MXFP4) g.tile_rows = 128;
    g.tiles = ws + (g.tile_rows == 256 ? l.off_tiles256 : l.off_tiles128);
    g.tile_count = ws + (g.tile_rows == 256 ? 3 : 1);
    g.expert_bounds = expert_bounds;
    g.x_rows = x_rows;
    g.y_rows = y_rows;
    if (has_act) g.act = *act; else g.act.act = HQ_ACT_NONE;
    g.status = status_dev;
    return launch_grouped_gemm(g, (int)(g.tile_rows == 256 ? l.max_tiles256 : l.max_tiles128), (cudaStream_t)stream);
  }
  GemvParams p{};
  fill_weight(p, w, w_up);
  p.m = 0;
  p.x = x; p.x_dtype = x_dtype; p.x_stride = w->k;
  p.y = out; p.y_dtype = out_dtype;
  p.y_stride = (has_act && w_up == nullptr) ? w->n / 2 : w->n;
  p.tiles = ws + l.off_tiles8;
  p.tile_count = ws;
  p.expert_bounds = expert_bounds;
  p.x_rows = x_rows;
  p.y_rows = y_rows;
  if (has_act) p.act = *act; else p.act.act = HQ_ACT_NONE;
  p.status = status_dev;
  return launch_gemv(p, (int)l.max_tiles8, (cudaStream_t)stream);
}

// ---- block-FP8 layers with FP8 activations (codes + 1 x 128 scales) ------------------------------------
static int32_t check_fp8_native(const hq_weight* w) {
  int32_t rc = check_weight(w);
  if (rc != HQ_OK) return rc;
  if (w->format != HQ_FMT_FP8_BLOCK) return HQ_ERR_FORMAT;
  if (!fp8_grouped_supported(w->n, w->k)) return HQ_ERR_SHAPE;
  return HQ_OK;
}
static void fill_fp8_native(Fp8GroupedParams& g, const hq_weight* w) {
  g.n = (int)w->n;
  g.k = (int)w->k;
  g.n_experts = w->n_experts;
  g.w = w->data;
  g.w_scales = (const float*)w->scales;
  g.fp8_nb = (int)((w->n + 127) / 128);
  g.fp8_kb = (int)((w->k + 127) / 128);
  g.bias = w->bias;
  g.bias_dtype = w->bias_dtype;
  g.spin_limit = (uint32_t)g_cfg[HQ_CFG_SPIN_LIMIT];
  g.test_skip_producer = (int)g_cfg[HQ_CFG_TEST_SKIP_PRODUCER];
  g.load_burst = (int)g_cfg[HQ_CFG_FP8_LOAD_BURST];
  g.load_burst_prefetch_off = g_cfg[HQ_CFG_FP8_L2_PREFETCH] == 0;
}

int32_t hq_fp8_quant_rows(const void* x, int32_t x_dtype, int64_t x_stride, const int32_t* row_map, int64_t n_rows,
                          int64_t k, uint8_t* codes, float* scales, void* stream) {
  if (n_rows < 0 || k < 128 || k % 128 != 0 || x_stride < k) return HQ_ERR_SHAPE;
  if (n_rows == 0) return HQ_OK;
  if (x == nullptr || codes == nullptr || scales == nullptr) return HQ_ERR_NULL;
  if (!valid_dtype(x_dtype)) return HQ_ERR_FORMAT;
  if (!aligned16(x) || (x_stride * dtype_size(x_dtype)) % 16 != 0) return HQ_ERR_ALIGN;
  return launch_fp8_quant_rows(x, x_dtype, x_stride, row_map, nullptr, n_rows, k, codes, scales, (cudaStream_t)stream);
}

int32_t hq_fp8_quant_rows_n(const void* x, int32_t x_dtype, int64_t x_stride, const int32_t* row_map,
                            const int32_t* n_valid_dev, int64_t n_rows, int64_t k, uint8_t* codes, float* scales,
                            void* stream) {
  if (n_rows < 0 || k < 128 || k % 128 != 0 || x_stride < k) return HQ_ERR_SHAPE;
  if (n_rows == 0) return HQ_OK;
  if (x == nullptr || codes == nullptr || scales == nullptr) return HQ_ERR_NULL;
  if (!valid_dtype(x_dtype)) return HQ_ERR_FORMAT;
  if (!aligned16(x) || (x_stride * dtype_size(x_dtype)) % 16 != 0) return HQ_ERR_ALIGN;
  return launch_fp8_quant_rows(x, x_dtype, x_stride, row_map, n_valid_dev, n_rows, k, codes, scales,
                               (cudaStream_t)stream);
}

int32_t hq_fp8_gather_rows(const uint8_t* src_codes, int64_t src_code_stride, const float* src_scales,
                           int64_t src_scale_stride_bytes, const int32_t* row_map, const int32_t* n_valid_dev,
                           int64_t n_rows, int64_t k, uint8_t* codes, float* scales, void* stream) {
  if (n_rows < 0 || k < 128 || k % 128 != 0 || src_code_stride < k || src_scale_stride_bytes < k / 32)
    return HQ_ERR_SHAPE;
  if (n_rows == 0) return HQ_OK;
  if (src_codes == nullptr || src_scales == nullptr || codes == nullptr || scales == nullptr) return HQ_ERR_NULL;
  if (!aligned16(src_codes) || !aligned16(codes) || src_code_stride % 16 != 0 || src_scale_stride_bytes % 4 != 0 ||
      (reinterpret_cast<uintptr_t>(src_scales) & 3u) != 0)
    return HQ_ERR_ALIGN;
  return launch_fp8_gather_rows(src_codes, src_code_stride, src_scales, src_scale_stride_bytes, row_map, n_valid_dev,
                                n_rows, k, codes, scales, (cudaStream_t)stream);
}

// ---- MXFP4 layers with MXFP8 activations (block-scaled MMA) ---------------------------------------------
int32_t hq_mxfp8_quant_rows(const void* x, int32_t x_dtype, int64_t x_stride, const int32_t* row_map,
                            const int32_t* n_valid_dev, int64_t n_rows, int64_t k, uint8_t* codes, uint8_t* scales,
                            void* stream) {
  if (n_rows < 0 || k < 32 || k % 32 != 0 || x_stride < k) return HQ_ERR_SHAPE;
  if (n_rows == 0) return HQ_OK;
  if (x == nullptr || codes == nullptr || scales == nullptr) return HQ_ERR_NULL;
  if (!valid_dtype(x_dtype)) return HQ_ERR_FORMAT;
  if ((reinterpret_cast<uintptr_t>(codes) & 7u) != 0) return HQ_ERR_ALIGN;
  return launch_mxfp8_quant_rows(x, x_dtype, x_stride, row_map, n_valid_dev, n_rows, k, codes, scales,
                                 (cudaStream_t)stream);
}

static int32_t fill_mx(MxGroupedParams& g, const hq_weight* w, const hq_act_args* act, const uint8_t* x_codes,
                       const uint8_t* x_scales) {
  int32_t rc = check_weight(w);
  if (rc != HQ_OK) return rc;
  if (w->format != HQ_FMT_MXFP4) return HQ_ERR_FORMAT;
  if (!mx_grouped_supported(w->n, w->k)) return HQ_ERR_SHAPE;
  if (x_codes == nullptr || x_scales == nullptr) return HQ_ERR_NULL;
  if (!aligned16(x_codes) || !aligned16(x_scales) || !aligned16(w->scales) ||
      (reinterpret_cast<uintptr_t>(w->data) & 31u) != 0)
    return HQ_ERR_ALIGN;
  g.n = (int)w->n;
  g.k = (int)w->k;
  g.n_experts = w->n_experts;
  g.w = w->data;
  g.w_scales = (const uint8_t*)w->scales;
  g.bias = w->bias;
  g.bias_dtype = w->bias_dtype;
  g.xq = x_codes;
  g.xs = x_scales;
  g.act.act = HQ_ACT_NONE;
  if (act != nullptr && act->act != HQ_ACT_NONE) {
    if (act->act != HQ_ACT_SWIGLU && act->act != HQ_ACT_GPTOSS) return HQ_ERR_FORMAT;
    if (w->n % 2 != 0) return HQ_ERR_SHAPE;
    g.act = *act;
    g.h_width = (int)(w->n / 2);
  }
  g.spin_limit = (uint32_t)g_cfg[HQ_CFG_SPIN_LIMIT];
  g.test_skip_producer = (int)g_cfg[HQ_CFG_TEST_SKIP_PRODUCER];
  return HQ_OK;
}

int32_t hq_mx_linear_forward(const hq_weight* w, const uint8_t* x_codes, const uint8_t* x_scales, int64_t m, void* y,
                             int32_t y_dtype, int64_t y_stride, int32_t* status_dev, void* stream) {
  MxGroupedParams g{};
  int32_t rc = fill_mx(g, w, nullptr, x_codes, x_scales);
  if (rc != HQ_OK) return rc;
  if (w->n_experts != 1 || m < 0 || m > (1 << 24) || y_stride < w->n) return HQ_ERR_SHAPE;
  if (m == 0) return HQ_OK;
  if (y == nullptr) return HQ_ERR_NULL;
  if (!valid_dtype(y_dtype)) return HQ_ERR_FORMAT;
  g.m = (int)m;
  g.n_rows = m;
  g.y = y; g.y_dtype = y_dtype; g.y_stride = y_stride;
  g.status = status_dev;
  return launch_mx_grouped(g, (cudaStream_t)stream);
}

int32_t hq_moe_mx_gather_forward(const hq_weight* w, const hq_act_args* act, const uint8_t* x_codes,
                                 const uint8_t* x_scales, int64_t n_tokens, int32_t top_k, const int32_t* expert_bounds,
                                 const int32_t* sorted_assign, void* out, int32_t out_dtype, int64_t out_stride,
                                 int32_t out_layout, uint8_t* h_codes, uint8_t* h_scales, int32_t* status_dev,
                                 void* stream) {
  MxGroupedParams g{};
  int32_t rc = fill_mx(g, w, act, x_codes, x_scales);
  if (rc != HQ_OK) return rc;
  if (n_tokens < 0 || top_k < 1) return HQ_ERR_SHAPE;
  if (n_tokens == 0) return HQ_OK;
  if (expert_bounds == nullptr) return HQ_ERR_NULL;
  const bool gated = g.act.act != HQ_ACT_NONE;
  const bool quantized_out = gated && h_codes != nullptr;
  if (quantized_out) {
    if (h_scales == nullptr) return HQ_ERR_NULL;
    if (g.h_width % 32 != 0 || !aligned16(h_codes)) return HQ_ERR_ALIGN;
    g.hq = h_codes;
    g.hs = h_scales;
  } else {
    if (out == nullptr) return HQ_ERR_NULL;
    if (!valid_dtype(out_dtype)) return HQ_ERR_FORMAT;
    if (out_stride < (gated ? w->n / 2 : w->n)) return HQ_ERR_SHAPE;
    if (out_layout != HQ_ROWS_PER_SLOT && out_layout != HQ_ROWS_SORTED) return HQ_ERR_FORMAT;
    if (gated && out_layout != HQ_ROWS_SORTED) return HQ_ERR_FORMAT;
    if (out_layout == HQ_ROWS_PER_SLOT && sorted_assign == nullptr) return HQ_ERR_NULL;
    g.y = out; g.y_dtype = out_dtype; g.y_stride = out_stride;
    g.y_rows = out_layout == HQ_ROWS_PER_SLOT ? sorted_assign : nullptr;
  }
  g.n_rows = n_tokens * top_k;
  g.expert_bounds = expert_bounds;
  g.status = status_dev;
  return launch_mx_grouped(g, (cudaStream_t)stream);
}

// ---- expert-parallel exchange helpers ------------------------------------------------------------------
int32_t hq_ep_layout_init(hq_ep_layout* l, int32_t world, int32_t top_k, int32_t experts_per_rank, int32_t capacity,
                          int64_t hidden, int32_t wire_dtype, int32_t fp8) {
  if (l == nullptr) return HQ_ERR_NULL;
  if (world < 1 || world > 64 || top_k < 1 || top_k > 64 || experts_per_rank < 1 || capacity < 1 ||
      capacity > (1 << 24) || hidden < 8)
    return HQ_ERR_SHAPE;
  if (fp8 ? (hidden % 512 != 0) : (hidden % 8 != 0)) return HQ_ERR_SHAPE;
  if (!fp8 && wire_dtype != HQ_DT_F16 && wire_dtype != HQ_DT_BF16) return HQ_ERR_FORMAT;
  l->world = world;
  l->top_k = top_k;
  l->experts_per_rank = experts_per_rank;
  l->capacity = capacity;
  l->fp8 = fp8 ? 1 : 0;
  l->wire_dtype = wire_dtype;
  l->hidden = hidden;
  l->row_bytes = fp8 ? hidden + hidden / 128 * 4 : hidden * 2;
  const int64_t meta = (int64_t)capacity * top_k * 8;
  l->pad_rows = (int32_t)((meta + l->row_bytes - 1) / l->row_bytes);
  l->rows_per_peer = capacity + l->pad_rows;
  l->message_bytes = (int64_t)l->rows_per_peer * l->row_bytes;
  return HQ_OK;
}

static int32_t check_ep_layout(const hq_ep_layout* l) {
  if (l == nullptr) return HQ_ERR_NULL;
  hq_ep_layout ref;
  const int32_t rc = hq_ep_layout_init(&ref, l->world, l->top_k, l->experts_per_rank, l->capacity, l->hidden,
                                       l->wire_dtype, l->fp8);
  if (rc != HQ_OK) return rc;
  if (ref.row_bytes != l->row_bytes || ref.pad_rows != l->pad_rows || ref.rows_per_peer != l->rows_per_peer ||
      ref.message_bytes != l->message_bytes)
    return HQ_ERR_SHAPE;
  return HQ_OK;
}

int32_t hq_ep_pack(const hq_ep_layout* l, const void* x, int32_t x_dtype, const uint32_t* ids, const float* weights,
                   int64_t n_tokens, void* send, int32_t* back_map, void* stream) {
  int32_t rc = check_ep_layout(l);
  if (rc != HQ_OK) return rc;
  if (n_tokens < 0 || n_tokens > l->capacity) return HQ_ERR_SHAPE;
  if (send == nullptr) return HQ_ERR_NULL;
  if (n_tokens > 0 && (x == nullptr || ids == nullptr || weights == nullptr || back_map == nullptr)) return HQ_ERR_NULL;
  if (!valid_dtype(x_dtype)) return HQ_ERR_FORMAT;
  if (!aligned16(x) || !aligned16(send)) return HQ_ERR_ALIGN;
  return launch_ep_pack(*l, x, x_dtype, ids, weights, n_tokens, send, back_map, (cudaStream_t)stream);
}

int32_t hq_ep_unpack_meta(const hq_ep_layout* l, const void* recv, uint32_t* ids_out, float* weights_out,
                          void* stream) {
  int32_t rc = check_ep_layout(l);
  if (rc != HQ_OK) return rc;
  if (recv == nullptr || ids_out == nullptr || weights_out == nullptr) return HQ_ERR_NULL;
  if (!aligned16(recv)) return HQ_ERR_ALIGN;
  return launch_ep_unpack_meta(*l, recv, ids_out, weights_out, (cudaStream_t)stream);
}

int32_t hq_ep_push(const void* send, void* const* peer_slabs_dev, int32_t world, int32_t rank, int64_t slab_bytes,
                   void* stream) {
  if (world < 1 || world > 64 || rank < 0 || rank >= world || slab_bytes < 0 || slab_bytes % 16 != 0) return HQ_ERR_SHAPE;
  if (slab_bytes == 0) return HQ_OK;
  if (send == nullptr || peer_slabs_dev == nullptr) return HQ_ERR_NULL;
  if (!aligned16(send)) return HQ_ERR_ALIGN;
  return launch_ep_push(send, peer_slabs_dev, world, rank, slab_bytes, (cudaStream_t)stream);
}

int32_t hq_ep_push_rows(const void* send, void* const* peer_slabs_dev, int32_t world, int32_t rank,
                        int32_t rows_per_slab, int64_t row_bytes, int32_t always_from, const int32_t* back_map,
                        int32_t n_tokens, const uint32_t* ids, int32_t top_k, void* stream) {
  if (world < 1 || world > 64 || rank < 0 || rank >= world || rows_per_slab < 0 || row_bytes < 0 || row_bytes % 16 != 0)
    return HQ_ERR_SHAPE;
  if (always_from < 0 || always_from > rows_per_slab) return HQ_ERR_SHAPE;
  if (rows_per_slab == 0 || row_bytes == 0) return HQ_OK;
  if (send == nullptr || peer_slabs_dev == nullptr) return HQ_ERR_NULL;
  if ((back_map == nullptr) == (ids == nullptr) && always_from > 0) return HQ_ERR_NULL;   // exactly one row filter
  if (ids != nullptr && (top_k < 1 || top_k > 64)) return HQ_ERR_SHAPE;
  if (!aligned16(send)) return HQ_ERR_ALIGN;
  return launch_ep_push_rows(send, peer_slabs_dev, world, rank, rows_per_slab, row_bytes, always_from, back_map,
                             n_tokens, ids, top_k, (cudaStream_t)stream);
}

int32_t hq_ep_barrier(int32_t* const* peer_flags_dev, int32_t world, int32_t rank, int32_t* seq_counter_dev,
                      int32_t* status_dev, void* stream) {
  if (world < 1 || world > 64 || rank < 0 || rank >= world) return HQ_ERR_SHAPE;
  if (peer_flags_dev == nullptr || seq_counter_dev == nullptr) return HQ_ERR_NULL;
  return launch_ep_barrier(peer_flags_dev, world, rank, seq_counter_dev, (uint32_t)g_cfg[HQ_CFG_SPIN_LIMIT],
                           status_dev, (cudaStream_t)stream);
}

int32_t hq_fp8_gated_quant_rows(const void* gate_up, int32_t dtype, int64_t n_rows, int64_t width,
                                const hq_act_args* act, uint8_t* codes, float* scales, void* stream) {
  if (n_rows < 0 || width < 128 || width % 128 != 0) return HQ_ERR_SHAPE;
  if (n_rows == 0) return HQ_OK;
  if (gate_up == nullptr || act == nullptr || codes == nullptr || scales == nullptr) return HQ_ERR_NULL;
  if (!valid_dtype(dtype) || act->act == HQ_ACT_NONE) return HQ_ERR_FORMAT;
  if (!aligned16(gate_up)) return HQ_ERR_ALIGN;
  return launch_fp8_gated_quant_rows(gate_up, dtype, n_rows, width, *act, codes, scales, (cudaStream_t)stream);
}

int32_t hq_fp8_linear_forward(const hq_weight* w, const uint8_t* x_codes, const float* x_scales, int64_t m, void* y,
                              int32_t y_dtype, int64_t y_stride, int32_t* status_dev, void* stream) {
  int32_t rc = check_fp8_native(w);
  if (rc != HQ_OK) return rc;
  if (w->n_experts != 1 || m < 0 || m > (1 << 24) || y_stride < w->n) return HQ_ERR_SHAPE;
  if (m == 0) return HQ_OK;
  if (x_codes == nullptr || x_scales == nullptr || y == nullptr) return HQ_ERR_NULL;
  if (!valid_dtype(y_dtype)) return HQ_ERR_FORMAT;
  if (!aligned16(x_codes) || !aligned16(x_scales)) return HQ_ERR_ALIGN;
  Fp8GroupedParams g{};
  fill_fp8_native(g, w);
  g.m = (int)m;
  g.xq = x_codes; g.xs = x_scales; g.n_rows = m;
  g.y = y; g.y_dtype = y_dtype; g.y_stride = y_stride;
  g.status = status_dev;
  return launch_fp8_grouped(g, (cudaStream_t)stream);
}

int32_t hq_moe_fp8_gather_forward(const hq_weight* w, const uint8_t* x_codes, const float* x_scales,
                                  int64_t n_tokens, int32_t top_k, const int32_t* expert_bounds,
                                  const int32_t* sorted_assign, const void* workspace, void* out, int32_t out_dtype,
                                  int64_t out_stride, int32_t out_layout, int32_t* status_dev, void* stream) {
  (void)workspace;   // the kernel cuts its token tiles from expert_bounds; the tile lists are not read any more
  int32_t rc = check_fp8_native(w);
  if (rc != HQ_OK) return rc;
  if (n_tokens < 0 || top_k < 1 || out_stride < w->n) return HQ_ERR_SHAPE;
  if (n_tokens == 0) return HQ_OK;
  if (x_codes == nullptr || x_scales == nullptr || out == nullptr || expert_bounds == nullptr) return HQ_ERR_NULL;
  if (out_layout == HQ_ROWS_PER_SLOT && sorted_assign == nullptr) return HQ_ERR_NULL;
  if (!valid_dtype(out_dtype) || (out_layout != HQ_ROWS_PER_SLOT && out_layout != HQ_ROWS_SORTED))
    return HQ_ERR_FORMAT;
  if (!aligned16(x_codes) || !aligned16(x_scales)) return HQ_ERR_ALIGN;
  Fp8GroupedParams g{};
  fill_fp8_native(g, w);
  g.xq = x_codes; g.xs = x_scales; g.n_rows = n_tokens * top_k;
  g.y = out; g.y_dtype = out_dtype; g.y_stride = out_stride;
  g.expert_bounds = expert_bounds;
  g.y_rows = out_layout == HQ_ROWS_PER_SLOT ? sorted_assign : nullptr;
  g.status = status_dev;
  return launch_fp8_grouped(g, (cudaStream_t)stream);
}

int32_t hq_moe_fp8_gate_up_forward(const hq_weight* w_gate, const hq_weight* w_up, const hq_act_args* act,
                                   const uint8_t* x_codes, const float* x_scales, int64_t n_tokens, int32_t top_k,
                                   const int32_t* expert_bounds, uint8_t* h_codes, float* h_scales,
                                   int32_t* status_dev, void* stream) {
  int32_t rc = check_fp8_native(w_gate);
  if (rc == HQ_OK) rc = check_fp8_native(w_up);
  if (rc != HQ_OK) return rc;
  if (w_up->n != w_gate->n || w_up->k != w_gate->k || w_up->n_experts != w_gate->n_experts) return HQ_ERR_SHAPE;
  if (act == nullptr) return HQ_ERR_NULL;
  if (act->act != HQ_ACT_SWIGLU && act->act != HQ_ACT_GPTOSS) return HQ_ERR_FORMAT;
  if (n_tokens < 0 || top_k < 1) return HQ_ERR_SHAPE;
  if (n_tokens == 0) return HQ_OK;
  if (x_codes == nullptr || x_scales == nullptr || h_codes == nullptr || h_scales == nullptr ||
      expert_bounds == nullptr)
    return HQ_ERR_NULL;
  if (!aligned16(x_codes) || !aligned16(x_scales) || !aligned16(h_codes)) return HQ_ERR_ALIGN;
  if (w_gate->bias != nullptr && w_up->bias != nullptr && w_gate->bias_dtype != w_up->bias_dtype) return HQ_ERR_FORMAT;
  Fp8GroupedParams g{};
  fill_fp8_native(g, w_gate);
  g.w_up = w_up->data;
  g.w_up_scales = (const float*)w_up->scales;
  g.bias_up = w_up->bias;
  if (g.bias == nullptr) g.bias_dtype = w_up->bias_dtype;
  g.xq = x_codes; g.xs = x_scales; g.n_rows = n_tokens * top_k;
  g.hq = h_codes; g.hs = h_scales;
  g.act = *act;
  g.expert_bounds = expert_bounds;
  g.status = status_dev;
  return launch_fp8_grouped(g, (cudaStream_t)stream);
}

int32_t hq_moe_weighted_reduce(const void* y, int32_t y_dtype, const float* w, const int32_t* row_map,
                               const void* addend, void* out, int32_t out_dtype, int64_t n_tokens, int32_t top_k,
                               int64_t hidden, void* stream) {
  if (n_tokens < 0 || top_k < 1 || top_k > 64 || hidden < 1) return HQ_ERR_SHAPE;
  if (n_tokens == 0) return HQ_OK;
  if (y == nullptr || w == nullptr || out == nullptr) return HQ_ERR_NULL;
  if (!valid_dtype(y_dtype) || !valid_dtype(out_dtype)) return HQ_ERR_FORMAT;
  if (!aligned16(y) || (hidden * dtype_size(y_dtype)) % 16 != 0) return HQ_ERR_ALIGN;
  return launch_weighted_reduce(y, y_dtype, w, row_map, addend, out, out_dtype, n_tokens, top_k, hidden,
                                (cudaStream_t)stream);
}

int32_t hq_fp8_vector_quant(const void* x, int32_t x_dtype, int64_t n_elems, uint8_t* codes, float* scales,
                            void* stream) {
  if (n_elems < 0 || n_elems % 128 != 0) return HQ_ERR_SHAPE;
  if (n_elems == 0) return HQ_OK;
  if (x == nullptr || codes == nullptr || scales == nullptr) return HQ_ERR_NULL;
  if (!valid_dtype(x_dtype)) return HQ_ERR_FORMAT;
  if ((reinterpret_cast<uintptr_t>(codes) & 3u) != 0) return HQ_ERR_ALIGN;
  return launch_fp8_vector_quant(x, x_dtype, n_elems, codes, scales, (cudaStream_t)stream);
}

int32_t hq_fp8_vector_dequant(const uint8_t* codes, const float* scales, int64_t n_elems, void* out,
                              int32_t out_dtype, void* stream) {
  if (n_elems < 0 || n_elems % 128 != 0) return HQ_ERR_SHAPE;
  if (n_elems == 0) return HQ_OK;
  if (codes == nullptr || scales == nullptr || out == nullptr) return HQ_ERR_NULL;
  if (!valid_dtype(out_dtype)) return HQ_ERR_FORMAT;
  return launch_fp8_vector_dequant(codes, scales, n_elems, out, out_dtype, (cudaStream_t)stream);
}

int32_t hq_fp8_block_quant(const void* w, int32_t w_dtype, int64_t rows, int64_t cols, int32_t by, int32_t bx,
                           uint8_t* codes, float* scales, void* stream) {
  if (rows < 0 || cols < 0 || by < 1 || bx < 1) return HQ_ERR_SHAPE;
  if (rows == 0 || cols == 0) return HQ_OK;
  if (w == nullptr || codes == nullptr || scales == nullptr) return HQ_ERR_NULL;
  if (!valid_dtype(w_dtype)) return HQ_ERR_FORMAT;
  if ((rows + by - 1) / by > 65535) return HQ_ERR_SHAPE;
  return launch_fp8_block_quant(w, w_dtype, rows, cols, by, bx, codes, scales, (cudaStream_t)stream);
}

int32_t hq_fp8_block_dequant(const uint8_t* codes, const float* scales, int64_t rows, int64_t cols, int32_t by,
                             int32_t bx, void* out, int32_t out_dtype, void* stream) {
  if (rows < 0 || cols < 0 || by < 1 || bx < 1) return HQ_ERR_SHAPE;
  if (rows == 0 || cols == 0) return HQ_OK;
  if (codes == nullptr || scales == nullptr || out == nullptr) return HQ_ERR_NULL;
  if (!valid_dtype(out_dtype)) return HQ_ERR_FORMAT;
  return launch_fp8_block_dequant(codes, scales, rows, cols, by, bx, out, out_dtype, (cudaStream_t)stream);
}

int32_t hq_fp8_scale_prepare(const float* scales, int32_t n_experts, int64_t n, int64_t k, float* tile_scale_out,
                             float* rel_scale_out, void* stream) {
  if (n_experts < 1 || n < 1 || k < 1) return HQ_ERR_SHAPE;
  if (scales == nullptr || tile_scale_out == nullptr || rel_scale_out == nullptr) return HQ_ERR_NULL;
  const int64_t groups = (int64_t)n_experts * ((n + 127) / 128);
  return launch_fp8_scale_prepare(scales, groups, (int)((k + 127) / 128), tile_scale_out, rel_scale_out,
                                  (cudaStream_t)stream);
}

int32_t hq_convert_status(const void* src, int32_t src_dtype, void* dst, int32_t dst_dtype, int64_t n_elems,
                          int32_t* status_dev, void* stream) {
  if (n_elems < 0) return HQ_ERR_SHAPE;
  if (n_elems == 0) return HQ_OK;
  if (src == nullptr || dst == nullptr) return HQ_ERR_NULL;
  if (!valid_dtype(src_dtype) || !valid_dtype(dst_dtype)) return HQ_ERR_FORMAT;
  return launch_convert(src, src_dtype, dst, dst_dtype, n_elems, status_dev, (cudaStream_t)stream);
}

int32_t hq_convert(const void* src, int32_t src_dtype, void* dst, int32_t dst_dtype, int64_t n_elems, void* stream) {
  return hq_convert_status(src, src_dtype, dst, dst_dtype, n_elems, nullptr, stream);
}

int32_t hq_gated_act(const void* gate, const void* up, int32_t dtype, int64_t n_elems, int32_t interleaved,
                     const hq_act_args* act, void* out, void* stream) {
  if (n_elems < 0) return HQ_ERR_SHAPE;
  if (n_elems == 0) return HQ_OK;
  if (gate == nullptr || out == nullptr || act == nullptr || (!interleaved && up == nullptr)) return HQ_ERR_NULL;
  if (!valid_dtype(dtype) || (act->act != HQ_ACT_SWIGLU && act->act != HQ_ACT_GPTOSS)) return HQ_ERR_FORMAT;
  return launch_gated_act(gate, up, dtype, n_elems, interleaved, *act, out, (cudaStream_t)stream);
}

int32_t hq_probe_tensor_peak(int32_t kind, int32_t n, int32_t iters, int32_t* status_dev, double* flops_host,
                             void* stream) {
  if (kind != 0 && kind != 1) return HQ_ERR_FORMAT;
  if (n < 16 || n > 256 || n % 16 != 0 || iters < 1 || iters > (1 << 20)) return HQ_ERR_SHAPE;
  return launch_probe_mma(kind, n, iters, status_dev, flops_host, (cudaStream_t)stream);
}

// ---- one MoE layer in one call -----------------------------------------------------------------------------
namespace {
struct MoeLayerPlan {
  int64_t t, k, e, hidden, inter, rows;
  bool interleaved, cast_x;
  int64_t off_ids, off_w, off_bounds, off_sa, off_st, off_inv, off_dws, dws_bytes, off_x16, off_h, off_y, total;
};
int64_t up256(int64_t v) { return (v + 255) / 256 * 256; }
int32_t plan_moe_layer(const hq_moe_layer* l, int64_t n_tokens, int32_t x_dtype, MoeLayerPlan& p) {
  if (l == nullptr || l->gate == nullptr || l->down == nullptr) return HQ_ERR_NULL;
  int32_t rc = check_weight(l->gate);
  if (rc == HQ_OK) rc = check_weight(l->down);
  if (rc == HQ_OK && l->up != nullptr) rc = check_weight(l->up);
  if (rc != HQ_OK) return rc;
  p.t = n_tokens;
  p.k = l->router.top_k;
  p.e = l->gate->n_experts;
  if (l->router.n_experts != p.e || l->down->n_experts != p.e || p.k < 1) return HQ_ERR_SHAPE;
  p.interleaved = l->up == nullptr;
  p.hidden = l->gate->k;
  p.inter = p.interleaved ? l->gate->n / 2 : l->gate->n;
  if (l->down->k != p.inter || l->down->n != p.hidden) return HQ_ERR_SHAPE;
  if (l->act.act == HQ_ACT_NONE) return HQ_ERR_FORMAT;
  p.rows = p.t * p.k;
  // the tensor-core kernel copies activations as f16: cast once per token here instead of per (token, slot) there
  p.cast_x = x_dtype != HQ_DT_F16 && p.rows >= moe_tensor_min_rows(l->gate->format) * p.e &&
             tensor_path_ok(l->gate, l->up, HQ_DT_F16, l->gate->k);
  int64_t o = 0;
  p.off_ids = o;    o += up256(p.rows * 4);
  p.off_w = o;      o += up256(p.rows * 4);
  p.off_bounds = o; o += up256((p.e + 1) * 4);
  p.off_sa = o;     o += up256(p.rows * 4);
  p.off_st = o;     o += up256(p.rows * 4);
  p.off_inv = o;    o += up256(p.rows * 4);
  p.dws_bytes = hq_moe_dispatch_workspace_bytes(p.t, (int32_t)p.k, (int32_t)p.e);
  p.off_dws = o;    o += up256(p.dws_bytes);
  p.off_x16 = o;    o += p.cast_x ? up256(p.t * p.hidden * 2) : 0;
  p.off_h = o;      o += up256(p.rows * p.inter * 2);
  p.off_y = o;      o += up256(p.rows * p.hidden * 4);
  p.total = o;
  return HQ_OK;
}
}  // namespace

int64_t hq_moe_layer_workspace_bytes(const hq_moe_layer* layer, int64_t n_tokens, int32_t x_dtype) {
  MoeLayerPlan p;
  if (n_tokens <= 0 || plan_moe_layer(layer, n_tokens, x_dtype, p) != HQ_OK) return 0;
  return p.total;
}

int32_t hq_moe_layer_forward(const hq_moe_layer* layer, const void* logits, int32_t logits_dtype, const void* x,
                             int32_t x_dtype, int64_t n_tokens, const void* shared_addend, void* out,
                             int32_t out_dtype, void* workspace, int64_t workspace_bytes, int32_t* status_dev,
                             void* stream) {
  if (n_tokens < 0) return HQ_ERR_SHAPE;
  if (n_tokens == 0) return HQ_OK;
  if (!valid_dtype(x_dtype) || !valid_dtype(out_dtype) || !valid_dtype(logits_dtype)) return HQ_ERR_FORMAT;
  MoeLayerPlan p;
  int32_t rc = plan_moe_layer(layer, n_tokens, x_dtype, p);
  if (rc != HQ_OK) return rc;
  if (logits == nullptr || x == nullptr || out == nullptr || workspace == nullptr) return HQ_ERR_NULL;
  if (workspace_bytes < p.total) return HQ_ERR_WORKSPACE;
  if (((uintptr_t)workspace & 255u) != 0) return HQ_ERR_ALIGN;
  uint8_t* ws = (uint8_t*)workspace;
  uint32_t* ids = (uint32_t*)(ws + p.off_ids);
  float* wts = (float*)(ws + p.off_w);
  int32_t* bounds = (int32_t*)(ws + p.off_bounds);
  int32_t* sa = (int32_t*)(ws + p.off_sa);
  int32_t* st = (int32_t*)(ws + p.off_st);
  int32_t* inv = (int32_t*)(ws + p.off_inv);
  void* dws = ws + p.off_dws;
  rc = hq_router_topk(logits, logits_dtype, n_tokens, &layer->router, ids, wts, stream);
  if (rc != HQ_OK) return rc;
  rc = hq_moe_dispatch_build(ids, n_tokens, (int32_t)p.k, (int32_t)p.e, bounds, sa, st, inv, dws, p.dws_bytes, stream);
  if (rc != HQ_OK) return rc;
  const void* xin = x;
  int32_t xin_dtype = x_dtype;
  if (p.cast_x) {
    rc = hq_convert_status(x, x_dtype, ws + p.off_x16, HQ_DT_F16, n_tokens * p.hidden, status_dev, stream);
    if (rc != HQ_OK) return rc;
    xin = ws + p.off_x16;
    xin_dtype = HQ_DT_F16;
  }
  void* h = ws + p.off_h;
  rc = hq_moe_gather_forward(layer->gate, layer->up, &layer->act, xin, xin_dtype, HQ_ROWS_PER_TOKEN, n_tokens,
                             (int32_t)p.k, bounds, sa, st, dws, h, HQ_DT_F16, HQ_ROWS_SORTED, status_dev, stream);
  if (rc != HQ_OK) return rc;
  void* y = ws + p.off_y;
  rc = hq_moe_gather_forward(layer->down, nullptr, nullptr, h, HQ_DT_F16, HQ_ROWS_SORTED, n_tokens, (int32_t)p.k,
                             bounds, sa, st, dws, y, HQ_DT_F32, HQ_ROWS_SORTED, status_dev, stream);
  if (rc != HQ_OK) return rc;
  return hq_moe_weighted_reduce(y, HQ_DT_F32, wts, inv, shared_addend, out, out_dtype, n_tokens, (int32_t)p.k,
                                p.hidden, stream);
}

}  // extern "C"
