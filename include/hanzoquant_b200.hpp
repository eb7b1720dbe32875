// C++ host layer over the C ABI of libhanzoquant_b200: the same operator interface hanzo-quant gives its
// callers -- `QuantMethod::{forward, gather_forward}` (hanzo-quant/src/lib.rs:1004-1108) implemented by
// `GgufMatMul` (src/gguf/mod.rs:31-399), `BlockwiseFP8Linear` (src/blockwise_fp8/mod.rs:24-198) and `MXFP4Layer`
// (src/mxfp4/mod.rs:29-174), `moe_router_topk` with `MoeRouterTopKConfig` (hanzo-engine/src/ops.rs:225-335) and
// the expert block `MoEExperts::forward` (hanzo-engine/src/moe/experts/mod.rs:241-266).  Header-only; link with
// -lhanzoquant_b200 -lcudart.  Errors are exceptions (the reference `bail!`s); there is no CPU path.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "hanzoquant_b200.h"

namespace hq {

struct Error : std::runtime_error {
  using std::runtime_error::runtime_error;
};
inline void check(int32_t rc, const char* what) {
  if (rc != HQ_OK) throw Error(std::string(what) + ": " + hq_error_string(rc));
}
inline void check_cuda(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw Error(std::string(what) + ": " + cudaGetErrorString(e));
}

enum class DType : int32_t { F32 = HQ_DT_F32, F16 = HQ_DT_F16, BF16 = HQ_DT_BF16, U8 = 100, I32 = 101 };
inline size_t dtype_bytes(DType d) {
  switch (d) {
    case DType::F32: case DType::I32: return 4;
    case DType::F16: case DType::BF16: return 2;
    default: return 1;
  }
}

// Device tensor: contiguous, ref-counted storage from cudaMalloc (what the reference gets from `dev.alloc`).
class Tensor {
 public:
  Tensor() = default;
  static Tensor empty(std::vector<int64_t> dims, DType dtype) {
    Tensor t;
    t.dims_ = std::move(dims);
    t.dtype_ = dtype;
    const size_t bytes = t.numel() * dtype_bytes(dtype);
    void* p = nullptr;
    if (bytes) check_cuda(cudaMalloc(&p, bytes), "cudaMalloc");
    t.buf_ = std::shared_ptr<void>(p, [](void* q) { if (q) cudaFree(q); });
    return t;
  }
  static Tensor from_host(const void* src, std::vector<int64_t> dims, DType dtype) {
    Tensor t = empty(std::move(dims), dtype);
    if (t.numel()) check_cuda(cudaMemcpy(t.data(), src, t.numel() * dtype_bytes(dtype), cudaMemcpyHostToDevice), "H2D");
    return t;
  }
  void to_host(void* dst) const {
    if (numel()) check_cuda(cudaMemcpy(dst, data(), numel() * dtype_bytes(dtype_), cudaMemcpyDeviceToHost), "D2H");
  }
  Tensor reshape(std::vector<int64_t> dims) const {
    Tensor t = *this;
    t.dims_ = std::move(dims);
    if (t.numel() != numel()) throw Error("reshape: element count mismatch");
    return t;
  }
  void* data() const { return buf_.get(); }
  const std::vector<int64_t>& dims() const { return dims_; }
  int64_t dim(int i) const { return dims_.at(i < 0 ? dims_.size() + i : i); }
  size_t rank() const { return dims_.size(); }
  DType dtype() const { return dtype_; }
  size_t numel() const {
    size_t n = 1;
    for (int64_t d : dims_) n *= (size_t)d;
    return n;
  }

 private:
  std::shared_ptr<void> buf_;
  std::vector<int64_t> dims_;
  DType dtype_ = DType::F32;
};

inline Tensor to_dtype(const Tensor& a, DType dtype, cudaStream_t stream = nullptr) {
  if (a.dtype() == dtype) return a;
  Tensor out = Tensor::empty(a.dims(), dtype);
  check(hq_convert(a.data(), (int32_t)a.dtype(), out.data(), (int32_t)dtype, (int64_t)a.numel(), stream), "hq_convert");
  return out;
}

// ---- router (hanzo-engine/src/ops.rs:194-335) -------------------------------------------------------------
enum class MoeRouterScoreFunction : int32_t { Raw = HQ_SCORE_RAW, Softmax = HQ_SCORE_SOFTMAX, Sigmoid = HQ_SCORE_SIGMOID };
enum class MoeRouterSelectedWeight : int32_t { Score = HQ_WEIGHT_SCORE, Softmax = HQ_WEIGHT_SOFTMAX, Sigmoid = HQ_WEIGHT_SIGMOID };
struct MoeRouterTopKConfig {
  size_t top_k = 1;
  MoeRouterScoreFunction score_function = MoeRouterScoreFunction::Softmax;
  MoeRouterSelectedWeight selected_weight = MoeRouterSelectedWeight::Score;
  bool renormalize = false;
  float norm_min = 0.f;
  float output_scale = 1.f;
  bool has_logit_clip = false;
  float logit_clip_min = 0.f, logit_clip_max = 0.f;
};
struct TopKOutput {
  Tensor values;   // f32 [T, k]
  Tensor indices;  // i32 [T, k] (bit pattern of the reference's u32 ids), descending selection order
};
inline TopKOutput moe_router_topk(const Tensor& logits, const MoeRouterTopKConfig& config,
                                  const Tensor* selection_bias = nullptr, const Tensor* expert_scale = nullptr,
                                  cudaStream_t stream = nullptr) {
  if (logits.rank() != 2) throw Error("moe_router_topk: logits must be [rows, experts]");
  const int64_t t = logits.dim(0), e = logits.dim(1);
  TopKOutput out{Tensor::empty({t, (int64_t)config.top_k}, DType::F32), Tensor::empty({t, (int64_t)config.top_k}, DType::I32)};
  hq_router_args a{};
  a.n_experts = (int32_t)e;
  a.top_k = (int32_t)config.top_k;
  a.score_mode = (int32_t)config.score_function;
  a.weight_mode = (int32_t)config.selected_weight;
  a.renormalize = config.renormalize;
  a.clamp_logits = config.has_logit_clip;
  a.clamp_min = config.logit_clip_min;
  a.clamp_max = config.logit_clip_max;
  a.norm_min = config.norm_min;
  a.output_scale = config.output_scale;
  a.selection_bias = selection_bias ? (const float*)selection_bias->data() : nullptr;
  a.expert_scale = expert_scale ? (const float*)expert_scale->data() : nullptr;
  check(hq_router_topk(logits.data(), (int32_t)logits.dtype(), t, &a, (uint32_t*)out.indices.data(),
                       (float*)out.values.data(), stream), "hq_router_topk");
  return out;
}

// ---- dispatch tables (hanzo-quant/src/gguf/cuda.rs:538-578) -------------------------------------------------
struct DispatchTables {
  int64_t n_tokens = 0;
  int32_t top_k = 0, n_experts = 0;
  Tensor expert_bounds, sorted_assign, sorted_token, inv_perm, workspace;
};
inline DispatchTables moe_dispatch_build(const Tensor& ids, int32_t n_experts, cudaStream_t stream = nullptr) {
  if (ids.rank() != 2 || ids.dtype() != DType::I32) throw Error("moe_dispatch_build: ids must be i32 [T, k]");
  DispatchTables d;
  d.n_tokens = ids.dim(0);
  d.top_k = (int32_t)ids.dim(1);
  d.n_experts = n_experts;
  const int64_t n = d.n_tokens * d.top_k;
  const int64_t ws = hq_moe_dispatch_workspace_bytes(d.n_tokens, d.top_k, n_experts);
  if (ws < 0) throw Error("moe_dispatch_build: bad sizes");
  d.expert_bounds = Tensor::empty({n_experts + 1}, DType::I32);
  d.sorted_assign = Tensor::empty({n}, DType::I32);
  d.sorted_token = Tensor::empty({n}, DType::I32);
  d.inv_perm = Tensor::empty({n}, DType::I32);
  d.workspace = Tensor::empty({ws / 4}, DType::I32);
  check(hq_moe_dispatch_build((const uint32_t*)ids.data(), d.n_tokens, d.top_k, n_experts, (int32_t*)d.expert_bounds.data(),
                              (int32_t*)d.sorted_assign.data(), (int32_t*)d.sorted_token.data(),
                              (int32_t*)d.inv_perm.data(), d.workspace.data(), ws, stream), "hq_moe_dispatch_build");
  return d;
}

// ---- QuantMethod (hanzo-quant/src/lib.rs:1004-1108) -----------------------------------------------------------
class QuantMethod {
 public:
  virtual ~QuantMethod() = default;
  virtual hq_weight weight() const = 0;
  // any 3-D input to gather_forward is one row per slot (MXFP4Layer, hanzo-quant/src/mxfp4/ops.rs:349-355)
  virtual bool input_3d_is_per_slot() const { return false; }

  int64_t n() const { return weight().n; }
  int64_t k() const { return weight().k; }
  int32_t n_experts() const { return weight().n_experts; }

  // y = a . W^T (+ b); leading dims flattened to rows; result in a's dtype unless out_dtype is given
  Tensor forward(const Tensor& a, cudaStream_t stream = nullptr) const { return forward_raw(a, a.dtype(), stream); }
  Tensor forward_raw(const Tensor& a, DType out_dtype, cudaStream_t stream = nullptr) const {
    const hq_weight w = weight();
    if (w.n_experts != 1) throw Error("forward on an expert bank: use gather_forward");
    if (a.rank() < 1 || a.dim(-1) != w.k) throw Error("forward: input feature count does not match the weight");
    const int64_t m = (int64_t)(a.numel() / (size_t)w.k);
    Tensor x = a;
    if (m >= hq_config_get(HQ_CFG_DENSE_TENSOR_MIN_ROWS)) x = to_dtype(a, DType::F16, stream);  // tensor-core path
    std::vector<int64_t> od(a.dims());
    od.back() = w.n;
    Tensor y = Tensor::empty(od, out_dtype);
    // scratch for the split-K form of the decode kernel, owned by the layer like the reference's Q8_1 buffer
    // (hanzo-quant/src/gguf/fast_mmvq.rs:107-148): zero-filled when (re)allocated, one stream at a time
    const int64_t need = hq_linear_workspace_bytes(&w, m);
    if (need > scratch_bytes_) {
      scratch_ = Tensor::empty({need}, DType::U8);
      check_cuda(cudaMemsetAsync(scratch_.data(), 0, (size_t)need, stream), "cudaMemsetAsync");
      scratch_bytes_ = need;
    }
    check(hq_linear_forward_ws(&w, x.data(), (int32_t)x.dtype(), w.k, y.data(), (int32_t)out_dtype, w.n, m,
                               need > 0 ? scratch_.data() : nullptr, need > 0 ? scratch_bytes_ : 0, nullptr, stream),
          "hq_linear_forward_ws");
    return y;
  }

  // per-assignment projection out of the bank: a [T, K] / [T, 1, K] (row per token) or [T, k, K] (row per slot),
  // indices i32 [T, k] -> [T, k, N]
  Tensor gather_forward(const Tensor& a, const Tensor& indices, cudaStream_t stream = nullptr) const {
    return gather_forward_raw(a, indices, a.dtype(), nullptr, stream);
  }
  Tensor gather_forward_raw(const Tensor& a, const Tensor& indices, DType out_dtype, const DispatchTables* tables = nullptr,
                            cudaStream_t stream = nullptr) const {
    const hq_weight w = weight();
    if (indices.rank() != 2) throw Error("gather_forward: indices must be [T, k]");
    const int64_t t = indices.dim(0), k = indices.dim(1);
    int32_t layout = HQ_ROWS_PER_TOKEN;
    if (a.rank() == 3 && (a.dim(1) > 1 || input_3d_is_per_slot())) {
      layout = HQ_ROWS_PER_SLOT;
      if (a.dim(1) != k) throw Error("gather_forward: per-slot input and indices disagree on top_k");
    }
    if (a.dim(0) != t || a.dim(-1) != w.k) throw Error("gather_forward: input / indices / weight shapes disagree");
    DispatchTables local;
    if (!tables) {
      local = moe_dispatch_build(indices, w.n_experts, stream);
      tables = &local;
    }
    Tensor x = a;
    if (t * k >= hq_config_get(HQ_CFG_MOE_TENSOR_MIN_ROWS) * w.n_experts) x = to_dtype(a, DType::F16, stream);
    Tensor out = Tensor::empty({t, k, w.n}, out_dtype);
    check(hq_moe_gather_forward(&w, nullptr, nullptr, x.data(), (int32_t)x.dtype(), layout, t, (int32_t)k,
                                (const int32_t*)tables->expert_bounds.data(), (const int32_t*)tables->sorted_assign.data(),
                                (const int32_t*)tables->sorted_token.data(), tables->workspace.data(), out.data(),
                                (int32_t)out_dtype, HQ_ROWS_PER_SLOT, nullptr, stream), "hq_moe_gather_forward");
    return out;
  }

 private:
  mutable Tensor scratch_;
  mutable int64_t scratch_bytes_ = 0;
};

// GGUF block-quantized linear / expert bank: `data` = raw GGUF block bytes, u8 [N, row_bytes] or [E, N, row_bytes]
class GgufMatMul : public QuantMethod {
 public:
  enum class GgmlType { Q8_0, Q4_K, Q6_K, Q5_K, Q4_0, Q5_0, Q4_1, Q5_1, Q2_K, Q3_K };
  GgufMatMul(Tensor data, GgmlType type, int64_t k, Tensor bias = Tensor()) : data_(std::move(data)), bias_(std::move(bias)) {
    if (k % 256) throw Error("GgufMatMul: K must be a multiple of 256");
    // {format, weights per block, bytes per block}
    static constexpr int32_t kTypes[10][3] = {{HQ_FMT_Q8_0, 32, 34},   {HQ_FMT_Q4_K, 256, 144}, {HQ_FMT_Q6_K, 256, 210},
                                              {HQ_FMT_Q5_K, 256, 176}, {HQ_FMT_Q4_0, 32, 18},   {HQ_FMT_Q5_0, 32, 22},
                                              {HQ_FMT_Q4_1, 32, 20},   {HQ_FMT_Q5_1, 32, 24},   {HQ_FMT_Q2_K, 256, 84},
                                              {HQ_FMT_Q3_K, 256, 110}};
    const int32_t* ty = kTypes[(int)type];
    const int64_t row_bytes = k / ty[1] * ty[2];
    if (data_.dtype() != DType::U8 || data_.rank() < 2 || data_.dim(-1) != row_bytes)
      throw Error("GgufMatMul: expected u8 rows of K/blk*bytes bytes");
    w_ = hq_weight{};
    w_.format = ty[0];
    w_.n_experts = data_.rank() == 3 ? (int32_t)data_.dim(0) : 1;
    w_.n = data_.dim(-2);
    w_.k = k;
    w_.data = data_.data();
    if (bias_.data()) { w_.bias = bias_.data(); w_.bias_dtype = (int32_t)bias_.dtype(); }
  }
  hq_weight weight() const override { return w_; }

 private:
  Tensor data_, bias_;
  hq_weight w_;
};

// e4m3 weight [N, K] / [E, N, K] with f32 `weight_scale_inv` [.., ceil(N/128), ceil(K/128)]
class BlockwiseFP8Linear : public QuantMethod {
 public:
  BlockwiseFP8Linear(Tensor weight, Tensor weight_scale_inv, Tensor bias = Tensor(), cudaStream_t stream = nullptr)
      : weight_(std::move(weight)), scale_(std::move(weight_scale_inv)), bias_(std::move(bias)) {
    if (weight_.dtype() != DType::U8 || scale_.dtype() != DType::F32) throw Error("BlockwiseFP8Linear: u8 codes and f32 scales");
    w_ = hq_weight{};
    w_.format = HQ_FMT_FP8_BLOCK;
    w_.n_experts = weight_.rank() == 3 ? (int32_t)weight_.dim(0) : 1;
    w_.n = weight_.dim(-2);
    w_.k = weight_.dim(-1);
    if (scale_.dim(-2) != (w_.n + 127) / 128 || scale_.dim(-1) != (w_.k + 127) / 128)
      throw Error("BlockwiseFP8Linear: scale grid does not match the weight");
    w_.data = weight_.data();
    w_.scales = scale_.data();
    if (bias_.data()) { w_.bias = bias_.data(); w_.bias_dtype = (int32_t)bias_.dtype(); }
    std::vector<int64_t> td(scale_.dims().begin(), scale_.dims().end() - 1);
    tile_scale_ = Tensor::empty(td, DType::F32);
    rel_scale_ = Tensor::empty(scale_.dims(), DType::F32);
    check(hq_fp8_scale_prepare((const float*)scale_.data(), w_.n_experts, w_.n, w_.k, (float*)tile_scale_.data(),
                               (float*)rel_scale_.data(), stream), "hq_fp8_scale_prepare");
    w_.fp8_tile_scale = tile_scale_.data();
    w_.fp8_rel_scale = rel_scale_.data();
  }
  hq_weight weight() const override { return w_; }

 private:
  Tensor weight_, scale_, bias_, tile_scale_, rel_scale_;
  hq_weight w_;
};

// MXFP4: blocks u8 [E, N, K/2] (low nibble = even element), scales u8 [E, N, K/32] (e8m0), optional bias [E, N]
class MXFP4Layer : public QuantMethod {
 public:
  MXFP4Layer(Tensor blocks, Tensor scales, Tensor bias = Tensor())
      : blocks_(std::move(blocks)), scales_(std::move(scales)), bias_(std::move(bias)) {
    w_ = hq_weight{};
    w_.format = HQ_FMT_MXFP4;
    w_.n_experts = blocks_.rank() == 3 ? (int32_t)blocks_.dim(0) : 1;
    w_.n = blocks_.dim(-2);
    w_.k = blocks_.dim(-1) * 2;
    if (w_.k % 32 || scales_.dim(-1) != w_.k / 32 || scales_.dim(-2) != w_.n) throw Error("MXFP4Layer: scales must be [.., N, K/32]");
    w_.data = blocks_.data();
    w_.scales = scales_.data();
    if (bias_.data()) { w_.bias = bias_.data(); w_.bias_dtype = (int32_t)bias_.dtype(); }
  }
  hq_weight weight() const override { return w_; }
  bool input_3d_is_per_slot() const override { return true; }

 private:
  Tensor blocks_, scales_, bias_;
  hq_weight w_;
};

// Expert block: gate/up projection + gated activation + down projection + weighted sum over the k slots
class MoEExperts {
 public:
  // separate gate / up banks (Qwen3, DeepSeek) ...
  MoEExperts(std::shared_ptr<QuantMethod> gate, std::shared_ptr<QuantMethod> up, std::shared_ptr<QuantMethod> down,
             hq_act_args act = {HQ_ACT_SWIGLU, 0, 0.f, 0.f})
      : gate_(std::move(gate)), up_(std::move(up)), down_(std::move(down)), act_(act) {}
  // ... or one bank whose rows interleave gate and up (gpt-oss)
  MoEExperts(std::shared_ptr<QuantMethod> gate_up, std::shared_ptr<QuantMethod> down, hq_act_args act)
      : gate_(std::move(gate_up)), down_(std::move(down)), act_(act) {}

  Tensor forward(const Tensor& xs, const Tensor& topk_weights, const Tensor& topk_ids, DType out_dtype,
                 const Tensor* shared_out = nullptr, cudaStream_t stream = nullptr) const {
    const int64_t t = topk_ids.dim(0), k = topk_ids.dim(1);
    const hq_weight w0 = gate_->weight(), wd = down_->weight();
    const DispatchTables tb = moe_dispatch_build(topk_ids, w0.n_experts, stream);
    Tensor x = xs.reshape({t, w0.k});
    if (t * k >= hq_config_get(HQ_CFG_MOE_TENSOR_MIN_ROWS) * w0.n_experts) x = to_dtype(x, DType::F16, stream);
    const int64_t inter = up_ ? w0.n : w0.n / 2;
    Tensor h = Tensor::empty({t * k, inter}, DType::F16);
    hq_weight w1{};
    if (up_) w1 = up_->weight();
    auto p = [](const Tensor& a) { return (const int32_t*)a.data(); };
    check(hq_moe_gather_forward(&w0, up_ ? &w1 : nullptr, &act_, x.data(), (int32_t)x.dtype(), HQ_ROWS_PER_TOKEN, t, (int32_t)k,
                                p(tb.expert_bounds), p(tb.sorted_assign), p(tb.sorted_token), tb.workspace.data(), h.data(),
                                HQ_DT_F16, HQ_ROWS_SORTED, nullptr, stream), "hq_moe_gather_forward(gate/up)");
    Tensor y = Tensor::empty({t * k, wd.n}, DType::F32);
    check(hq_moe_gather_forward(&wd, nullptr, nullptr, h.data(), HQ_DT_F16, HQ_ROWS_SORTED, t, (int32_t)k, p(tb.expert_bounds),
                                p(tb.sorted_assign), p(tb.sorted_token), tb.workspace.data(), y.data(), HQ_DT_F32,
                                HQ_ROWS_SORTED, nullptr, stream), "hq_moe_gather_forward(down)");
    Tensor out = Tensor::empty({t, wd.n}, out_dtype);
    check(hq_moe_weighted_reduce(y.data(), HQ_DT_F32, (const float*)topk_weights.data(), p(tb.inv_perm),
                                 shared_out ? shared_out->data() : nullptr, out.data(), (int32_t)out_dtype, t, (int32_t)k, wd.n,
                                 stream), "hq_moe_weighted_reduce");
    return out;
  }

 private:
  std::shared_ptr<QuantMethod> gate_, up_, down_;
  hq_act_args act_;
};

}  // namespace hq
