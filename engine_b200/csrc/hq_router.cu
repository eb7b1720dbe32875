// MoE router: per token row, score (raw / softmax / sigmoid) -> optional
// selection bias -> top-k by (selection DESC, expert id ASC) -> weights (score /
// softmax over the selected logits / sigmoid of the selected logits) ->
// optional renormalisation, output scale and per-expert scale.
//
// One warp per row; the row's logits, scores and selection keys live in shared
// memory, every reduction is a fixed-order warp shuffle tree, so the same
// logits always give the same ids.  HBM bytes per row: E*sizeof(logit) + k*8.
#include <math_constants.h>

#include "hq_common.cuh"
#include "hq_kernels.h"

namespace hq {

constexpr int kRouterWarps = 4;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  return v;
}

__global__ void __launch_bounds__(kRouterWarps * 32) router_kernel(const void* __restrict__ logits, int dtype,
                                                                   int64_t n_rows, hq_router_args a, int n_group,
                                                                   int topk_group, int group_mode,
                                                                   uint32_t* __restrict__ ids,
                                                                   float* __restrict__ weights) {
  extern __shared__ float rsm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kRouterWarps + warp;
  if (row >= n_rows) return;
  const int E = a.n_experts;
  float* raw = rsm + (size_t)warp * 3 * E;
  float* score = raw + E;
  float* sel = score + E;

  for (int e = lane; e < E; e += 32) {
    float v = load_as_float(logits, dtype, row * E + e);
    if (a.clamp_logits) v = fminf(fmaxf(v, a.clamp_min), a.clamp_max);
    if (v != v) v = -CUDART_INF_F;
    raw[e] = v;
  }
  __syncwarp();
  if (a.score_mode == HQ_SCORE_SOFTMAX) {
    float m = -CUDART_INF_F;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, raw[e]);
    m = warp_max(m);
    float s = 0.f;
    for (int e = lane; e < E; e += 32) {
      const float ex = expf(raw[e] - m);
      score[e] = ex;
      s += ex;
    }
    s = warp_sum(s);
    for (int e = lane; e < E; e += 32) score[e] = score[e] / s;
  } else if (a.score_mode == HQ_SCORE_SIGMOID) {
    for (int e = lane; e < E; e += 32) score[e] = 1.f / (1.f + expf(-raw[e]));
  } else {
    for (int e = lane; e < E; e += 32) score[e] = raw[e];
  }
  for (int e = lane; e < E; e += 32) {
    float v = score[e];
    if (a.selection_bias != nullptr) v += a.selection_bias[e];
    if (v != v) v = -CUDART_INF_F;
    sel[e] = v;
  }
  __syncwarp();

  // Group-limited selection (DeepSeek): experts form n_group contiguous groups; a group's score is the sum of its
  // two best selection scores (group_mode 0, "noaux_tc") or its best one (1, "group_limited_greedy"); only the
  // topk_group best groups stay selectable, the selection score of every other expert becomes 0
  // (hanzo-engine/src/models/deepseek3.rs:623-690).  Lane g scores group g; ties go to the lower group.
  if (n_group > 1) {
    const int gs = E / n_group;
    float gscore = -CUDART_INF_F;
    if (lane < n_group) {
      float t1 = -CUDART_INF_F, t2 = -CUDART_INF_F;
      for (int e = lane * gs; e < (lane + 1) * gs; ++e) {
        const float v = sel[e];
        if (v > t1) { t2 = t1; t1 = v; }
        else if (v > t2) t2 = v;
      }
      gscore = group_mode == 0 ? t1 + t2 : t1;
    }
    uint32_t keep = 0;
    bool consumed = lane >= n_group;
    for (int r = 0; r < topk_group; ++r) {
      float best = consumed ? -CUDART_INF_F : gscore;
      int best_g = consumed ? 0x7fffffff : lane;
#pragma unroll
      for (int m = 16; m > 0; m >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, m);
        const int og = __shfl_xor_sync(0xffffffffu, best_g, m);
        if (og != 0x7fffffff && (best_g == 0x7fffffff || ov > best || (ov == best && og < best_g))) {
          best = ov;
          best_g = og;
        }
      }
      if (best_g != 0x7fffffff) keep |= 1u << best_g;
      if (lane == best_g) consumed = true;
    }
    for (int e = lane; e < E; e += 32)
      if (((keep >> (e / gs)) & 1u) == 0u) sel[e] = 0.f;
    __syncwarp();
  }

  // k rounds of arg-max; ties go to the lower expert id.  Lane j keeps the j-th result.
  float my_w = 0.f;
  uint32_t my_id = 0;
  for (int r = 0; r < a.top_k; ++r) {
    float best = -CUDART_INF_F;
    int best_e = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = sel[e];
      // a consumed entry is marked NaN; everything else (including -inf) stays selectable
      if (v == v && (best_e == 0x7fffffff || v > best)) { best = v; best_e = e; }
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, m);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, m);
      if (oe != 0x7fffffff && (best_e == 0x7fffffff || ov > best || (ov == best && oe < best_e))) {
        best = ov;
        best_e = oe;
      }
    }
    float out = score[best_e];
    if (a.weight_mode == HQ_WEIGHT_SOFTMAX) out = raw[best_e];
    else if (a.weight_mode == HQ_WEIGHT_SIGMOID) out = 1.f / (1.f + expf(-raw[best_e]));
    if (lane == r) { my_w = out; my_id = (uint32_t)best_e; }
    if (lane == (best_e & 31)) sel[best_e] = CUDART_NAN_F;
    __syncwarp();
  }
  const bool mine = lane < a.top_k;
  if (a.weight_mode == HQ_WEIGHT_SOFTMAX) {
    const float m = warp_max(mine ? my_w : -CUDART_INF_F);
    const float ex = mine ? expf(my_w - m) : 0.f;
    const float s = warp_sum(ex);
    my_w = ex / s;
  }
  if (a.renormalize) {
    float s = warp_sum(mine ? my_w : 0.f);
    if (a.norm_min > 0.f) s = fmaxf(s, a.norm_min);
    my_w = my_w / s;
  }
  if (a.output_scale != 1.0f) my_w *= a.output_scale;
  if (mine) {
    if (a.expert_scale != nullptr) my_w *= a.expert_scale[my_id];
    weights[row * a.top_k + lane] = my_w;
    ids[row * a.top_k + lane] = my_id;
  }
}

int32_t launch_router(const void* logits, int dtype, int64_t n_rows, const hq_router_args& a, int n_group,
                      int topk_group, int group_mode, uint32_t* ids, float* weights, cudaStream_t stream) {
  if (n_rows == 0) return HQ_OK;
  const size_t smem = (size_t)kRouterWarps * 3 * a.n_experts * sizeof(float);
  const unsigned grid = (unsigned)((n_rows + kRouterWarps - 1) / kRouterWarps);
  router_kernel<<<grid, kRouterWarps * 32, smem, stream>>>(logits, dtype, n_rows, a, n_group, topk_group, group_mode,
                                                          ids, weights);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

}  // namespace hq
