// Pieces shared by the decode mat-vec kernels: the work-item walk and the output stage
// (bias, gated activation, scatter of up to eight activation rows per item).
#pragma once
#include "hq_common.cuh"
#include "hq_kernels.h"

namespace hq {

__device__ __forceinline__ float gated(float g, float u, const hq_act_args& a) {
  if (a.act == HQ_ACT_GPTOSS) {
    g = fminf(g, a.limit);
    u = fminf(fmaxf(u, -a.limit), a.limit);
    const float glu = g / (1.f + expf(-a.alpha * g));
    return (u + 1.f) * glu;
  }
  if (a.has_limit) {
    g = fminf(g, a.limit);
    u = fminf(fmaxf(u, -a.limit), a.limit);
  }
  return (g / (1.f + expf(-g))) * u;
}

// One work item: up to eight activation rows (all of one expert in expert-indexed mode) against a tile
// of RT output rows starting at n0.
struct WorkItem {
  int expert, row0, nrows, n0, y;
};

template <int RT>
__device__ __forceinline__ WorkItem get_item(const GemvParams& p, int w, int n_rt) {
  WorkItem it;
  it.y = w / n_rt;
  it.n0 = (w - it.y * n_rt) * RT;
  if (p.tiles != nullptr) {
    it.expert = p.tiles[2 * it.y];
    it.row0 = p.tiles[2 * it.y + 1];
    it.nrows = min(8, p.expert_bounds[it.expert + 1] - it.row0);
  } else {
    it.expert = 0;
    it.row0 = 8 * it.y;
    it.nrows = min(8, p.m - it.row0);
  }
  return it;
}

// Output stage of one 16-row item, executed by a whole warp.  Lane 4*g + t holds, per weight bank b,
// v[b][0], v[b][1] = output row n0 + g, activation rows col0, col0 + 1 and v[b][2], v[b][3] = output row
// n0 + g + 8.  Lanes with col_owner false hold nothing to write but take part in the shuffles.
__device__ __forceinline__ void gemv_store_item(const GemvParams& p, const WorkItem& wi, int g, int col0,
                                                bool col_owner, float (&v)[2][4]) {
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int n = wi.n0 + g + 8 * half;
    const bool n_ok = n < p.n;
    float v0 = v[0][2 * half], v1 = v[0][2 * half + 1];
    float u0 = v[1][2 * half], u1 = v[1][2 * half + 1];
    if (n_ok && p.bias != nullptr) {
      const float bv = load_as_float(p.bias, p.bias_dtype, (int64_t)wi.expert * p.n + n);
      v0 += bv; v1 += bv;
    }
    if (n_ok && p.n_banks == 2 && p.bias_up != nullptr) {
      const float bv = load_as_float(p.bias_up, p.bias_dtype, (int64_t)wi.expert * p.n + n);
      u0 += bv; u1 += bv;
    }
    int64_t out_n = n;
    bool write = n_ok && col_owner;
    if (p.act.act != HQ_ACT_NONE) {
      if (p.n_banks == 2) {
        v0 = gated(v0, u0, p.act);
        v1 = gated(v1, u1, p.act);
      } else {
        // interleaved bank: even row = gate, odd row = up (the neighbour lane group g+1)
        const float p0 = __shfl_down_sync(0xffffffffu, v0, 4);
        const float p1 = __shfl_down_sync(0xffffffffu, v1, 4);
        v0 = gated(v0, p0, p.act);
        v1 = gated(v1, p1, p.act);
        write = write && (n & 1) == 0;
        out_n = n >> 1;
      }
    }
    if (write) {
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int col = col0 + cc;
        if (col < wi.nrows) {
          const int64_t yr = p.y_rows ? (int64_t)p.y_rows[wi.row0 + col] : (int64_t)(wi.row0 + col);
          store_from_float(p.y, p.y_dtype, yr * p.y_stride + out_n, cc ? v1 : v0);
        }
      }
    }
  }
}

// ---- cp.async pieces of the kernels that stage weight rows through shared memory --------------------------------
// The GGML block types start on 2-byte boundaries, too narrow for wide loads from global memory.  A warp instead
// copies the aligned 16-byte pieces that cover a stretch of a row with cp.async (several stretches in flight), into
// a buffer in which every byte keeps its address modulo 16, and picks the fields out of shared memory.  The first
// and the last piece may hold up to 15 bytes that are not part of the stretch; they lie in the same aligned
// 16-byte granule as a byte that is, so they are readable, and they are never looked at.
__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

inline int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// the Q6_K / Q5_K / Q4_0 / Q5_0 decode kernel on warp MMAs (hq_gemv_ggml_mma.cu)
int32_t launch_gemv_ggml_mma(const GemvParams& p, int n_y_max, cudaStream_t stream);

// the Q8_0 / Q4_K decode kernel (hq_gemv_int8.cu)
int32_t launch_gemv_int8(const GemvParams& p, int n_y_max, int max_rows, cudaStream_t stream);

}  // namespace hq
