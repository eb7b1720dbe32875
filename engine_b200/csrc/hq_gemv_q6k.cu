// Decode mat-vec for GGUF Q6_K weights (block_q6_K {uint8 ql[128]; uint8 qh[64]; int8 scales[16]; half d},
// 210 bytes per 256 weights, value = d * scale * (q - 32); the type carries attn_v / ffn_down in Q4_K_M files and
// is in the reference's decode list, hanzo-quant/src/gguf/fast_mmvq.rs:36-50).
//
// One warp per output row and work item (up to eight activation rows, all of one expert in expert-indexed mode).
// Per 128-element half of a super-block lane l reads ql[l], ql[l + 32] and qh[l] -- three coalesced byte loads for
// the warp -- which hold the elements l, l + 32, l + 64, l + 96 of that half; the sixteen sub-block scales are
// loaded by lanes 0..15 and passed round by shuffle.  Weights are expanded to f32 in registers (exact: 6-bit code x
// int8 scale x f16 d) and multiplied with the activation rows read straight from global memory (they stay in L1
// across the eight warps of a CTA).  Blocks start on 2-byte boundaries, hence the byte loads.
// HBM-bound for one or two rows, issue-bound beyond; algorithmic bytes per launch = N*K*210/256 + M*K*sizeof(x) +
// M*N*sizeof(y).  Two banks (gate, up) share the activation loads and feed one gated activation.
#include "hq_gemv_shared.cuh"

namespace hq {

constexpr int kQ6Warps = 8;

template <int XDT>
__device__ __forceinline__ float q6_load_x(const void* row, int col) {
  if (XDT == HQ_DT_F32) return __ldg(reinterpret_cast<const float*>(row) + col);
  if (XDT == HQ_DT_F16) return __half2float(__ldg(reinterpret_cast<const __half*>(row) + col));
  return __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16*>(row) + col));
}

template <int BANKS, int XDT>
__global__ void __launch_bounds__(kQ6Warps * 32) gemv_q6k_kernel(const GemvParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_rt = (p.n + kQ6Warps - 1) / kQ6Warps;
  const int n_y = p.tiles != nullptr ? p.tile_count[0] : (p.m + 7) / 8;
  const int total = n_y * n_rt;
  const int nsb = p.k / 256;
  const int64_t row_bytes = (int64_t)nsb * 210;
  const int xsz = dtype_size(XDT);
  for (int w = blockIdx.x; w < total; w += gridDim.x) {
    const WorkItem wi = get_item<kQ6Warps>(p, w, n_rt);
    if (wi.nrows <= 0) continue;
    const int n = wi.n0 + warp;
    if (n >= p.n) continue;
    const char* xrow[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const int sr = wi.row0 + min(r, wi.nrows - 1);
      const int64_t xr = p.x_rows != nullptr ? (int64_t)p.x_rows[sr] : (int64_t)sr;
      xrow[r] = reinterpret_cast<const char*>(p.x) + xr * p.x_stride * xsz;
    }
    float acc[BANKS][8];
#pragma unroll
    for (int b = 0; b < BANKS; ++b)
#pragma unroll
      for (int r = 0; r < 8; ++r) acc[b][r] = 0.f;
    const uint8_t* wrow[BANKS];
    wrow[0] = reinterpret_cast<const uint8_t*>(p.w) + (int64_t)wi.expert * p.w_expert_stride + (int64_t)n * row_bytes;
    if (BANKS == 2)
      wrow[BANKS - 1] =
          reinterpret_cast<const uint8_t*>(p.w_up) + (int64_t)wi.expert * p.w_expert_stride + (int64_t)n * row_bytes;
    for (int sb = 0; sb < nsb; ++sb) {
      float d[BANKS];
      int sc[BANKS];
#pragma unroll
      for (int b = 0; b < BANKS; ++b) {
        const uint8_t* blk = wrow[b] + 210 * sb;
        d[b] = __half2float(__ldg(reinterpret_cast<const __half*>(blk + 208)));
        sc[b] = (int)(int8_t)__ldg(blk + 192 + (lane & 15));
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float wv[BANKS][4];
#pragma unroll
        for (int b = 0; b < BANKS; ++b) {
          const uint8_t* blk = wrow[b] + 210 * sb;
          const uint32_t ql0 = __ldg(blk + 64 * h + lane), ql1 = __ldg(blk + 64 * h + 32 + lane);
          const uint32_t qh = __ldg(blk + 128 + 32 * h + lane);
          const int q0 = (int)((ql0 & 15u) | ((qh & 3u) << 4)) - 32;
          const int q1 = (int)((ql1 & 15u) | (((qh >> 2) & 3u) << 4)) - 32;
          const int q2 = (int)((ql0 >> 4) | (((qh >> 4) & 3u) << 4)) - 32;
          const int q3 = (int)((ql1 >> 4) | (((qh >> 6) & 3u) << 4)) - 32;
          const int qs[4] = {q0, q1, q2, q3};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int s = __shfl_sync(0xffffffffu, sc[b], 8 * h + 2 * j + (lane >> 4));
            wv[b][j] = d[b] * (float)(s * qs[j]);
          }
        }
        const int col = 256 * sb + 128 * h + lane;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          if (r < wi.nrows) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float x = q6_load_x<XDT>(xrow[r], col + 32 * j);
#pragma unroll
              for (int b = 0; b < BANKS; ++b) acc[b][r] = fmaf(wv[b][j], x, acc[b][r]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int b = 0; b < BANKS; ++b)
#pragma unroll
      for (int r = 0; r < 8; ++r)
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) acc[b][r] += __shfl_xor_sync(0xffffffffu, acc[b][r], m);
    if (lane == 0) {
      float bias0 = 0.f, bias1 = 0.f;
      if (p.bias != nullptr) bias0 = load_as_float(p.bias, p.bias_dtype, (int64_t)wi.expert * p.n + n);
      if (BANKS == 2 && p.bias_up != nullptr) bias1 = load_as_float(p.bias_up, p.bias_dtype, (int64_t)wi.expert * p.n + n);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (r < wi.nrows) {
          float v = acc[0][r] + bias0;
          if (BANKS == 2) v = gated(v, acc[BANKS - 1][r] + bias1, p.act);
          const int64_t yr = p.y_rows != nullptr ? (int64_t)p.y_rows[wi.row0 + r] : (int64_t)(wi.row0 + r);
          store_from_float(p.y, p.y_dtype, yr * p.y_stride + n, v);
        }
      }
    }
  }
}

template <int BANKS>
static int32_t launch_q6k_banks(const GemvParams& p, unsigned grid, cudaStream_t stream) {
  switch (p.x_dtype) {
    case HQ_DT_F32: gemv_q6k_kernel<BANKS, HQ_DT_F32><<<grid, kQ6Warps * 32, 0, stream>>>(p); break;
    case HQ_DT_F16: gemv_q6k_kernel<BANKS, HQ_DT_F16><<<grid, kQ6Warps * 32, 0, stream>>>(p); break;
    case HQ_DT_BF16: gemv_q6k_kernel<BANKS, HQ_DT_BF16><<<grid, kQ6Warps * 32, 0, stream>>>(p); break;
    default: return HQ_ERR_FORMAT;
  }
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

// Plain projection, or a gate and an up bank with a gated activation; an interleaved gate/up bank is not taken.
int32_t launch_gemv_q6k(const GemvParams& p, int n_y_max, cudaStream_t stream) {
  if (p.k % 256 != 0) return HQ_ERR_SHAPE;
  if (p.n_banks == 1 && p.act.act != HQ_ACT_NONE) return HQ_ERR_FORMAT;
  if (p.n_banks == 2 && p.act.act == HQ_ACT_NONE) return HQ_ERR_FORMAT;
  const int64_t items = (int64_t)n_y_max * ((p.n + kQ6Warps - 1) / kQ6Warps);
  if (items <= 0) return HQ_OK;
  const int64_t cap = (int64_t)sm_count() * 16;
  const unsigned grid = (unsigned)(items < cap ? items : cap);
  return p.n_banks == 2 ? launch_q6k_banks<2>(p, grid, stream) : launch_q6k_banks<1>(p, grid, stream);
}

}  // namespace hq
