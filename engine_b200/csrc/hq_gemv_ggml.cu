// Decode mat-vec for the further GGML types of the reference's decode list (hanzo-quant/src/gguf/fast_mmvq.rs:36-50):
// Q5_K (176 bytes / 256 weights), Q4_0 (18 bytes / 32) and Q5_0 (22 bytes / 32).
//
// One warp per output row and work item (up to eight activation rows, all of one expert in expert-indexed mode).
// Per step the warp covers 256 consecutive weights, lane l the eight weights 8 l .. 8 l + 7: their codes are eight
// consecutive bytes of the block (low or high nibbles), expanded exactly to f32 in registers
// (Q5_K: d sc q - dmin m; Q4_0: d (q - 8); Q5_0: d (q - 16)) and multiplied with eight consecutive activations of
// every row (one 16-byte load per row for 16-bit activations).  Q4_0 / Q5_0 blocks start on 2-byte boundaries, so
// their bytes are fetched as 16-bit words.  Straightforward and not tuned against the HBM roofline; rows beyond
// eight are served eight at a time (the weights are then read once per eight rows).
// Algorithmic bytes per launch = N*K*bits/8 + M*K*sizeof(x) + M*N*sizeof(y) (bits: 5.5, 4.5, 5.5).
#include "hq_gemv_shared.cuh"

namespace hq {

constexpr int kGgmlWarps = 8;

template <int XDT>
__device__ __forceinline__ void ggml_load_x8(const char* row, int col, bool vec, float (&v)[8]) {
  if (XDT == HQ_DT_F32) {
    const float* p = reinterpret_cast<const float*>(row) + col;
    if (vec) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = __ldg(p + i);
    }
  } else {
    const uint16_t* p = reinterpret_cast<const uint16_t*>(row) + col;
    uint32_t w[4];
    if (vec) {
      const uint4 t = __ldg(reinterpret_cast<const uint4*>(p));
      w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w;
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) w[i] = (uint32_t)__ldg(p + 2 * i) | ((uint32_t)__ldg(p + 2 * i + 1) << 16);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (XDT == HQ_DT_BF16) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
      } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
      }
    }
  }
}

// eight consecutive bytes at a 2-byte aligned address
__device__ __forceinline__ uint2 ggml_load_8b(const uint8_t* p) {
  const uint16_t* h = reinterpret_cast<const uint16_t*>(p);
  uint2 r;
  r.x = (uint32_t)__ldg(h) | ((uint32_t)__ldg(h + 1) << 16);
  r.y = (uint32_t)__ldg(h + 2) | ((uint32_t)__ldg(h + 3) << 16);
  return r;
}

// the eight weights 8 lane .. 8 lane + 7 of the 256-weight span `it` of one row, as f32
template <int FMT>
__device__ __forceinline__ void ggml_dequant8(const uint8_t* row, int it, int lane, float (&w)[8]) {
  if (FMT == HQ_FMT_Q5_K) {
    const uint8_t* blk = row + 176 * it;                         // 16-byte aligned (rows are multiples of 176)
    const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(blk));   // {d | dmin, 12 scale bytes}
    const int c = lane >> 3, hi = (lane >> 2) & 1, l0 = 8 * (lane & 3);
    const int j = 2 * c + hi;
    uint32_t sc, mn;
    if (j < 4) {
      sc = (hdr.y >> (8 * j)) & 63u;
      mn = (hdr.z >> (8 * j)) & 63u;
    } else {
      const int jj = j - 4;
      sc = ((hdr.w >> (8 * jj)) & 0xFu) | (((hdr.y >> (8 * jj + 6)) & 3u) << 4);
      mn = ((hdr.w >> (8 * jj + 4)) & 0xFu) | (((hdr.z >> (8 * jj + 6)) & 3u) << 4);
    }
    const float d1 = half_bits_to_float(hdr.x) * (float)sc;      // exact
    const float m1 = half_bits_to_float(hdr.x >> 16) * (float)mn;
    const uint2 qs = __ldg(reinterpret_cast<const uint2*>(blk + 48 + 32 * c + l0));
    const uint2 qh = __ldg(reinterpret_cast<const uint2*>(blk + 16 + l0));
    const uint32_t qw[2] = {qs.x, qs.y}, hw[2] = {qh.x, qh.y};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t b = (qw[i >> 2] >> (8 * (i & 3))) & 0xFFu;
      const uint32_t h = (hw[i >> 2] >> (8 * (i & 3) + j)) & 1u;
      const uint32_t q = (hi ? (b >> 4) : (b & 15u)) | (h << 4);
      // product and difference rounded separately (the dequantize-then-multiply arithmetic), no contraction
      w[i] = __fsub_rn(__fmul_rn(d1, (float)q), m1);
    }
  } else {
    // blocks of 32: eight blocks per span; lane -> block lane / 4, elements 8 (lane & 3) .. + 7 of it
    constexpr int BB = FMT == HQ_FMT_Q4_0 ? 18 : 22;
    const uint8_t* blk = row + (int64_t)BB * (8 * it + (lane >> 2));
    const float d = __half2float(__ldg(reinterpret_cast<const __half*>(blk)));
    const int j0 = 8 * (lane & 3);                               // 0, 8, 16, 24
    const int hi = j0 >> 4, b0 = j0 & 15;
    const uint2 qs = ggml_load_8b(blk + (FMT == HQ_FMT_Q4_0 ? 2 : 6) + b0);
    const uint32_t qw[2] = {qs.x, qs.y};
    uint32_t qh = 0;
    if (FMT == HQ_FMT_Q5_0)
      qh = ((uint32_t)__ldg(reinterpret_cast<const uint16_t*>(blk + 2)) |
            ((uint32_t)__ldg(reinterpret_cast<const uint16_t*>(blk + 4)) << 16)) >> j0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t b = (qw[i >> 2] >> (8 * (i & 3))) & 0xFFu;
      int q = (int)(hi ? (b >> 4) : (b & 15u));
      if (FMT == HQ_FMT_Q5_0) q = (q | (int)(((qh >> i) & 1u) << 4)) - 16;
      else q -= 8;
      w[i] = d * (float)q;
    }
  }
}

template <int FMT, int BANKS, int XDT>
__global__ void __launch_bounds__(kGgmlWarps * 32) gemv_ggml_kernel(const GemvParams p, const int x_vec) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_rt = (p.n + kGgmlWarps - 1) / kGgmlWarps;
  const int n_y = p.tiles != nullptr ? p.tile_count[0] : (p.m + 7) / 8;
  const int total = n_y * n_rt;
  const int spans = p.k / 256;
  constexpr int BITS16 = FMT == HQ_FMT_Q5_K ? 11 : (FMT == HQ_FMT_Q4_0 ? 9 : 11);   // bytes per 16 weights
  const int64_t row_bytes = (int64_t)(p.k / 16) * BITS16;
  const int xsz = dtype_size(XDT);
  for (int w = blockIdx.x; w < total; w += gridDim.x) {
    const WorkItem wi = get_item<kGgmlWarps>(p, w, n_rt);
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
    for (int it = 0; it < spans; ++it) {
      float wv[BANKS][8];
#pragma unroll
      for (int b = 0; b < BANKS; ++b) ggml_dequant8<FMT>(wrow[b], it, lane, wv[b]);
      const int col = 256 * it + 8 * lane;
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (r < wi.nrows) {
          float xv[8];
          ggml_load_x8<XDT>(xrow[r], col, x_vec != 0, xv);
#pragma unroll
          for (int b = 0; b < BANKS; ++b)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[b][r] = fmaf(wv[b][i], xv[i], acc[b][r]);
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

template <int FMT, int BANKS>
static int32_t launch_ggml_x(const GemvParams& p, unsigned grid, int x_vec, cudaStream_t stream) {
  switch (p.x_dtype) {
    case HQ_DT_F32: gemv_ggml_kernel<FMT, BANKS, HQ_DT_F32><<<grid, kGgmlWarps * 32, 0, stream>>>(p, x_vec); break;
    case HQ_DT_F16: gemv_ggml_kernel<FMT, BANKS, HQ_DT_F16><<<grid, kGgmlWarps * 32, 0, stream>>>(p, x_vec); break;
    case HQ_DT_BF16: gemv_ggml_kernel<FMT, BANKS, HQ_DT_BF16><<<grid, kGgmlWarps * 32, 0, stream>>>(p, x_vec); break;
    default: return HQ_ERR_FORMAT;
  }
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

template <int FMT>
static int32_t launch_ggml_fmt(const GemvParams& p, unsigned grid, int x_vec, cudaStream_t stream) {
  return p.n_banks == 2 ? launch_ggml_x<FMT, 2>(p, grid, x_vec, stream) : launch_ggml_x<FMT, 1>(p, grid, x_vec, stream);
}

// Plain projection, or a gate and an up bank with a gated activation; an interleaved gate/up bank is not taken.
int32_t launch_gemv_ggml(const GemvParams& p, int n_y_max, cudaStream_t stream) {
  if (p.k % 256 != 0) return HQ_ERR_SHAPE;
  if (p.n_banks == 1 && p.act.act != HQ_ACT_NONE) return HQ_ERR_FORMAT;
  if (p.n_banks == 2 && p.act.act == HQ_ACT_NONE) return HQ_ERR_FORMAT;
  const int64_t items = (int64_t)n_y_max * ((p.n + kGgmlWarps - 1) / kGgmlWarps);
  if (items <= 0) return HQ_OK;
  const int64_t cap = (int64_t)sm_count() * 16;
  const unsigned grid = (unsigned)(items < cap ? items : cap);
  const int esz = dtype_size(p.x_dtype);
  const int x_vec = (reinterpret_cast<uintptr_t>(p.x) & 15u) == 0 && (p.x_stride * esz) % 16 == 0 ? 1 : 0;
  switch (p.format) {
    case HQ_FMT_Q5_K: return launch_ggml_fmt<HQ_FMT_Q5_K>(p, grid, x_vec, stream);
    case HQ_FMT_Q4_0: return launch_ggml_fmt<HQ_FMT_Q4_0>(p, grid, x_vec, stream);
    case HQ_FMT_Q5_0: return launch_ggml_fmt<HQ_FMT_Q5_0>(p, grid, x_vec, stream);
    default: return HQ_ERR_FORMAT;
  }
}

}  // namespace hq
