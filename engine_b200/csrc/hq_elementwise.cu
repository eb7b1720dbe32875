// Memory-bound helpers around the expert GEMMs: weighted un-permute/reduce,
// FP8 quantizers (1x128 activation groups, 128x128 weight blocks), gated
// activations.  All are single-pass: each input byte is read once, each output
// byte written once, accumulation in f32.
#include <cuda_fp8.h>

#include "hq_common.cuh"
#include "hq_kernels.h"

namespace hq {

// ---- out[t,:] = sum_s w[t,s] * y[row(t,s),:] (+ addend[t,:]) ----------------------
// One CTA per (token, 2048-column slab); slots are added in slot order, so the f32
// sum is reproducible.  Bytes: T*k*H*sizeof(y) read + T*H*sizeof(out) written.
template <typename TY, typename TO>
__global__ void __launch_bounds__(256) weighted_reduce_kernel(const TY* __restrict__ y, const float* __restrict__ w,
                                                              const int32_t* __restrict__ row_map,
                                                              const TO* __restrict__ addend, TO* __restrict__ out,
                                                              int top_k, int64_t hidden) {
  const int64_t t = blockIdx.x;
  __shared__ float sw[64];
  __shared__ int64_t srow[64];
  for (int s = threadIdx.x; s < top_k; s += blockDim.x) {
    sw[s] = w[t * top_k + s];
    srow[s] = row_map ? (int64_t)row_map[t * top_k + s] : t * top_k + s;
  }
  __syncthreads();
  constexpr int V = 16 / sizeof(TY);  // elements per 16-byte load
  const int64_t h0 = ((int64_t)blockIdx.y * blockDim.x + threadIdx.x) * V;
  if (h0 >= hidden) return;
  float acc[V];
#pragma unroll
  for (int i = 0; i < V; ++i) acc[i] = 0.f;
  if (h0 + V <= hidden && (hidden % V) == 0) {
    for (int s = 0; s < top_k; ++s) {
      if (srow[s] < 0) continue;      // slot without a row (skipped id): adds nothing
      const uint4 raw = *reinterpret_cast<const uint4*>(y + srow[s] * hidden + h0);
      const TY* v = reinterpret_cast<const TY*>(&raw);
      const float ws = sw[s];
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] = fmaf(ws, to_float<TY>(v[i]), acc[i]);
    }
#pragma unroll
    for (int i = 0; i < V; ++i) {
      float r = acc[i];
      if (addend) r += to_float<TO>(addend[t * hidden + h0 + i]);
      if constexpr (sizeof(TO) == 4) out[t * hidden + h0 + i] = r;
      else if constexpr (std::is_same<TO, __half>::value) out[t * hidden + h0 + i] = __float2half_rn(r);
      else out[t * hidden + h0 + i] = __float2bfloat16_rn(r);
    }
  } else {
    for (int i = 0; i < V && h0 + i < hidden; ++i) {
      float r = 0.f;
      for (int s = 0; s < top_k; ++s)
        if (srow[s] >= 0) r = fmaf(sw[s], to_float<TY>(y[srow[s] * hidden + h0 + i]), r);
      if (addend) r += to_float<TO>(addend[t * hidden + h0 + i]);
      if constexpr (sizeof(TO) == 4) out[t * hidden + h0 + i] = r;
      else if constexpr (std::is_same<TO, __half>::value) out[t * hidden + h0 + i] = __float2half_rn(r);
      else out[t * hidden + h0 + i] = __float2bfloat16_rn(r);
    }
  }
}

template <typename TY, typename TO>
static int32_t launch_wr(const void* y, const float* w, const int32_t* row_map, const void* addend, void* out,
                         int64_t n_tokens, int top_k, int64_t hidden, cudaStream_t stream) {
  constexpr int V = 16 / sizeof(TY);
  dim3 grid((unsigned)n_tokens, (unsigned)((hidden + 256 * V - 1) / (256 * V)));
  weighted_reduce_kernel<TY, TO><<<grid, 256, 0, stream>>>((const TY*)y, w, row_map, (const TO*)addend, (TO*)out,
                                                          top_k, hidden);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

int32_t launch_weighted_reduce(const void* y, int y_dtype, const float* w, const int32_t* row_map,
                               const void* addend, void* out, int out_dtype, int64_t n_tokens, int top_k,
                               int64_t hidden, cudaStream_t stream) {
  if (n_tokens == 0) return HQ_OK;
#define HQ_WR(TYC, TY, TOC, TO) \
  if (y_dtype == TYC && out_dtype == TOC) return launch_wr<TY, TO>(y, w, row_map, addend, out, n_tokens, top_k, hidden, stream);
  HQ_WR(HQ_DT_F32, float, HQ_DT_F32, float)
  HQ_WR(HQ_DT_F32, float, HQ_DT_BF16, __nv_bfloat16)
  HQ_WR(HQ_DT_F32, float, HQ_DT_F16, __half)
  HQ_WR(HQ_DT_BF16, __nv_bfloat16, HQ_DT_F32, float)
  HQ_WR(HQ_DT_BF16, __nv_bfloat16, HQ_DT_BF16, __nv_bfloat16)
  HQ_WR(HQ_DT_F16, __half, HQ_DT_F32, float)
  HQ_WR(HQ_DT_F16, __half, HQ_DT_F16, __half)
  HQ_WR(HQ_DT_F16, __half, HQ_DT_BF16, __nv_bfloat16)
  HQ_WR(HQ_DT_BF16, __nv_bfloat16, HQ_DT_F16, __half)
#undef HQ_WR
  return HQ_ERR_FORMAT;
}

// ---- FP8 e4m3 -------------------------------------------------------------------
__device__ __forceinline__ uint8_t f32_to_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ float e4m3_to_f32(uint8_t c) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)c, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

// one warp per group of 128 values; lane owns 4 consecutive values
__global__ void __launch_bounds__(256) fp8_vector_quant_kernel(const void* __restrict__ x, int dtype,
                                                               int64_t n_groups, uint8_t* __restrict__ codes,
                                                               float* __restrict__ scales) {
  const int64_t grp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (grp >= n_groups) return;
  const int lane = threadIdx.x & 31;
  const int64_t base = grp * 128 + lane * 4;
  float v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = load_as_float(x, dtype, base + i);
  float m = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
  const float scale = m > 0.f ? __fdiv_rn(m, 448.f) : 1e-12f;
  uint32_t packed = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float q = fminf(fmaxf(__fdiv_rn(v[i], scale), -448.f), 448.f);
    packed |= (uint32_t)f32_to_e4m3(q) << (8 * i);
  }
  *reinterpret_cast<uint32_t*>(codes + base) = packed;
  if (lane == 0) scales[grp] = scale;
}

__global__ void __launch_bounds__(256) fp8_vector_dequant_kernel(const uint8_t* __restrict__ codes,
                                                                 const float* __restrict__ scales, int64_t n,
                                                                 void* __restrict__ out, int dtype) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  store_from_float(out, dtype, i, e4m3_to_f32(codes[i]) * scales[i / 128]);
}

// one CTA per (by x bx) block
__global__ void __launch_bounds__(256) fp8_block_quant_kernel(const void* __restrict__ w, int dtype, int64_t rows,
                                                              int64_t cols, int by, int bx,
                                                              uint8_t* __restrict__ codes,
                                                              float* __restrict__ scales) {
  const int64_t r0 = (int64_t)blockIdx.y * by, c0 = (int64_t)blockIdx.x * bx;
  const int nr = (int)min((int64_t)by, rows - r0), nc = (int)min((int64_t)bx, cols - c0);
  __shared__ float red[8];
  float m = 0.f;
  for (int i = threadIdx.x; i < nr * nc; i += blockDim.x)
    m = fmaxf(m, fabsf(load_as_float(w, dtype, (r0 + i / nc) * cols + c0 + i % nc)));
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  m = red[0];
  for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
  const float scale = m > 0.f ? __fdiv_rn(m, 448.f) : 1e-12f;
  if (threadIdx.x == 0) scales[(int64_t)blockIdx.y * gridDim.x + blockIdx.x] = scale;
  for (int i = threadIdx.x; i < nr * nc; i += blockDim.x) {
    const int64_t idx = (r0 + i / nc) * cols + c0 + i % nc;
    const float q = fminf(fmaxf(__fdiv_rn(load_as_float(w, dtype, idx), scale), -448.f), 448.f);
    codes[idx] = f32_to_e4m3(q);
  }
}

__global__ void __launch_bounds__(256) fp8_block_dequant_kernel(const uint8_t* __restrict__ codes,
                                                                const float* __restrict__ scales, int64_t rows,
                                                                int64_t cols, int by, int bx, int64_t sc_cols,
                                                                void* __restrict__ out, int dtype) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * cols) return;
  const int64_t r = i / cols, c = i % cols;
  store_from_float(out, dtype, i, e4m3_to_f32(codes[i]) * scales[(r / by) * sc_cols + c / bx]);
}

int32_t launch_fp8_vector_quant(const void* x, int x_dtype, int64_t n, uint8_t* codes, float* scales,
                                cudaStream_t stream) {
  const int64_t groups = n / 128;
  if (groups == 0) return HQ_OK;
  fp8_vector_quant_kernel<<<(unsigned)((groups + 7) / 8), 256, 0, stream>>>(x, x_dtype, groups, codes, scales);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}
// four consecutive elements starting at element index i (a multiple of 4; rows are 16-byte aligned)
__device__ __forceinline__ void load4_as_float(const void* p, int dtype, int64_t i, float (&v)[4]) {
  if (dtype == HQ_DT_F32) {
    const float4 t = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
    const uint2 t = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(p) + i);
    if (dtype == HQ_DT_BF16) {
      v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xFFFF0000u);
      v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xFFFF0000u);
    } else {
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&t.x));
      const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&t.y));
      v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
  }
}

// The same 1 x 128 quantizer over rows that are looked up first (token order -> expert-sorted order).  Feeds the
// FP8 expert GEMM, whose operand boxes need whole sorted rows.  One warp per (output row, 512 columns): a lane owns
// 8 consecutive values in each half of the chunk (16-byte loads on 16-bit inputs, both issued before anything is
// used), a 128-column group is 16 lanes.
__global__ void __launch_bounds__(256) fp8_quant_rows_kernel(const void* __restrict__ x, int dtype, int64_t x_stride,
                                                             const int32_t* __restrict__ row_map,
                                                             const int32_t* __restrict__ n_valid, int64_t n_rows,
                                                             int kgroups, uint8_t* __restrict__ codes,
                                                             float* __restrict__ scales) {
  const int chunks = (kgroups + 3) / 4;
  const int64_t item = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int64_t limit = n_valid != nullptr ? min((int64_t)*n_valid, n_rows) : n_rows;   // rows the map is defined for
  if (item >= limit * chunks) return;
  const int lane = threadIdx.x & 31;
  const int64_t row = item / chunks;
  const int chunk = (int)(item - row * chunks);
  const int64_t src_row = row_map != nullptr ? (int64_t)row_map[row] : row;
  const int k = kgroups * 128;
  float v[2][8];
  bool in[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int c0 = chunk * 512 + j * 256 + lane * 8;
    in[j] = c0 < k;
    if (in[j]) {
      load4_as_float(x, dtype, src_row * x_stride + c0, *reinterpret_cast<float(*)[4]>(&v[j][0]));
      load4_as_float(x, dtype, src_row * x_stride + c0 + 4, *reinterpret_cast<float(*)[4]>(&v[j][4]));
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[j][i] = 0.f;
    }
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[j][i]));
#pragma unroll
    for (int d = 8; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
    if (!in[j]) continue;
    const float scale = m > 0.f ? __fdiv_rn(m, 448.f) : 1e-12f;
    uint32_t packed[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float q = fminf(fmaxf(__fdiv_rn(v[j][i], scale), -448.f), 448.f);
      packed[i >> 2] |= (uint32_t)f32_to_e4m3(q) << (8 * (i & 3));
    }
    const int c0 = chunk * 512 + j * 256 + lane * 8;
    *reinterpret_cast<uint2*>(codes + row * k + c0) = make_uint2(packed[0], packed[1]);
    if ((lane & 15) == 0) scales[row * kgroups + c0 / 128] = scale;
  }
}

int32_t launch_fp8_quant_rows(const void* x, int x_dtype, int64_t x_stride, const int32_t* row_map,
                              const int32_t* n_valid, int64_t n_rows, int64_t k, uint8_t* codes, float* scales,
                              cudaStream_t stream) {
  const int64_t items = n_rows * ((k / 128 + 3) / 4);
  if (items == 0) return HQ_OK;
  fp8_quant_rows_kernel<<<(unsigned)((items + 7) / 8), 256, 0, stream>>>(x, x_dtype, x_stride, row_map, n_valid,
                                                                        n_rows, (int)(k / 128), codes, scales);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

int32_t launch_fp8_vector_dequant(const uint8_t* codes, const float* scales, int64_t n, void* out, int out_dtype,
                                  cudaStream_t stream) {
  if (n == 0) return HQ_OK;
  fp8_vector_dequant_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(codes, scales, n, out, out_dtype);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}
int32_t launch_fp8_block_quant(const void* w, int w_dtype, int64_t rows, int64_t cols, int by, int bx,
                               uint8_t* codes, float* scales, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return HQ_OK;
  dim3 grid((unsigned)((cols + bx - 1) / bx), (unsigned)((rows + by - 1) / by));
  fp8_block_quant_kernel<<<grid, 256, 0, stream>>>(w, w_dtype, rows, cols, by, bx, codes, scales);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}
int32_t launch_fp8_block_dequant(const uint8_t* codes, const float* scales, int64_t rows, int64_t cols, int by,
                                 int bx, void* out, int out_dtype, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return HQ_OK;
  const int64_t n = rows * cols;
  fp8_block_dequant_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(codes, scales, rows, cols, by, bx,
                                                                           (cols + bx - 1) / bx, out, out_dtype);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

// ---- dtype conversion (hosts holding bf16 / f32 activations cast once before a prefill-sized call) -------
// Eight elements per thread (16-byte accesses on the 16-bit side).  A finite value beyond the f16 range is clamped
// to +-65504 instead of becoming inf, and the call says so through the status word: the tensor-core kernels
// multiply in f16, which the reference's bf16 / f32 activation paths do not, so the caller has to know.
__global__ void __launch_bounds__(256) convert_kernel(const void* __restrict__ src, int src_dtype,
                                                      void* __restrict__ dst, int dst_dtype, int64_t n, int vec_ok,
                                                      int32_t* __restrict__ status) {
  const int64_t i0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i0 >= n) return;
  float v[8];
  const bool full = vec_ok && i0 + 8 <= n;
  if (full) {
    load4_as_float(src, src_dtype, i0, *reinterpret_cast<float(*)[4]>(&v[0]));
    load4_as_float(src, src_dtype, i0 + 4, *reinterpret_cast<float(*)[4]>(&v[4]));
  } else {
    for (int j = 0; j < 8; ++j) v[j] = i0 + j < n ? load_as_float(src, src_dtype, i0 + j) : 0.f;
  }
  if (dst_dtype == HQ_DT_F16 && src_dtype != HQ_DT_F16) {
    bool clamped = false;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float a = fabsf(v[j]);
      if (a > 65504.f && a <= 3.4028235e38f) {       // finite and out of range (inf / NaN pass through)
        v[j] = copysignf(65504.f, v[j]);
        clamped = true;
      }
    }
    if (clamped) report_status(status, HQ_DEV_F16_RANGE, 900);
  }
  if (full && dst_dtype != HQ_DT_F32) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (dst_dtype == HQ_DT_F16) {
        w[j] = pack_half2(v[2 * j], v[2 * j + 1]);
      } else {
        __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
        w[j] = *reinterpret_cast<uint32_t*>(&b);
      }
    }
    *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(dst) + i0) = make_uint4(w[0], w[1], w[2], w[3]);
  } else if (full) {
    float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + i0);
    o[0] = make_float4(v[0], v[1], v[2], v[3]);
    o[1] = make_float4(v[4], v[5], v[6], v[7]);
  } else {
    for (int j = 0; j < 8 && i0 + j < n; ++j) store_from_float(dst, dst_dtype, i0 + j, v[j]);
  }
}

int32_t launch_convert(const void* src, int src_dtype, void* dst, int dst_dtype, int64_t n, int32_t* status,
                       cudaStream_t stream) {
  if (n == 0) return HQ_OK;
  const int64_t threads = (n + 7) / 8;
  const int vec_ok = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0;
  convert_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(src, src_dtype, dst, dst_dtype, n, vec_ok,
                                                                        status);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

// ---- gated activations --------------------------------------------------------------
__device__ __forceinline__ float gated_act(float g, float u, const hq_act_args& a) {
  if (a.act == HQ_ACT_GPTOSS) {
    g = fminf(g, a.limit);
    u = fminf(fmaxf(u, -a.limit), a.limit);
    return (u + 1.f) * (g / (1.f + expf(-a.alpha * g)));
  }
  if (a.has_limit) {
    g = fminf(g, a.limit);
    u = fminf(fmaxf(u, -a.limit), a.limit);
  }
  return (g / (1.f + expf(-g))) * u;
}

__global__ void __launch_bounds__(256) gated_act_kernel(const void* __restrict__ gate, const void* __restrict__ up,
                                                        int dtype, int64_t n, int interleaved, hq_act_args a,
                                                        void* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float g, u;
  if (interleaved) {
    g = load_as_float(gate, dtype, 2 * i);
    u = load_as_float(gate, dtype, 2 * i + 1);
  } else {
    g = load_as_float(gate, dtype, i);
    u = load_as_float(up, dtype, i);
  }
  store_from_float(out, dtype, i, gated_act(g, u, a));
}

int32_t launch_gated_act(const void* gate, const void* up, int dtype, int64_t n, int interleaved,
                         const hq_act_args& act, void* out, cudaStream_t stream) {
  if (n == 0) return HQ_OK;
  gated_act_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(gate, up, dtype, n, interleaved, act, out);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

// Gated activation of a [rows, 2 * width] matrix {gate | up} followed by the 1 x 128 FP8 quantizer: the expert
// intermediate goes to the FP8 down projection without a 16-bit round trip through memory.
__global__ void __launch_bounds__(256) fp8_gated_quant_rows_kernel(const void* __restrict__ gu, int dtype,
                                                                   int64_t n_rows, int width, hq_act_args act,
                                                                   uint8_t* __restrict__ codes,
                                                                   float* __restrict__ scales) {
  const int kgroups = width / 128;
  const int64_t grp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (grp >= n_rows * kgroups) return;
  const int lane = threadIdx.x & 31;
  const int64_t row = grp / kgroups;
  const int g = (int)(grp - row * kgroups);
  const int64_t src = row * 2 * width + g * 128 + lane * 4;
  float gv[4], uv[4], v[4];
  load4_as_float(gu, dtype, src, gv);
  load4_as_float(gu, dtype, src + width, uv);
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = gated_act(gv[i], uv[i], act);
  float m = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
  const float scale = m > 0.f ? __fdiv_rn(m, 448.f) : 1e-12f;
  uint32_t packed = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float q = fminf(fmaxf(__fdiv_rn(v[i], scale), -448.f), 448.f);
    packed |= (uint32_t)f32_to_e4m3(q) << (8 * i);
  }
  *reinterpret_cast<uint32_t*>(codes + grp * 128 + lane * 4) = packed;
  if (lane == 0) scales[grp] = scale;
}

int32_t launch_fp8_gated_quant_rows(const void* gu, int dtype, int64_t n_rows, int64_t width, const hq_act_args& act,
                                    uint8_t* codes, float* scales, cudaStream_t stream) {
  const int64_t groups = n_rows * (width / 128);
  if (groups == 0) return HQ_OK;
  fp8_gated_quant_rows_kernel<<<(unsigned)((groups + 7) / 8), 256, 0, stream>>>(gu, dtype, n_rows, (int)width, act,
                                                                               codes, scales);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

}  // namespace hq
