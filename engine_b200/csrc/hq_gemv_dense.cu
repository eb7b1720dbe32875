// Unquantized decode mat-vec: y[b, n] = sum_k x[b, k] * W[n, k] (+ bias[n]) for 1..8 activation rows, W in f16,
// bf16 or f32.  HBM-bound byte streaming (algorithmic bytes = N*K*sizeof(W) + b*K*sizeof(x) + b*N*sizeof(y)):
// every weight is read once with 16-byte loads, the activation rows are staged in shared memory one 2048-column
// chunk at a time (as f32) and shared by the 16 output rows of a block; a warp owns two output rows, keeps
// 2 x 8 partial sums in registers across the chunks and reduces them with shuffles at the end.  Many small blocks
// (seven per SM by shared memory) keep enough loads in flight; no tensor cores: with <= 8 rows there is nothing
// for them to do.
#include "hq_common.cuh"
#include "hq_kernels.h"

namespace hq {

namespace {

constexpr int kDgThreads = 256;
constexpr int kDgRowsPerWarp = 2;
constexpr int kDgRowsPerBlock = (kDgThreads / 32) * kDgRowsPerWarp;
constexpr int kDgChunk = 2048;      // activation columns staged at a time

template <typename TW>
__device__ __forceinline__ void dg_load8(const TW* p, float (&v)[8]);
template <>
__device__ __forceinline__ void dg_load8<float>(const float* p, float (&v)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void dg_load8<__half>(const __half* p, float (&v)[8]) {
  const uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
  const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void dg_load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

template <typename TW>
__global__ void __launch_bounds__(kDgThreads) dense_gemv_kernel(const TW* __restrict__ w, int64_t n, int64_t k,
                                                                const void* __restrict__ bias, int bias_dtype,
                                                                const void* __restrict__ x, int x_dtype,
                                                                int64_t x_stride, void* __restrict__ y, int y_dtype,
                                                                int64_t y_stride, int m) {
  extern __shared__ float xs[];      // [m][kDgChunk]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row0 = (int64_t)blockIdx.x * kDgRowsPerBlock + warp * kDgRowsPerWarp;
  float acc[kDgRowsPerWarp][8];
#pragma unroll
  for (int r = 0; r < kDgRowsPerWarp; ++r)
#pragma unroll
    for (int b = 0; b < 8; ++b) acc[r][b] = 0.f;
  for (int64_t k0 = 0; k0 < k; k0 += kDgChunk) {
    const int kc = (int)min((int64_t)kDgChunk, k - k0);
    __syncthreads();      // everyone is done with the previous chunk
    for (int i = threadIdx.x; i < m * kc; i += kDgThreads) {
      const int b = i / kc, c = i - b * kc;
      xs[b * kDgChunk + c] = load_as_float(x, x_dtype, (int64_t)b * x_stride + k0 + c);
    }
    __syncthreads();
    for (int c = lane * 8; c < kc; c += 256) {
      float wv[kDgRowsPerWarp][8];
#pragma unroll
      for (int r = 0; r < kDgRowsPerWarp; ++r) {
        if (row0 + r < n) dg_load8<TW>(w + (row0 + r) * k + k0 + c, wv[r]);
        else
#pragma unroll
          for (int j = 0; j < 8; ++j) wv[r][j] = 0.f;
      }
#pragma unroll
      for (int b = 0; b < 8; ++b) {
        if (b < m) {
          const float4 x0 = *reinterpret_cast<const float4*>(xs + b * kDgChunk + c);
          const float4 x1 = *reinterpret_cast<const float4*>(xs + b * kDgChunk + c + 4);
#pragma unroll
          for (int r = 0; r < kDgRowsPerWarp; ++r) {
            float s = acc[r][b];
            s = fmaf(wv[r][0], x0.x, s); s = fmaf(wv[r][1], x0.y, s); s = fmaf(wv[r][2], x0.z, s);
            s = fmaf(wv[r][3], x0.w, s); s = fmaf(wv[r][4], x1.x, s); s = fmaf(wv[r][5], x1.y, s);
            s = fmaf(wv[r][6], x1.z, s); s = fmaf(wv[r][7], x1.w, s);
            acc[r][b] = s;
          }
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kDgRowsPerWarp; ++r)
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      float s = acc[r][b];
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
      acc[r][b] = s;
    }
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < kDgRowsPerWarp; ++r) {
      if (row0 + r >= n) continue;
      const float bv = bias != nullptr ? load_as_float(bias, bias_dtype, row0 + r) : 0.f;
#pragma unroll
      for (int b = 0; b < 8; ++b)
        if (b < m) store_from_float(y, y_dtype, (int64_t)b * y_stride + row0 + r, acc[r][b] + bv);
    }
  }
}

}  // namespace

int32_t launch_dense_gemv(const void* w, int w_dtype, int64_t n, int64_t k, const void* bias, int bias_dtype,
                          const void* x, int x_dtype, int64_t x_stride, void* y, int y_dtype, int64_t y_stride, int m,
                          cudaStream_t stream) {
  const unsigned grid = (unsigned)((n + kDgRowsPerBlock - 1) / kDgRowsPerBlock);
  const size_t smem = (size_t)m * kDgChunk * sizeof(float);
  static bool attr_done[3][64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return HQ_ERR_CUDA;
#define HQ_DG(IDX, TW)                                                                                          \
  {                                                                                                             \
    if (dev < 64 && !attr_done[IDX][dev]) {                                                                     \
      if (cudaFuncSetAttribute(dense_gemv_kernel<TW>, cudaFuncAttributeMaxDynamicSharedMemorySize,              \
                               8 * kDgChunk * (int)sizeof(float)) != cudaSuccess)                               \
        return HQ_ERR_CUDA;                                                                                     \
      attr_done[IDX][dev] = true;                                                                               \
    }                                                                                                           \
    dense_gemv_kernel<TW><<<grid, kDgThreads, smem, stream>>>(static_cast<const TW*>(w), n, k, bias, bias_dtype, x, \
                                                              x_dtype, x_stride, y, y_dtype, y_stride, m);      \
  }
  if (w_dtype == HQ_DT_F32) HQ_DG(0, float)
  else if (w_dtype == HQ_DT_F16) HQ_DG(1, __half)
  else HQ_DG(2, __nv_bfloat16)
#undef HQ_DG
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

}  // namespace hq
