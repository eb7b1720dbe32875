// Expert-parallel exchange helpers: what a rank does to its tokens before the dispatch all-to-all and to the
// received slabs after it.  The collectives themselves stay with the host (NCCL send/recv or all-to-all over
// equal-sized messages), so a host binding only adds those calls.
//
// Message to peer d = rows_per_peer rows of row_bytes bytes:
//   rows 0 .. capacity-1   payload of token t if one of its experts lives on d (otherwise the row is not written):
//                          16-bit wire: hidden values in the wire dtype; FP8 wire: hidden e4m3 codes followed by
//                          hidden / 128 f32 scales (the reference's 1 x 128 vector quantizer, so the expert rank
//                          feeds them to the FP8 MMA unchanged)
//   rows capacity ..       the meta block: for every row t < capacity its top_k slots as (int32 local expert id
//                          or -1, f32 router weight).  Written for every row, so the receiver needs no counts.
// One row per (token, destination rank): a token whose k experts sit on one rank travels there once, and that
// rank returns one row, the router-weighted sum over the token's experts it hosts.  Every slab has the same size,
// so no split sizes have to reach the host and nothing on this path synchronises with it.
#include <cuda_fp8.h>

#include "hq_common.cuh"
#include "hq_kernels.h"

namespace hq {

namespace {

__device__ __forceinline__ void ep_load4(const void* p, int dtype, int64_t i, float (&v)[4]) {
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

// One CTA per slab row t (0 .. capacity-1).  Rows at or beyond n_tokens only get their (all -1) meta.
__global__ void __launch_bounds__(256) ep_pack_kernel(const hq_ep_layout l, const void* __restrict__ x, int x_dtype,
                                                      const uint32_t* __restrict__ ids,
                                                      const float* __restrict__ weights, int n_tokens,
                                                      uint8_t* __restrict__ send, int32_t* __restrict__ back_map) {
  const int t = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  __shared__ uint32_t s_id[64];
  __shared__ float s_w[64];
  __shared__ int s_go[64];           // per destination rank: does this token travel there
  const int k = l.top_k, world = l.world;
  const bool live = t < n_tokens;
  for (int s = tid; s < k; s += 256) {
    s_id[s] = live ? ids[(int64_t)t * k + s] : 0xFFFFFFFFu;
    s_w[s] = live ? weights[(int64_t)t * k + s] : 0.f;
  }
  for (int d = tid; d < world; d += 256) s_go[d] = 0;
  __syncthreads();
  const uint32_t n_global = (uint32_t)world * (uint32_t)l.experts_per_rank;
  for (int s = tid; s < k; s += 256)
    if (s_id[s] < n_global) s_go[s_id[s] / (uint32_t)l.experts_per_rank] = 1;     // benign race: all write 1
  __syncthreads();
  // meta rows and the map the final reduce reads
  for (int i = tid; i < world * k; i += 256) {
    const int d = i / k, s = i - d * k;
    const uint32_t e = s_id[s];
    const bool mine = e < n_global && (int)(e / (uint32_t)l.experts_per_rank) == d;
    uint8_t* meta = send + (int64_t)d * l.message_bytes + (int64_t)l.capacity * l.row_bytes + ((int64_t)t * k + s) * 8;
    *reinterpret_cast<int2*>(meta) =
        make_int2(mine ? (int)(e - (uint32_t)d * (uint32_t)l.experts_per_rank) : -1, __float_as_int(mine ? s_w[s] : 0.f));
  }
  if (live)
    for (int d = tid; d < world; d += 256)
      back_map[(int64_t)t * world + d] = s_go[d] ? d * l.rows_per_peer + t : -1;
  if (!live) return;
  const int64_t hidden = l.hidden;
  if (l.fp8) {
    // one warp per group of 128 values, lane owns 4: the reference's vector quantizer
    // (hanzo-quant/src/vector_fp8/ops.rs:235-287), quantized once and stored to every destination
    for (int g = warp; g < hidden / 128; g += 8) {
      float v[4];
      ep_load4(x, x_dtype, (int64_t)t * hidden + g * 128 + lane * 4, v);
      float m = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
      const float scale = m > 0.f ? __fdiv_rn(m, 448.f) : 1e-12f;
      uint32_t packed = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float qv = fminf(fmaxf(__fdiv_rn(v[i], scale), -448.f), 448.f);
        packed |= (uint32_t)__nv_cvt_float_to_fp8(qv, __NV_SATFINITE, __NV_E4M3) << (8 * i);
      }
      for (int d = 0; d < world; ++d) {
        if (!s_go[d]) continue;
        uint8_t* row = send + (int64_t)d * l.message_bytes + (int64_t)t * l.row_bytes;
        *reinterpret_cast<uint32_t*>(row + g * 128 + lane * 4) = packed;
        if (lane == 0) *reinterpret_cast<float*>(row + hidden + g * 4) = scale;
      }
    }
  } else {
    for (int64_t i = (int64_t)tid * 4; i < hidden; i += 1024) {
      float v[4];
      ep_load4(x, x_dtype, (int64_t)t * hidden + i, v);
      uint2 o;
      if (l.wire_dtype == HQ_DT_F16) {
        o.x = pack_half2(v[0], v[1]);
        o.y = pack_half2(v[2], v[3]);
      } else {
        __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        o.x = *reinterpret_cast<uint32_t*>(&a);
        o.y = *reinterpret_cast<uint32_t*>(&b);
      }
      for (int d = 0; d < world; ++d) {
        if (!s_go[d]) continue;
        uint8_t* row = send + (int64_t)d * l.message_bytes + (int64_t)t * l.row_bytes;
        *reinterpret_cast<uint2*>(row + i * 2) = o;
      }
    }
  }
}

// Meta blocks of the world received slabs -> ids [world * rows_per_peer, k], weights likewise; the pad rows that
// carry the meta bytes themselves get id -1.
__global__ void __launch_bounds__(256) ep_unpack_meta_kernel(const hq_ep_layout l, const uint8_t* __restrict__ recv,
                                                             uint32_t* __restrict__ ids,
                                                             float* __restrict__ weights) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  const int64_t per_peer = (int64_t)l.rows_per_peer * l.top_k;
  if (i >= per_peer * l.world) return;
  const int src = (int)(i / per_peer);
  const int64_t r = i - src * per_peer;          // row * k + slot inside the slab
  int id = -1;
  float w = 0.f;
  if (r < (int64_t)l.capacity * l.top_k) {
    const int2 m = *reinterpret_cast<const int2*>(recv + src * l.message_bytes + (int64_t)l.capacity * l.row_bytes + r * 8);
    id = m.x;
    w = __int_as_float(m.y);
  }
  ids[i] = (uint32_t)id;
  weights[i] = w;
}

// dst row r = src row row_map[r] for r < *n_valid: e4m3 codes (k bytes) and their k / 128 scales, each side with
// its own row stride.  One warp per row.
__global__ void __launch_bounds__(256) fp8_gather_rows_kernel(const uint8_t* __restrict__ src_codes,
                                                              int64_t src_code_stride,
                                                              const uint8_t* __restrict__ src_scales,
                                                              int64_t src_scale_stride,
                                                              const int32_t* __restrict__ row_map,
                                                              const int32_t* __restrict__ n_valid, int64_t n_rows,
                                                              int k, uint8_t* __restrict__ codes,
                                                              float* __restrict__ scales) {
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int64_t limit = n_valid != nullptr ? min((int64_t)*n_valid, n_rows) : n_rows;
  if (row >= limit) return;
  const int64_t src = row_map != nullptr ? (int64_t)row_map[row] : row;
  const uint4* sc = reinterpret_cast<const uint4*>(src_codes + src * src_code_stride);
  uint4* dc = reinterpret_cast<uint4*>(codes + row * k);
  for (int i = lane; i < k / 16; i += 32) dc[i] = sc[i];
  const float* ss = reinterpret_cast<const float*>(src_scales + src * src_scale_stride);
  for (int i = lane; i < k / 128; i += 32) scales[row * (k / 128) + i] = ss[i];
}


// ---- the exchange itself over peer memory --------------------------------------------------------------
// Slab d of the local send buffer goes to slot `rank` of peer d's receive buffer with plain stores over NVLink
// (16 bytes per store, a grid-stride loop per slab; peer pointers come from a symmetric allocation the host set
// up).  No TMA, no multicast.  Each thread ends with a system-scope fence; the barrier kernel below tells the
// peers that the data is there.
__global__ void __launch_bounds__(256) ep_push_kernel(const uint4* __restrict__ send, uint4* const* __restrict__ peers,
                                                      int world, int rank, int64_t slab_vec, int ctas_per_slab) {
  const int d = blockIdx.x / ctas_per_slab;
  const int c = blockIdx.x - d * ctas_per_slab;
  if (d >= world) return;
  const uint4* src = send + (int64_t)d * slab_vec;
  uint4* dst = peers[d] + (int64_t)rank * slab_vec;
  const int64_t stride = (int64_t)ctas_per_slab * 256;
  int64_t i = (int64_t)c * 256 + threadIdx.x;
  for (; i + 3 * stride < slab_vec; i += 4 * stride) {
    const uint4 a = __ldg(src + i), b = __ldg(src + i + stride), e = __ldg(src + i + 2 * stride),
                f = __ldg(src + i + 3 * stride);
    dst[i] = a;
    dst[i + stride] = b;
    dst[i + 2 * stride] = e;
    dst[i + 3 * stride] = f;
  }
  for (; i < slab_vec; i += stride) dst[i] = __ldg(src + i);
  __threadfence_system();
}

// The same push row by row, leaving out the rows nobody will read: a token travels to 5 of 8 ranks on average, so
// a third of the rows of a slab carry nothing.  CTAs stride over the slab rows.  A row is sent when
//   - it lies at or behind `always_from` (the meta rows of the dispatch slabs), or
//   - dispatch: back_map[t * world + d] >= 0 (token t goes to rank d), or
//   - return: any of the row's top_k slot ids is a real expert (ids != 0xFFFFFFFF).
__global__ void __launch_bounds__(256) ep_push_rows_kernel(const uint4* __restrict__ send,
                                                           uint4* const* __restrict__ peers, int world, int rank,
                                                           int rows_per_slab, int row_vec, int always_from,
                                                           const int32_t* __restrict__ back_map, int n_tokens,
                                                           const uint32_t* __restrict__ ids, int top_k) {
  const int64_t total = (int64_t)world * rows_per_slab;
  for (int64_t gr = blockIdx.x; gr < total; gr += gridDim.x) {      // row over all slabs
    const int d = (int)(gr / rows_per_slab);
    const int r = (int)(gr - (int64_t)d * rows_per_slab);
    if (r < always_from) {
      bool live;
      if (back_map != nullptr) {
        live = r < n_tokens && back_map[(int64_t)r * world + d] >= 0;
      } else {
        live = false;
        for (int s = 0; s < top_k; ++s) live = live || ids[gr * top_k + s] != 0xFFFFFFFFu;
      }
      if (!live) continue;                              // block-uniform
    }
    const uint4* src = send + gr * row_vec;
    uint4* dst = peers[d] + ((int64_t)rank * rows_per_slab + r) * row_vec;
    for (int i = threadIdx.x; i < row_vec; i += 256) dst[i] = __ldg(src + i);
  }
  __threadfence_system();
}

// Barrier over the ranks of the exchange: thread p tells peer p "rank `rank` has finished its step `seq`" by
// storing seq into slot `rank` of peer p's flag array, then waits until slot p of the local flag array has
// reached seq.  Flags only grow, one per barrier, so a peer that is already one barrier ahead satisfies the
// wait as well; it cannot get further ahead without this rank's next signal.  The wait is bounded: after
// `spin_limit` polls the kernel reports HQ_DEV_WAIT_TIMEOUT (tag 950 + p) and returns.
__global__ void __launch_bounds__(64) ep_barrier_kernel(int32_t* const* __restrict__ flags, int world, int rank,
                                                        int32_t* __restrict__ seq_counter, uint32_t spin_limit,
                                                        int32_t* __restrict__ status) {
  const int p = threadIdx.x;
  const int32_t seq = *seq_counter + 1;
  if (p < world) {
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flags[p] + rank), "r"(seq) : "memory");
    const int32_t* mine = flags[rank] + p;
    bool ok = false;
    for (uint32_t it = 0; it < spin_limit; ++it) {
      int32_t v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if (v - seq >= 0) {
        ok = true;
        break;
      }
      __nanosleep(100);
    }
    if (!ok) report_status(status, HQ_DEV_WAIT_TIMEOUT, 950 + p);
  }
  __syncthreads();
  if (p == 0) *seq_counter = seq;
}

}  // namespace

int32_t launch_ep_pack(const hq_ep_layout& l, const void* x, int x_dtype, const uint32_t* ids, const float* weights,
                       int64_t n_tokens, void* send, int32_t* back_map, cudaStream_t stream) {
  ep_pack_kernel<<<(unsigned)l.capacity, 256, 0, stream>>>(l, x, x_dtype, ids, weights, (int)n_tokens,
                                                          (uint8_t*)send, back_map);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

int32_t launch_ep_unpack_meta(const hq_ep_layout& l, const void* recv, uint32_t* ids, float* weights,
                              cudaStream_t stream) {
  const int64_t n = (int64_t)l.world * l.rows_per_peer * l.top_k;
  ep_unpack_meta_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(l, (const uint8_t*)recv, ids, weights);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

int32_t launch_fp8_gather_rows(const void* src_codes, int64_t src_code_stride, const void* src_scales,
                               int64_t src_scale_stride, const int32_t* row_map, const int32_t* n_valid,
                               int64_t n_rows, int64_t k, uint8_t* codes, float* scales, cudaStream_t stream) {
  if (n_rows == 0) return HQ_OK;
  fp8_gather_rows_kernel<<<(unsigned)((n_rows + 7) / 8), 256, 0, stream>>>(
      (const uint8_t*)src_codes, src_code_stride, (const uint8_t*)src_scales, src_scale_stride, row_map, n_valid,
      n_rows, (int)k, codes, scales);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

int32_t launch_ep_push(const void* send, void* const* peers, int world, int rank, int64_t slab_bytes,
                       cudaStream_t stream) {
  if (world <= 0 || slab_bytes <= 0) return HQ_OK;
  const int64_t slab_vec = slab_bytes / 16;
  int per = (int)((slab_vec + 256 * 16 - 1) / (256 * 16));       // about 16 stores per thread
  const int cap = 8 * 148 / world > 0 ? 8 * 148 / world : 1;
  if (per > cap) per = cap;
  if (per < 1) per = 1;
  ep_push_kernel<<<(unsigned)(world * per), 256, 0, stream>>>(reinterpret_cast<const uint4*>(send),
                                                             reinterpret_cast<uint4* const*>(peers), world, rank,
                                                             slab_vec, per);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

int32_t launch_ep_push_rows(const void* send, void* const* peers, int world, int rank, int rows_per_slab,
                            int64_t row_bytes, int always_from, const int32_t* back_map, int n_tokens,
                            const uint32_t* ids, int top_k, cudaStream_t stream) {
  const int64_t rows = (int64_t)world * rows_per_slab;
  if (rows <= 0 || row_bytes <= 0) return HQ_OK;
  const int64_t cap = 8 * 148;
  ep_push_rows_kernel<<<(unsigned)(rows < cap ? rows : cap), 256, 0, stream>>>(reinterpret_cast<const uint4*>(send),
                                                          reinterpret_cast<uint4* const*>(peers), world, rank,
                                                          rows_per_slab, (int)(row_bytes / 16), always_from, back_map,
                                                          n_tokens, ids, top_k);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

int32_t launch_ep_barrier(int32_t* const* flags, int world, int rank, int32_t* seq_counter, uint32_t spin_limit,
                          int32_t* status, cudaStream_t stream) {
  ep_barrier_kernel<<<1, 64, 0, stream>>>(flags, world, rank, seq_counter, spin_limit, status);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

}  // namespace hq
