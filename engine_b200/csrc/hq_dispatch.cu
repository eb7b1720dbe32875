// Token -> expert dispatch tables: a stable counting sort of the flat
// assignment index t*top_k+s by expert id, built without output atomics so the
// permutation is identical on every run (the reference's CUDA scatter orders
// rows by atomic arrival; its host grouping is the stable order reproduced
// here).
//
//   pass 1  per-chunk expert histograms (1024 assignments per block)
//   pass 2  one block: per-expert exclusive prefix over chunks, expert bounds,
//           tile lists (work items of <= 8, <= 128 and <= 256 sorted rows per expert)
//   pass 3  stable scatter: warps take their 32 assignments in turn; inside a
//           warp the rank among equal experts comes from a match mask + popcount
//
// HBM bytes: T*k*4 read twice + T*k*4*3 written; negligible next to the GEMMs.
#include <atomic>

#include "hq_common.cuh"
#include "hq_kernels.h"

namespace hq {

DispatchLayout dispatch_layout(int64_t n_tokens, int top_k, int n_experts) {
  DispatchLayout l;
  const int64_t total = n_tokens * top_k;
  l.n_blocks = (total + kDispatchChunk - 1) / kDispatchChunk;
  if (l.n_blocks < 1) l.n_blocks = 1;
  l.off_counts = 4;
  l.max_tiles8 = (total + 7) / 8 + n_experts;
  l.max_tiles128 = (total + 127) / 128 + n_experts;
  l.off_tiles8 = l.off_counts + l.n_blocks * n_experts;
  l.max_tiles256 = (total + 255) / 256 + n_experts;
  l.off_tiles128 = l.off_tiles8 + 2 * l.max_tiles8;
  l.off_tiles256 = l.off_tiles128 + 2 * l.max_tiles128;
  l.total_words = l.off_tiles256 + 2 * l.max_tiles256;
  return l;
}

__global__ void __launch_bounds__(1024) dispatch_count_kernel(const uint32_t* __restrict__ ids, int total,
                                                              int n_experts, int32_t* __restrict__ counts) {
  extern __shared__ int32_t hist[];
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int i = blockIdx.x * kDispatchChunk + threadIdx.x;
  if (i < total) {
    const uint32_t e = ids[i];
    if (e < (uint32_t)n_experts) atomicAdd(&hist[e], 1);  // integer counts: order does not matter
  }
  __syncthreads();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[(int64_t)blockIdx.x * n_experts + e] = hist[e];
}

// counts[b][e] -> exclusive offset of chunk b inside expert e (in place); bounds; tile lists
__global__ void __launch_bounds__(1024) dispatch_scan_kernel(int32_t* __restrict__ counts, int n_blocks,
                                                             int n_experts, int32_t* __restrict__ bounds,
                                                             int32_t* __restrict__ header,
                                                             int32_t* __restrict__ tiles8,
                                                             int32_t* __restrict__ tiles128,
                                                             int32_t* __restrict__ tiles256) {
  extern __shared__ int32_t sm[];
  int32_t* tot = sm;                    // [E] expert totals, then exclusive bounds
  int32_t* t8 = sm + n_experts;         // [E] tile8 offsets
  int32_t* t128 = sm + 2 * n_experts;   // [E] tile128 offsets
  int32_t* t256 = sm + 3 * n_experts;   // [E] tile256 offsets
  __shared__ int32_t s_total;
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
    int32_t run = 0;
    // eight chunk counts are loaded before the first running sum is written back, so the loads overlap
    for (int b0 = 0; b0 < n_blocks; b0 += 8) {
      int32_t c[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) c[j] = b0 + j < n_blocks ? counts[(int64_t)(b0 + j) * n_experts + e] : 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (b0 + j < n_blocks) counts[(int64_t)(b0 + j) * n_experts + e] = run;
        run += c[j];
      }
    }
    tot[e] = run;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    // warp scan over experts, 32 at a time, carrying the running totals
    int32_t carry = 0, c8 = 0, c128 = 0, c256 = 0;
    for (int base = 0; base < n_experts; base += 32) {
      const int e = base + threadIdx.x;
      const int32_t cnt = e < n_experts ? tot[e] : 0;
      int32_t v = cnt, v8 = (cnt + 7) / 8, v128 = (cnt + 127) / 128, v256 = (cnt + 255) / 256;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int32_t o = __shfl_up_sync(0xffffffffu, v, d);
        const int32_t o8 = __shfl_up_sync(0xffffffffu, v8, d);
        const int32_t o128 = __shfl_up_sync(0xffffffffu, v128, d);
        const int32_t o256 = __shfl_up_sync(0xffffffffu, v256, d);
        if ((int)threadIdx.x >= d) { v += o; v8 += o8; v128 += o128; v256 += o256; }
      }
      if (e < n_experts) {
        bounds[e] = carry + v - cnt;
        tot[e] = carry + v - cnt;
        t8[e] = c8 + v8 - (cnt + 7) / 8;
        t128[e] = c128 + v128 - (cnt + 127) / 128;
        t256[e] = c256 + v256 - (cnt + 255) / 256;
      }
      carry += __shfl_sync(0xffffffffu, v, 31);
      c8 += __shfl_sync(0xffffffffu, v8, 31);
      c128 += __shfl_sync(0xffffffffu, v128, 31);
      c256 += __shfl_sync(0xffffffffu, v256, 31);
    }
    if (threadIdx.x == 0) {
      bounds[n_experts] = carry;
      s_total = carry;
      header[0] = c8;
      header[1] = c128;
      header[2] = carry;
      header[3] = c256;
    }
  }
  __syncthreads();
  // add the expert base to every chunk offset
  for (int64_t i = threadIdx.x; i < (int64_t)n_blocks * n_experts; i += blockDim.x) counts[i] += tot[i % n_experts];
  // tile lists: one warp per expert, lanes over the expert's tiles
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  for (int e = warp; e < n_experts; e += n_warps) {
    const int32_t start = tot[e];
    const int32_t cnt = (e + 1 < n_experts ? tot[e + 1] : s_total) - start;
    for (int i = lane; i < (cnt + 7) / 8; i += 32) {
      tiles8[2 * (t8[e] + i)] = e;
      tiles8[2 * (t8[e] + i) + 1] = start + 8 * i;
    }
    for (int i = lane; i < (cnt + 127) / 128; i += 32) {
      tiles128[2 * (t128[e] + i)] = e;
      tiles128[2 * (t128[e] + i) + 1] = start + 128 * i;
    }
    for (int i = lane; i < (cnt + 255) / 256; i += 32) {
      tiles256[2 * (t256[e] + i)] = e;
      tiles256[2 * (t256[e] + i) + 1] = start + 256 * i;
    }
  }
}

__global__ void __launch_bounds__(1024) dispatch_scatter_kernel(const uint32_t* __restrict__ ids, int total,
                                                                int top_k, int n_experts,
                                                                const int32_t* __restrict__ offsets,
                                                                int32_t* __restrict__ sorted_assign,
                                                                int32_t* __restrict__ sorted_token,
                                                                int32_t* __restrict__ inv_perm) {
  extern __shared__ int32_t cur[];  // running position per expert for this chunk
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) cur[e] = offsets[(int64_t)blockIdx.x * n_experts + e];
  __syncthreads();
  const int i = blockIdx.x * kDispatchChunk + threadIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool ok = i < total;
  const uint32_t e = ok ? ids[i] : 0xFFFFFFFFu;
  const bool routed = ok && e < (uint32_t)n_experts;
  // ids outside [0, n_experts) are skipped (padding slots such as -1): they get no sorted row and their
  // inverse-map entry says so, which the weighted reduce reads as "contributes nothing"
  if (ok && !routed) inv_perm[i] = -1;
  // rank inside the warp among lanes with the same expert
  const uint32_t peers = __match_any_sync(0xffffffffu, e);
  const int rank = __popc(peers & ((1u << lane) - 1u));
  const int group = __popc(peers);
  const bool leader = rank == 0;
  // warps commit in index order so earlier assignments get earlier positions
  for (int w = 0; w < kDispatchChunk / 32; ++w) {
    if (w == warp && routed) {
      const int pos = cur[e] + rank;
      sorted_assign[pos] = i;
      sorted_token[pos] = i / top_k;
      inv_perm[i] = pos;
    }
    __syncthreads();
    if (w == warp && routed && leader) cur[e] += group;
    __syncthreads();
  }
}

int32_t launch_dispatch(const uint32_t* ids, int64_t n_tokens, int top_k, int n_experts, int32_t* bounds,
                        int32_t* sorted_assign, int32_t* sorted_token, int32_t* inv_perm, int32_t* ws,
                        cudaStream_t stream) {
  const DispatchLayout l = dispatch_layout(n_tokens, top_k, n_experts);
  const int total = (int)(n_tokens * top_k);
  int32_t* counts = ws + l.off_counts;
  const size_t sm1 = (size_t)n_experts * 4;
  // no tokens: only the scan runs and writes all-zero bounds (a grid of zero blocks is not a valid launch)
  if (l.n_blocks > 0) dispatch_count_kernel<<<(unsigned)l.n_blocks, 1024, sm1, stream>>>(ids, total, n_experts, counts);
  dispatch_scan_kernel<<<1, 1024, 4 * sm1, stream>>>(counts, (int)l.n_blocks, n_experts, bounds, ws,
                                                    ws + l.off_tiles8, ws + l.off_tiles128, ws + l.off_tiles256);
  if (l.n_blocks > 0)
    dispatch_scatter_kernel<<<(unsigned)l.n_blocks, 1024, sm1, stream>>>(ids, total, top_k, n_experts, counts,
                                                                        sorted_assign, sorted_token, inv_perm);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

// ---- variant for callers that cannot allocate ------------------------------------------------------
// Some hosts have no way to hand this library a workspace: every byte of device memory is already owned by
// their own pool (a serving engine that sizes its KV cache to whatever is free), or the call is made from
// a place where asking the CUDA runtime for memory is not allowed.  For them the chunk histograms and the
// tile lists live in a fixed array inside the library image.  It is sized for kNoAllocMaxAssignments
// assignments and kNoAllocMaxExperts experts (about 220 KB), exists once per GPU that loads the library
// and is shared by every call: two calls that overlap on the GPU (different streams, or graphs replayed
// concurrently) race on it.  Nothing in it has to start at zero -- every word that is read is written
// first by the same call.
constexpr int kNoAllocMaxAssignments = 65536;
constexpr int kNoAllocMaxExperts = 512;
constexpr int64_t kNoAllocWords = 4 + (int64_t)(kNoAllocMaxAssignments / kDispatchChunk) * kNoAllocMaxExperts +
                                  2 * ((int64_t)kNoAllocMaxAssignments / 8 + kNoAllocMaxExperts) +
                                  2 * ((int64_t)kNoAllocMaxAssignments / 128 + kNoAllocMaxExperts) +
                                  2 * ((int64_t)kNoAllocMaxAssignments / 256 + kNoAllocMaxExperts);
static __device__ __align__(256) int32_t g_noalloc_scratch[kNoAllocWords];

int32_t launch_dispatch_noalloc(const uint32_t* ids, int64_t n_tokens, int top_k, int n_experts, int32_t* bounds,
                                int32_t* sorted_assign, int32_t* sorted_token, int32_t* inv_perm,
                                cudaStream_t stream) {
  if (n_tokens * top_k > kNoAllocMaxAssignments || n_experts > kNoAllocMaxExperts) return HQ_ERR_TOO_LARGE;
  const DispatchLayout l = dispatch_layout(n_tokens, top_k, n_experts);
  if (l.total_words > kNoAllocWords) return HQ_ERR_TOO_LARGE;
  // The array's name is only a host-side handle; kernels need its device address, which differs per device.
  // Looked up on the first call made with a given device current (a plain runtime query, no allocation).
  // The cache is written by whichever host thread gets there first; every writer stores the same value.
  static std::atomic<int32_t*> dev_ptr[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return HQ_ERR_CUDA;
  int32_t* scratch = dev_ptr[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) return HQ_ERR_CUDA;
    scratch = static_cast<int32_t*>(p);
    dev_ptr[dev].store(scratch, std::memory_order_release);
  }
  return launch_dispatch(ids, n_tokens, top_k, n_experts, bounds, sorted_assign, sorted_token, inv_perm, scratch,
                         stream);
}

}  // namespace hq
