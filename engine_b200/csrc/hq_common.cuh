// Shared device helpers for the sm_100a kernels: mbarrier, bulk (TMA) copies,
// warp MMA, bounded waits, status word.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hanzoquant_b200.h"

namespace hq {

// Device status word layout (int32[4]): [0] = first error code (0 = none),
// [1] = blockIdx.x, [2] = blockIdx.y, [3] = phase tag of the wait that gave up.
// The codes themselves (HQ_DEV_*) are part of the public header.

__device__ __forceinline__ void report_status(int32_t* status, int code, int tag) {
  if (status != nullptr && atomicCAS(status, 0, code) == 0) {
    status[1] = (int32_t)blockIdx.x;
    status[2] = (int32_t)blockIdx.y;
    status[3] = tag;
  }
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// ---- mbarrier -------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after `spin_limit` polls (each poll may itself block for a
// hardware-defined short time).  Returns false on give-up; the caller reports and leaves.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t spin_limit) {
  for (uint32_t i = 0; i < spin_limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}

// Same bounded wait for warps that only hand work over (MMA issuer, epilogue, reducers): they back off
// between polls so their polling does not take issue slots from the warps doing the arithmetic.
__device__ __forceinline__ bool mbar_wait_backoff(uint64_t* bar, uint32_t parity, uint32_t spin_limit) {
  for (uint32_t i = 0; i < spin_limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    __nanosleep(i < 8 ? 32 : 128);
  }
  return false;
}

// ---- bulk async copy global -> shared (TMA, untiled) ----------------------
// Both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void bulk_g2s_hint(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar,
                                              uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
          smem_u32(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

// ---- named barrier among a subset of warps --------------------------------
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---- shared loads (the byte offset is an immediate, so no address arithmetic is issued per load) ------------
template <int OFF = 0>
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
  return v;
}
template <int OFF = 0>
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(OFF));
  return v;
}
template <int OFF = 0>
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1+%2];" : "=h"(v) : "r"(addr), "n"(OFF));
  return v;
}

// ---- warp MMA m16n8k16, f16 x f16 -> f32 -----------------------------------
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
  // not volatile: a pure function of its register operands, so the compiler may interleave independent MMAs
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// same MMA with explicit C operands (D = A.B + C), D write-only
__device__ __forceinline__ void mma_f16_16816_c(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                uint32_t b0, uint32_t b1, float c0, float c1, float c2, float c3) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c0), "f"(c1), "f"(c2), "f"(c3));
}

__device__ __forceinline__ float half_bits_to_float(uint32_t h) {
  return __half2float(__ushort_as_half((unsigned short)(h & 0xFFFFu)));
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// value conversion for the three activation/output dtypes that cross the ABI
template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ float load_as_float(const void* p, int dtype, int64_t i) {
  if (dtype == HQ_DT_F32) return ((const float*)p)[i];
  if (dtype == HQ_DT_F16) return __half2float(((const __half*)p)[i]);
  return __bfloat162float(((const __nv_bfloat16*)p)[i]);
}
__device__ __forceinline__ void store_from_float(void* p, int dtype, int64_t i, float v) {
  if (dtype == HQ_DT_F32) ((float*)p)[i] = v;
  else if (dtype == HQ_DT_F16) ((__half*)p)[i] = __float2half_rn(v);
  else ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
}

__host__ __device__ __forceinline__ int dtype_size(int dtype) { return dtype == HQ_DT_F32 ? 4 : 2; }

}  // namespace hq
