// Measurement aid: the dense issue rate of tcgen05.mma from every SM with the operands resident in shared
// memory.  A benchmark times the launch with CUDA events and divides; the figure is the denominator for the
// FP8 expert GEMM's tensor-core fraction (the 16-bit peak has a library GEMM to measure it with, FP8 on this
// instruction does not).  One CTA per SM, one issuing lane, accumulators alternate between two tensor-memory
// buffers so consecutive instructions do not depend on each other.  The final wait is bounded.
#include "hq_common.cuh"
#include "hq_kernels.h"

namespace hq {

namespace {

__device__ __forceinline__ uint64_t probe_desc(uint32_t a) {
  uint64_t d = 0;
  d |= (uint64_t)((a >> 4) & 0x3FFFu);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

constexpr int kProbeSmem = 64 * 1024 + 1024;   // A tile 128 x 128 B, B tile 256 x 128 B (zero-filled), + alignment

template <int KIND>   // 0 = kind::f16 (f16 operands, K = 16 per instruction), 1 = kind::f8f6f4 (e4m3, K = 32)
__global__ void __launch_bounds__(128, 1) probe_mma_kernel(int n_dim, int iters, int32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  for (int i = threadIdx.x; i < 48 * 1024 / 4; i += 128) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_barrier_init();
  }
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  fence_proxy_async_smem();
  const uint32_t tb = slot;
  if (threadIdx.x == 0) {
    const uint32_t idesc = (1u << 4) | ((uint32_t)(n_dim >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    const uint64_t ad = probe_desc(smem_u32(smem)), bd = probe_desc(smem_u32(smem) + 16384);
    for (int it = 0; it < iters; ++it) {
      const uint32_t d = tb + (uint32_t)((it & 1) * 256);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        if (KIND == 0)
          asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d),
                       "l"(ad + 2 * kk), "l"(bd + 2 * kk), "r"(idesc), "r"(kk > 0 ? 1u : 0u)
                       : "memory");
        else
          asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}\n" ::"r"(d),
                       "l"(ad + 2 * kk), "l"(bd + 2 * kk), "r"(idesc), "r"(kk > 0 ? 1u : 0u)
                       : "memory");
      }
    }
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bar)) : "memory");
    if (!mbar_wait(&bar, 0, 1u << 24)) report_status(status, HQ_DEV_WAIT_TIMEOUT, 990);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tb), "r"(512) : "memory");
  }
}

}  // namespace

int32_t launch_probe_mma(int kind, int n_dim, int iters, int32_t* status, double* flops_out, cudaStream_t stream) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return HQ_ERR_CUDA;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return HQ_ERR_CUDA;
  cudaError_t e = kind == 0
                      ? cudaFuncSetAttribute(probe_mma_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, kProbeSmem)
                      : cudaFuncSetAttribute(probe_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kProbeSmem);
  if (e != cudaSuccess) return HQ_ERR_CUDA;
  if (kind == 0) probe_mma_kernel<0><<<sms, 128, kProbeSmem, stream>>>(n_dim, iters, status);
  else probe_mma_kernel<1><<<sms, 128, kProbeSmem, stream>>>(n_dim, iters, status);
  if (flops_out != nullptr)
    *flops_out = 2.0 * 128.0 * n_dim * (kind == 0 ? 16.0 : 32.0) * 4.0 * iters * sms;
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

}  // namespace hq
