// Block-FP8 expert GEMM with FP8 activations on tcgen05 (kind::f8f6f4), nothing converted on the way in.
//
// y[row, n] = sum over 128-column blocks kb of  ws[expert, n/128, kb] * xs[row, kb] *
//             sum_{k in kb} e4m3(W[expert, n, k]) * e4m3(X[row, k])
// W: the reference's e4m3 codes [E, N, K] + f32 128x128 block scales; X: activation rows already quantized
// 1 x 128 (codes + one f32 scale per row and block) and already in expert-sorted order, so a tile of 128
// token rows of one expert is a plain 2-D box.  Both operands go from HBM to shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle, one 128 x 128-byte box each per stage) and from there into the
// tensor core unchanged; the products of e4m3 values are exact and accumulate in f32 in tensor memory.
// Because the scales change every 128 columns the accumulation is cut there: each 128-column block is
// multiplied into a fresh tensor-memory buffer (four buffers in rotation), and the eight epilogue warps fold
// it into register accumulators with one FMA per element (factor = weight-block scale x the token's
// scale for that block, from a per-item factor table the epilogue warps build out of the scales TMA
// brought in) while the next block is already being multiplied.  With 128 tokens per expert every weight byte is used once, so the kernel is
// bound by streaming the weights: five 32 KiB stages are kept in flight.
//
// Roles (one persistent CTA per SM, 11 warps): warp 0 issues TMA, warps 1 and 10 issue the MMAs of alternate
// 128-column blocks (one elected lane each), warps 2-9 are the epilogue: warp w reads tensor-memory lanes 32 * (w % 4) .. + 31 (its 32 output
// features) and the 64 token columns (w - 2) / 4 * 64 .. + 63.  Swapped roles as in the 16-bit kernel: lanes =
// output features, columns = tokens.  Every wait is bounded; a wait that runs out is reported in the status
// word and the kernel still reaches its normal exit.  No multicast, no peer memory.
#include <cuda.h>

#include "hq_common.cuh"
#include "hq_kernels.h"

namespace hq {

constexpr int kF8Threads = 352;                          // TMA warp, MMA warp, 8 epilogue warps, second MMA warp
constexpr int kF8Stages = 5;
constexpr int kF8TileBytes = 128 * 128;                  // one operand box: 128 rows x 128 bytes
constexpr int kF8StageBytes = 2 * kF8TileBytes;
constexpr int kF8MaxKB = 64;                             // 128-column blocks per row (K <= 8192)
constexpr int kF8AccBufs = 4;                            // 128-column accumulator buffers in tensor memory
constexpr uint32_t kF8Spin = 1u << 22;

struct F8Smem {
  static constexpr int OFF_RAW = kF8Stages * kF8StageBytes;          // activation scales as TMA brings them: [128 tokens][KB]
  static constexpr int OFF_FAC = OFF_RAW + 128 * kF8MaxKB * 4;       // factors the epilogue reads: [KB][128 tokens]
  static constexpr int OFF_BAR = OFF_FAC + 128 * kF8MaxKB * 4;
  static constexpr int TOTAL = OFF_BAR + (2 * kF8Stages + 12) * 8 + 16 + 1024;    // + alignment slack
};
static_assert(F8Smem::TOTAL <= 227 * 1024, "shared memory budget");

__device__ __forceinline__ void f8_tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void f8_tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void f8_tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void f8_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void f8_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void f8_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void f8_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void f8_tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void f8_tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand tile of 128-byte rows, 128-byte swizzle, 8-row groups 1024 bytes apart, descriptor version 1
__device__ __forceinline__ uint64_t f8_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFFu);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// kind::f8f6f4 instruction descriptor: f32 accumulate, A and B e4m3 (format code 0), both K-major, M = N = 128
__device__ __forceinline__ uint32_t f8_idesc() {
  return (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

// one 2-D box by TMA; x = innermost (byte / element) coordinate, y = row
__device__ __forceinline__ void f8_tma_2d(void* dst_smem, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
          "r"(smem_u32(dst_smem)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

struct F8Item {
  int expert, row_start, count, n0;
};
__device__ __forceinline__ F8Item f8_item(const Fp8GroupedParams& p, int w, int n_nt) {
  F8Item t;
  const int tt = w / n_nt;
  t.n0 = (w - tt * n_nt) * 128;
  if (p.tiles != nullptr) {
    t.expert = p.tiles[2 * tt];
    t.row_start = p.tiles[2 * tt + 1];
    t.count = min(128, p.expert_bounds[t.expert + 1] - t.row_start);
  } else {
    t.expert = 0;
    t.row_start = 128 * tt;
    t.count = min(128, p.m - t.row_start);
  }
  return t;
}

__global__ void __launch_bounds__(kF8Threads, 1)
fp8_grouped_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                   const __grid_constant__ CUtensorMap tm_s, const Fp8GroupedParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  float* sc_raw = reinterpret_cast<float*>(smem + F8Smem::OFF_RAW);
  float* sc_fac = reinterpret_cast<float*>(smem + F8Smem::OFF_FAC);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + F8Smem::OFF_BAR);
  uint64_t* empty = full + kF8Stages;
  uint64_t* acc_full = empty + kF8Stages;            // [4] a 128-column block has been multiplied into buffer b
  uint64_t* acc_empty = acc_full + kF8AccBufs;       // [4] ... and has been read out by all epilogue warps
  uint64_t* sc_full = acc_empty + kF8AccBufs;        // the tile's activation scales have landed (slot [1] unused)
  uint64_t* sc_empty = sc_full + 2;         // ... and have been turned into the factor table
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sc_empty + 2);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_nt = p.n / 128;
  const int n_tt = p.tiles != nullptr ? p.tile_count[0] : (p.m + 127) / 128;
  const int total = n_tt * n_nt;
  const int KB = p.k / 128;

  if (tid == 0) {
    for (int s = 0; s < kF8Stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < kF8AccBufs; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sc_full[b], 1);
      mbar_init(&sc_empty[b], 8);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    f8_tmem_alloc(smem_u32(tmem_slot), 128 * kF8AccBufs);
    f8_tmem_relinquish();
  }
  f8_fence_before();
  __syncthreads();
  f8_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // =========================== TMA issuer =========================================================
    if (lane == 0) {
      uint32_t spin = kF8Spin;
      int s = 0, round = 0, item = 0;
      for (int w = blockIdx.x; w < total; w += gridDim.x, ++item) {
        const F8Item t = f8_item(p, w, n_nt);
        if (item >= 1) {
          if (!mbar_wait_backoff(&sc_empty[0], (item - 1) & 1, spin)) {
            report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 700);
            spin = 1;
          }
        }
        mbar_arrive_expect_tx(&sc_full[0], (uint32_t)(128 * KB * 4));
        f8_tma_2d(sc_raw, &tm_s, 0, t.row_start, &sc_full[0]);
        const int wrow = t.expert * p.n + t.n0;
        for (int kb = 0; kb < KB; ++kb) {
          if (round > 0) {
            if (!mbar_wait_backoff(&empty[s], (round - 1) & 1, spin)) {
              report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 710 + s);
              spin = 1;
            }
          }
          uint8_t* stage = smem + s * kF8StageBytes;
          mbar_arrive_expect_tx(&full[s], (uint32_t)kF8StageBytes);
          f8_tma_2d(stage, &tm_w, kb * 128, wrow, &full[s]);
          f8_tma_2d(stage + kF8TileBytes, &tm_x, kb * 128, t.row_start, &full[s]);
          if (++s == kF8Stages) {
            s = 0;
            ++round;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1 || warp == 10) {
    // =========================== MMA issuers ========================================================
    // tcgen05.commit holds its thread until the MMAs before it have gone through the pipe, and the waits that
    // follow would leave the tensor core idle: two issuing lanes take alternate 128-column blocks, so one is
    // always ready to issue while the other waits
    if (lane == 0) {
      const int me = warp == 1 ? 0 : 1;
      const uint32_t idesc = f8_idesc();
      uint32_t spin = kF8Spin;
      int blk = 0;      // 128-column blocks so far (buffer = blk % kF8AccBufs, stage = blk % kF8Stages)
      for (int w = blockIdx.x; w < total; w += gridDim.x) {
        for (int kb = 0; kb < KB; ++kb, ++blk) {
          if ((blk & 1) != me) continue;
          const int buf = blk % kF8AccBufs;
          const int s = blk % kF8Stages;
          if (blk >= kF8AccBufs) {
            if (!mbar_wait(&acc_empty[buf], ((blk / kF8AccBufs) - 1) & 1, spin)) {
              report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 720 + buf);
              spin = 1;
            }
          }
          if (!mbar_wait(&full[s], (blk / kF8Stages) & 1, spin)) {
            report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 730 + s);
            spin = 1;
          }
          f8_fence_after();
          const uint32_t stage = smem_u32(smem + s * kF8StageBytes);
          const uint64_t adesc = f8_smem_desc(stage), bdesc = f8_smem_desc(stage + kF8TileBytes);
          const uint32_t d = tmem_base + (uint32_t)(buf * 128);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)   // 32 k = 32 bytes per instruction: advance the start address by 2 units
            f8_mma(d, adesc + 2 * kk, bdesc + 2 * kk, idesc, kk > 0 ? 1u : 0u);
          f8_commit(&empty[s]);        // the stage is free once these MMAs have read it
          f8_commit(&acc_full[buf]);   // the block's products are complete
        }
      }
    }
    __syncwarp();
  } else {
    // =========================== epilogue ===========================================================
    const int q = warp & 3;                 // tensor-memory lane quarter this warp may read
    const int half = (warp - 2) >> 2;       // which 64 of the tile's 128 token columns
    uint32_t spin = kF8Spin;
    int item = 0, blk = 0;
    for (int w = blockIdx.x; w < total; w += gridDim.x, ++item) {
      const F8Item t = f8_item(p, w, n_nt);
      const float* wsc = p.w_scales + ((int64_t)t.expert * p.fp8_nb + t.n0 / 128) * p.fp8_kb;
      if (!mbar_wait_backoff(&sc_full[0], item & 1, spin)) {
        if (lane == 0) report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 740);
        spin = 1;
      }
      // factor table of this item: fac[kb][token] = weight-block scale x token scale, so the inner loop reads four
      // tokens per shared load at fixed offsets and spends one FMA per element
      named_bar_sync(2, 256);                 // every epilogue warp is done with the previous item's factors
      for (int idx = tid - 64; idx < 128 * KB; idx += 256) {
        const int kb = idx >> 7, tok = idx & 127;
        sc_fac[idx] = sc_raw[tok * KB + kb] * __ldg(wsc + kb);
      }
      named_bar_sync(2, 256);
      if (lane == 0) mbar_arrive(&sc_empty[0]);   // the raw scales may be overwritten by the next item's
      const uint32_t fac_w = smem_u32(sc_fac) + (uint32_t)(half * 64) * 4u;
      float acc[64];
#pragma unroll
      for (int j = 0; j < 64; ++j) acc[j] = 0.f;
      for (int kb = 0; kb < KB; ++kb, ++blk) {
        const int buf = blk % kF8AccBufs;
        if (!mbar_wait(&acc_full[buf], (blk / kF8AccBufs) & 1, spin)) {
          if (lane == 0) report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 750 + buf);
          spin = 1;
        }
        f8_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(buf * 128 + half * 64);
        uint32_t c0[32], c1[32];
        f8_tmem_ld32(taddr, c0);
        f8_tmem_ld32(taddr + 32, c1);
        f8_tmem_ld_wait();
        f8_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);     // the buffer may be overwritten: values are in registers
        const uint32_t fk = fac_w + (uint32_t)kb * 512u;
#pragma unroll
        for (int j4 = 0; j4 < 8; ++j4) {
          float4 f0, f1;
          asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=f"(f0.x), "=f"(f0.y), "=f"(f0.z), "=f"(f0.w) : "r"(fk + 16u * j4));
          asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=f"(f1.x), "=f"(f1.y), "=f"(f1.z), "=f"(f1.w) : "r"(fk + 128u + 16u * j4));
          acc[4 * j4 + 0] = fmaf(__uint_as_float(c0[4 * j4 + 0]), f0.x, acc[4 * j4 + 0]);
          acc[4 * j4 + 1] = fmaf(__uint_as_float(c0[4 * j4 + 1]), f0.y, acc[4 * j4 + 1]);
          acc[4 * j4 + 2] = fmaf(__uint_as_float(c0[4 * j4 + 2]), f0.z, acc[4 * j4 + 2]);
          acc[4 * j4 + 3] = fmaf(__uint_as_float(c0[4 * j4 + 3]), f0.w, acc[4 * j4 + 3]);
          acc[32 + 4 * j4 + 0] = fmaf(__uint_as_float(c1[4 * j4 + 0]), f1.x, acc[32 + 4 * j4 + 0]);
          acc[32 + 4 * j4 + 1] = fmaf(__uint_as_float(c1[4 * j4 + 1]), f1.y, acc[32 + 4 * j4 + 1]);
          acc[32 + 4 * j4 + 2] = fmaf(__uint_as_float(c1[4 * j4 + 2]), f1.z, acc[32 + 4 * j4 + 2]);
          acc[32 + 4 * j4 + 3] = fmaf(__uint_as_float(c1[4 * j4 + 3]), f1.w, acc[32 + 4 * j4 + 3]);
        }
      }
      // ---- write this warp's 32 features x 64 tokens --------------------------------------------------
      const int n = t.n0 + 32 * q + lane;
      float bias = 0.f;
      if (p.bias != nullptr) bias = load_as_float(p.bias, p.bias_dtype, (int64_t)t.expert * p.n + n);
      const int esz = dtype_size(p.y_dtype);
      char* const ybase = reinterpret_cast<char*>(p.y) + (int64_t)n * esz;
      const int64_t ystride_b = p.y_stride * esz;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int col = half * 64 + 32 * cc + lane;        // the token whose output row this lane looks up
        int myrow = -1;
        if (col < t.count) {
          const int sp = t.row_start + col;
          myrow = p.y_rows != nullptr ? __ldg(p.y_rows + sp) : sp;
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int orow = __shfl_sync(0xffffffffu, myrow, j);
          if (orow >= 0) {
            const float v = acc[32 * cc + j] + bias;
            char* dst = ybase + orow * ystride_b;
            if (p.y_dtype == HQ_DT_F16) *reinterpret_cast<__half*>(dst) = __float2half_rn(v);
            else if (p.y_dtype == HQ_DT_BF16) *reinterpret_cast<__nv_bfloat16*>(dst) = __float2bfloat16_rn(v);
            else *reinterpret_cast<float*>(dst) = v;
          }
        }
      }
    }
  }

  f8_fence_before();
  __syncthreads();
  if (warp == 1) {
    f8_fence_after();
    f8_tmem_dealloc(tmem_base, 128 * kF8AccBufs);
  }
}

// ---- host -----------------------------------------------------------------------------------------
// cuTensorMapEncodeTiled is a driver entry point: it is looked up through the runtime when first needed, so the
// library itself does not depend on the driver library being present where no GPU is (builds, symbol checks).
typedef CUresult (*F8EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static F8EncodeTiledFn f8_encode_fn() {
  static F8EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<F8EncodeTiledFn>(ptr);
  }
  return fn;
}
static bool f8_encode_2d(CUtensorMap* map, CUtensorMapDataType type, const void* base, uint64_t inner, uint64_t rows,
                         uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle swz) {
  const F8EncodeTiledFn encode = f8_encode_fn();
  if (encode == nullptr) return false;
  cuuint64_t gdim[2] = {inner, rows};
  cuuint64_t gstride[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return encode(map, type, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool fp8_grouped_supported(int64_t n, int64_t k) {
  return n % 128 == 0 && k % 512 == 0 && k / 128 <= kF8MaxKB;
}

int32_t launch_fp8_grouped(const Fp8GroupedParams& p, int max_tiles, cudaStream_t stream) {
  if (!fp8_grouped_supported(p.n, p.k)) return HQ_ERR_SHAPE;
  if (p.n_rows <= 0 || max_tiles <= 0) return HQ_OK;
  CUtensorMap tm_w, tm_x, tm_s;
  if (!f8_encode_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.w, (uint64_t)p.k, (uint64_t)p.n_experts * p.n,
                    (uint64_t)p.k, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B) ||
      !f8_encode_2d(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.xq, (uint64_t)p.k, (uint64_t)p.n_rows, (uint64_t)p.k, 128,
                    128, CU_TENSOR_MAP_SWIZZLE_128B) ||
      !f8_encode_2d(&tm_s, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, p.xs, (uint64_t)(p.k / 128), (uint64_t)p.n_rows,
                    (uint64_t)(p.k / 128) * 4, (uint32_t)(p.k / 128), 128, CU_TENSOR_MAP_SWIZZLE_NONE))
    return HQ_ERR_CUDA;
  static bool attr_done[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return HQ_ERR_CUDA;
  if (dev < 64 && !attr_done[dev]) {
    if (cudaFuncSetAttribute(fp8_grouped_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F8Smem::TOTAL) !=
        cudaSuccess)
      return HQ_ERR_CUDA;
    attr_done[dev] = true;
  }
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  const int64_t items = (int64_t)max_tiles * (p.n / 128);
  const int64_t grid = items < sms ? items : sms;
  fp8_grouped_kernel<<<(unsigned)grid, kF8Threads, F8Smem::TOTAL, stream>>>(tm_w, tm_x, tm_s, p);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

}  // namespace hq
