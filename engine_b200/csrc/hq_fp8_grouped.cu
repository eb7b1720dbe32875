// Block-FP8 expert GEMM with FP8 activations on tcgen05 (kind::f8f6f4), nothing converted on the way in.
//
// y[row, n] = sum over 128-column blocks kb of  ws[expert, n/128, kb] * xs[row, kb] *
//             sum_{k in kb} e4m3(W[expert, n, k]) * e4m3(X[row, k])
// W: the reference's e4m3 codes [E, N, K] + f32 128x128 block scales; X: activation rows already quantized
// 1 x 128 (codes + one f32 scale per row and block) and already in expert-sorted order, so the token rows of one
// expert are a plain 2-D box.  Both operands go from HBM to shared memory by TMA (cp.async.bulk.tensor, 128-byte
// swizzle) and from there into the tensor core unchanged; the products of e4m3 values are exact and accumulate
// in f32 in tensor memory.  Because the scales change every 128 columns the accumulation is cut there: each
// 128-column block is multiplied into a fresh tensor-memory buffer (three in rotation) and the epilogue warps
// fold it into register accumulators with one packed FMA per two elements (factor = weight-block scale x the
// token's scale for that block) while the next blocks are being multiplied.
//
// Work item = (token tile, 128 output features).  Token tiles are cut inside the kernel from expert_bounds: an
// expert with c rows gets ceil(c / 144) tiles of equal size rounded up to 16 rows, and a tile's MMA is issued
// with N = its row count rounded up to 16, so an expert with 130 rows costs 144 columns, not 256.  Swapped
// roles: tensor-memory lanes = output features (MMA M = 128), columns = tokens (MMA N = 16 .. 144).
//
// Two modes.  Plain: one pass over K, output rows in f32 / f16 / bf16 (16-bit rows leave through a shared-memory
// transpose as 16-byte stores).  Gated: the item runs the gate bank's 128 rows over K, keeps gate (rounded to
// f16) in shared memory, runs the up bank's rows of the same features over K, applies the gated activation,
// rounds to f16, quantizes each token's 128 values 1 x 128 and writes e4m3 codes + scale: the {gate | up}
// matrix and the separate activation / quantization pass never touch HBM.
//
// Roles (one persistent CTA per SM, 16 warps): warp 0 issues TMA, warps 1 and 2 issue the MMAs of alternate
// 128-column blocks (one elected lane each), warp 3 builds the factor tables (four blocks at a time, four
// tables in rotation), warps 4-15 are the epilogue: warp w reads tensor-memory lanes 32 * (w % 4) .. + 31 (its
// 32 output features) and every third 16-column chunk.  Every wait is bounded; a wait that runs out is reported
// in the status word, the rest of the kernel's waits then poll once, nothing more is stored, and the kernel
// reaches its normal exit (tensor memory is always freed).  No multicast, no peer memory.
#include <cuda.h>
#include <cuda_fp8.h>

#include "hq_common.cuh"
#include "hq_kernels.h"

namespace hq {

constexpr int kF8Threads = 512;
constexpr int kF8Cap = 144;                              // most token rows per tile (MMA N), a multiple of 16
constexpr int kF8Stages = 5;
constexpr int kF8ATile = 128 * 128;                      // weight box: 128 rows x 128 bytes
constexpr int kF8BTile = kF8Cap * 128;                   // largest activation box
constexpr int kF8StageBytes = kF8ATile + kF8BTile;
constexpr int kF8MaxKB = 64;                             // 128-column blocks per row (K <= 8192)
constexpr int kF8AccBufs = 3;                            // accumulator buffers of kF8Cap columns in tensor memory
constexpr int kF8TmemCols = 512;
constexpr int kF8FacSlots = 4;                           // factor tables in rotation
constexpr int kF8FacBlocks = 4;                          // 128-column blocks per factor table
constexpr int kF8FacSlotBytes = kF8FacBlocks * kF8Cap * 4;
constexpr int kF8TilePitch = 272;                        // bytes per token row of the transposed tile (128 x 2 + pad)
constexpr int kF8EpiWarps = 12;
constexpr int kF8MaxExperts = 1024;
static_assert(kF8StageBytes % 1024 == 0, "stages stay 1024-byte aligned");
static_assert(kF8AccBufs * kF8Cap <= kF8TmemCols, "accumulator buffers fit tensor memory");

struct F8Smem {
  static constexpr int OFF_FAC = kF8Stages * kF8StageBytes;
  static constexpr int OFF_TILE = OFF_FAC + kF8FacSlots * kF8FacSlotBytes;
  static constexpr int OFF_PREF = OFF_TILE + kF8Cap * kF8TilePitch;
  static constexpr int OFF_BAR = OFF_PREF + (kF8MaxExperts + 1) * 4 + 12;
  static constexpr int N_BAR = 2 * kF8Stages + 2 * kF8AccBufs + 2 * kF8FacSlots;
  static constexpr int TOTAL = OFF_BAR + N_BAR * 8 + 16 + 1024;    // + alignment slack
};
static_assert(F8Smem::OFF_BAR % 8 == 0, "barriers are 8-byte aligned");
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
// 32 lanes x 16 consecutive 32-bit columns
__device__ __forceinline__ void f8_tmem_ld16(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void f8_tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// acc{0,1} += x{0,1} * f{0,1} as one packed instruction
__device__ __forceinline__ void f8_fma2(float& a0, float& a1, uint32_t x0, uint32_t x1, float f0, float f1) {
  asm("{\n"
      ".reg .b64 ra, rx, rf;\n"
      "mov.b64 ra, {%0, %1};\n"
      "mov.b64 rx, {%2, %3};\n"
      "mov.b64 rf, {%4, %5};\n"
      "fma.rn.f32x2 ra, rx, rf, ra;\n"
      "mov.b64 {%0, %1}, ra;\n"
      "}\n"
      : "+f"(a0), "+f"(a1)
      : "r"(x0), "r"(x1), "f"(f0), "f"(f1));
}

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
// kind::f8f6f4 instruction descriptor: f32 accumulate, A and B e4m3 (format code 0), both K-major, M = 128, N = ncols
__device__ __forceinline__ uint32_t f8_idesc(int ncols) {
  return (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(ncols >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

// one 2-D box by TMA; x = innermost (byte / element) coordinate, y = row
__device__ __forceinline__ void f8_tma_2d(void* dst_smem, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
          "r"(smem_u32(dst_smem)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ float f8_gated(float g, float u, const hq_act_args& a) {
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

struct F8Item {
  int expert, row_start, count, ncols, n0;
};
// Item w -> (token tile, feature tile).  pref[e] = tiles of the experts before e.
__device__ __forceinline__ F8Item f8_item(const Fp8GroupedParams& p, const int32_t* pref, int n_exp, int w, int n_nt) {
  F8Item t;
  const int tt = w / n_nt;
  t.n0 = (w - tt * n_nt) * 128;
  int lo = 0, hi = n_exp - 1;
  while (lo < hi) {                       // largest e with pref[e] <= tt (its own tile count is then > 0)
    const int mid = (lo + hi + 1) >> 1;
    if (pref[mid] <= tt) lo = mid; else hi = mid - 1;
  }
  t.expert = lo;
  int base = 0, cnt = p.m;
  if (p.expert_bounds != nullptr) {
    base = __ldg(p.expert_bounds + lo);
    cnt = __ldg(p.expert_bounds + lo + 1) - base;
  }
  const int ntile = pref[lo + 1] - pref[lo];
  const int j = tt - pref[lo];
  const int rpt = ((cnt + ntile - 1) / ntile + 15) & ~15;
  t.row_start = base + j * rpt;
  t.count = min(rpt, cnt - j * rpt);
  t.ncols = (t.count + 15) & ~15;
  return t;
}

__global__ void __launch_bounds__(kF8Threads, 1)
fp8_grouped_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_wu,
                   const __grid_constant__ CUtensorMap tm_x0, const __grid_constant__ CUtensorMap tm_x1,
                   const __grid_constant__ CUtensorMap tm_x2, const Fp8GroupedParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  float* fac = reinterpret_cast<float*>(smem + F8Smem::OFF_FAC);
  uint8_t* tile = smem + F8Smem::OFF_TILE;
  int32_t* pref = reinterpret_cast<int32_t*>(smem + F8Smem::OFF_PREF);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + F8Smem::OFF_BAR);
  uint64_t* empty = full + kF8Stages;
  uint64_t* acc_full = empty + kF8Stages;            // [3] a 128-column block has been multiplied into buffer b
  uint64_t* acc_empty = acc_full + kF8AccBufs;       // [3] ... and has been read out by all epilogue warps
  uint64_t* fac_full = acc_empty + kF8AccBufs;       // [4] a factor table has been written
  uint64_t* fac_empty = fac_full + kF8FacSlots;      // [4] ... and every epilogue warp is done with it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(fac_empty + kF8FacSlots);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_nt = p.n / 128;
  const int KB = p.k / 128;
  const int n_exp = p.expert_bounds != nullptr ? p.n_experts : 1;
  const int npass = p.w_up != nullptr ? 2 : 1;

  // ---- token tiles per expert -> exclusive prefix -------------------------------------------------------
  for (int e = tid; e < n_exp; e += kF8Threads) {
    const int cnt = p.expert_bounds != nullptr ? __ldg(p.expert_bounds + e + 1) - __ldg(p.expert_bounds + e) : p.m;
    pref[e + 1] = (cnt + kF8Cap - 1) / kF8Cap;
  }
  if (tid == 0) {
    pref[0] = 0;
    for (int s = 0; s < kF8Stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < kF8AccBufs; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], kF8EpiWarps);
    }
    for (int b = 0; b < kF8FacSlots; ++b) {
      mbar_init(&fac_full[b], 1);
      mbar_init(&fac_empty[b], kF8EpiWarps);
    }
    fence_barrier_init();
  }
  __syncthreads();
  if (warp == 0) {
    int carry = 0;
    for (int base = 0; base < n_exp; base += 32) {
      const int e = base + lane;
      int v = e < n_exp ? pref[e + 1] : 0;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += o;
      }
      if (e < n_exp) pref[e + 1] = carry + v;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
  }
  if (warp == 1) {
    f8_tmem_alloc(smem_u32(tmem_slot), kF8TmemCols);
    f8_tmem_relinquish();
  }
  f8_fence_before();
  __syncthreads();
  f8_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total = pref[n_exp] * n_nt;
  const uint32_t spin_limit = p.spin_limit;

  if (warp == 0) {
    // =========================== TMA issuer =========================================================
    if (lane == 0 && !p.test_skip_producer) {
      uint32_t spin = spin_limit;
      int s = 0, round = 0;
      for (int w = blockIdx.x; w < total; w += gridDim.x) {
        const F8Item t = f8_item(p, pref, n_exp, w, n_nt);
        const CUtensorMap* mx = t.ncols <= 48 ? &tm_x0 : (t.ncols <= 96 ? &tm_x1 : &tm_x2);
        const uint32_t box_bytes = (uint32_t)(t.ncols <= 48 ? 48 : (t.ncols <= 96 ? 96 : kF8Cap)) * 128u;
        const int wrow = t.expert * p.n + t.n0;
        for (int pass = 0; pass < npass; ++pass) {
          const CUtensorMap* mw = pass == 0 ? &tm_w : &tm_wu;
          for (int kb = 0; kb < KB; ++kb) {
            if (round > 0) {
              if (!mbar_wait_backoff(&empty[s], (round - 1) & 1, spin)) {
                report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 710 + s);
                spin = 1;
              }
            }
            uint8_t* stage = smem + s * kF8StageBytes;
            mbar_arrive_expect_tx(&full[s], (uint32_t)kF8ATile + box_bytes);
            f8_tma_2d(stage, mw, kb * 128, wrow, &full[s]);
            f8_tma_2d(stage + kF8ATile, mx, kb * 128, t.row_start, &full[s]);
            if (++s == kF8Stages) {
              s = 0;
              ++round;
            }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1 || warp == 2) {
    // =========================== MMA issuers ========================================================
    // tcgen05.commit holds its thread until the MMAs before it have gone through the pipe, and the waits that
    // follow would leave the tensor core idle: two issuing lanes take alternate 128-column blocks, so one is
    // always ready to issue while the other waits
    if (lane == 0) {
      const int me = warp - 1;
      uint32_t spin = spin_limit;
      bool failed = false;
      int blk = 0;      // 128-column blocks so far (buffer = blk % kF8AccBufs, stage = blk % kF8Stages)
      for (int w = blockIdx.x; w < total; w += gridDim.x) {
        const F8Item t = f8_item(p, pref, n_exp, w, n_nt);
        const uint32_t idesc = f8_idesc(t.ncols);
        for (int i = 0; i < npass * KB; ++i, ++blk) {
          if ((blk & 1) != me) continue;
          const int buf = blk % kF8AccBufs;
          const int s = blk % kF8Stages;
          if (blk >= kF8AccBufs) {
            if (!mbar_wait(&acc_empty[buf], ((blk / kF8AccBufs) - 1) & 1, spin)) {
              report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 720 + buf);
              spin = 1;
              failed = true;
            }
          }
          if (!mbar_wait(&full[s], (blk / kF8Stages) & 1, spin)) {
            report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 730 + s);
            spin = 1;
            failed = true;
          }
          if (failed) continue;        // nothing more is multiplied once a wait has run out
          f8_fence_after();
          const uint32_t stage = smem_u32(smem + s * kF8StageBytes);
          const uint64_t adesc = f8_smem_desc(stage), bdesc = f8_smem_desc(stage + kF8ATile);
          const uint32_t d = tmem_base + (uint32_t)(buf * kF8Cap);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)   // 32 k = 32 bytes per instruction: advance the start address by 2 units
            f8_mma(d, adesc + 2 * kk, bdesc + 2 * kk, idesc, kk > 0 ? 1u : 0u);
          f8_commit(&empty[s]);        // the stage is free once these MMAs have read it
          f8_commit(&acc_full[buf]);   // the block's products are complete
        }
      }
    }
    __syncwarp();
  } else if (warp == 3) {
    // =========================== factor tables ======================================================
    // fac[slot][b][token] = weight-block scale(kb) x token scale(token, kb) for the four blocks kb = 4c + b of
    // chunk c: the epilogue reads four tokens per shared load at fixed offsets and spends one packed FMA per two
    // elements.  Rows are read straight from the scale matrix (L2-resident) one 16-byte load per token and chunk.
    uint32_t spin = spin_limit;
    int chunk = 0;
    for (int w = blockIdx.x; w < total; w += gridDim.x) {
      const F8Item t = f8_item(p, pref, n_exp, w, n_nt);
      for (int pass = 0; pass < npass; ++pass) {
        const float* wsc = (pass == 0 ? p.w_scales : p.w_up_scales) +
                           ((int64_t)t.expert * p.fp8_nb + t.n0 / 128) * p.fp8_kb;
        for (int c4 = 0; c4 < KB / kF8FacBlocks; ++c4, ++chunk) {
          const int slot = chunk % kF8FacSlots;
          float4 v[5];
#pragma unroll
          for (int r = 0; r < 5; ++r) {
            const int tok = lane + 32 * r;
            v[r] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (tok < t.count)
              v[r] = __ldg(reinterpret_cast<const float4*>(p.xs + (int64_t)(t.row_start + tok) * KB + 4 * c4));
          }
          const float4 ws4 = __ldg(reinterpret_cast<const float4*>(wsc + 4 * c4));
          if (chunk >= kF8FacSlots) {
            if (!mbar_wait_backoff(&fac_empty[slot], ((chunk / kF8FacSlots) - 1) & 1, spin)) {
              if (lane == 0) report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 760 + slot);
              spin = 1;
            }
          }
          float* dst = fac + slot * (kF8FacBlocks * kF8Cap);
#pragma unroll
          for (int r = 0; r < 5; ++r) {
            const int tok = lane + 32 * r;
            if (tok < t.ncols) {
              dst[tok] = v[r].x * ws4.x;
              dst[kF8Cap + tok] = v[r].y * ws4.y;
              dst[2 * kF8Cap + tok] = v[r].z * ws4.z;
              dst[3 * kF8Cap + tok] = v[r].w * ws4.w;
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&fac_full[slot]);
        }
      }
    }
  } else {
    // =========================== epilogue ===========================================================
    const int q = warp & 3;                 // tensor-memory lane quarter this warp may read
    const int third = (warp - 4) >> 2;      // takes the 16-column chunks 3i + third
    const int et = tid - 128;               // 0 .. 383 among the epilogue threads
    uint32_t spin = spin_limit;
    bool failed = false;
    int blk = 0, chunk = 0;
    const bool y16 = p.y_dtype != HQ_DT_F32;
    const bool via_tile = npass == 2 || (y16 && p.y_tile_ok);
    for (int w = blockIdx.x; w < total; w += gridDim.x) {
      const F8Item t = f8_item(p, pref, n_exp, w, n_nt);
      const int n = t.n0 + 32 * q + lane;
      float acc[48];
#pragma unroll
      for (int j = 0; j < 48; ++j) acc[j] = 0.f;
      for (int pass = 0; pass < npass; ++pass) {
        for (int kb = 0; kb < KB; ++kb, ++blk) {
          const int slot = chunk % kF8FacSlots;
          if ((kb & (kF8FacBlocks - 1)) == 0) {
            if (!mbar_wait(&fac_full[slot], (chunk / kF8FacSlots) & 1, spin)) {
              if (lane == 0) report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 740 + slot);
              spin = 1;
              failed = true;
            }
          }
          const int buf = blk % kF8AccBufs;
          if (!mbar_wait(&acc_full[buf], (blk / kF8AccBufs) & 1, spin)) {
            if (lane == 0) report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 750 + buf);
            spin = 1;
            failed = true;
          }
          if (!failed) {
            f8_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(buf * kF8Cap);
            uint32_t c[48];
#pragma unroll
            for (int i = 0; i < 3; ++i) {
              const int col0 = 16 * (3 * i + third);
              if (col0 < t.ncols) f8_tmem_ld16(taddr + col0, &c[16 * i]);
            }
            f8_tmem_ld_wait();
            f8_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);     // the buffer may be overwritten: values are in registers
            const uint32_t fk = smem_u32(fac) + (uint32_t)(slot * kF8FacSlotBytes) +
                                (uint32_t)((kb & (kF8FacBlocks - 1)) * kF8Cap * 4);
#pragma unroll
            for (int i = 0; i < 3; ++i) {
              const int col0 = 16 * (3 * i + third);
              if (col0 < t.ncols) {
#pragma unroll
                for (int j4 = 0; j4 < 4; ++j4) {
                  float4 f;
                  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                               : "=f"(f.x), "=f"(f.y), "=f"(f.z), "=f"(f.w) : "r"(fk + 4u * (col0 + 4 * j4)));
                  f8_fma2(acc[16 * i + 4 * j4 + 0], acc[16 * i + 4 * j4 + 1], c[16 * i + 4 * j4 + 0],
                          c[16 * i + 4 * j4 + 1], f.x, f.y);
                  f8_fma2(acc[16 * i + 4 * j4 + 2], acc[16 * i + 4 * j4 + 3], c[16 * i + 4 * j4 + 2],
                          c[16 * i + 4 * j4 + 3], f.z, f.w);
                }
              }
            }
          }
          if ((kb & (kF8FacBlocks - 1)) == kF8FacBlocks - 1) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&fac_empty[slot]);
            ++chunk;
          }
        }
        // ---- end of a pass over K: this warp holds 32 features x its chunks of the tile's tokens -----
        float bias = 0.f;
        const void* bias_p = pass == 0 ? p.bias : p.bias_up;
        if (bias_p != nullptr) bias = load_as_float(bias_p, p.bias_dtype, (int64_t)t.expert * p.n + n);
        if (via_tile) {
          // [token][feature] tile of 16-bit values: each thread writes (and, in gated mode, later reads back)
          // only its own positions, so no barrier is needed until rows are read across threads
          const bool last = pass == npass - 1;
#pragma unroll
          for (int i = 0; i < 3; ++i) {
            const int col0 = 16 * (3 * i + third);
            if (col0 < t.ncols) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                uint8_t* cell = tile + (col0 + j) * kF8TilePitch + (32 * q + lane) * 2;
                float v = acc[16 * i + j] + bias;
                if (npass == 2) {
                  // gate and up are rounded to f16 where a 16-bit pipeline would store them; the activated value
                  // is rounded once more before the quantizer sees it
                  v = __half2float(__float2half_rn(v));
                  if (last) v = f8_gated(__half2float(*reinterpret_cast<const __half*>(cell)), v, p.act);
                  *reinterpret_cast<__half*>(cell) = __float2half_rn(v);
                } else if (p.y_dtype == HQ_DT_F16) {
                  *reinterpret_cast<__half*>(cell) = __float2half_rn(v);
                } else {
                  *reinterpret_cast<__nv_bfloat16*>(cell) = __float2bfloat16_rn(v);
                }
                acc[16 * i + j] = 0.f;
              }
            }
          }
          if (last) {
            named_bar_sync(2, 32 * kF8EpiWarps);
            // two threads per token row, 64 features each
            const int row = et >> 1, hf = et & 1;
            const bool live = row < t.count && !failed;
            const uint8_t* src = tile + row * kF8TilePitch + hf * 128;
            if (npass == 2) {
              float m = 0.f;
              if (row < kF8Cap) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const uint4 raw = *reinterpret_cast<const uint4*>(src + 16 * i);
                  const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const float2 f = __half22float2(__habs2(h2[j]));
                    m = fmaxf(m, fmaxf(f.x, f.y));
                  }
                }
              }
              m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
              if (live) {
                const float scale = m > 0.f ? __fdiv_rn(m, 448.f) : 1e-12f;
                const int64_t orow = t.row_start + row;
                uint8_t* dst = p.hq + orow * p.n + t.n0 + 64 * hf;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  uint32_t wds[4];
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    // four f16 values = 8 bytes of the tile row -> four e4m3 codes
                    const uint2 raw = *reinterpret_cast<const uint2*>(src + 32 * i + 8 * j);
                    const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
                    const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                    const float vv[4] = {f0.x, f0.y, f1.x, f1.y};
                    uint32_t pk = 0;
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                      const float qv = fminf(fmaxf(__fdiv_rn(vv[b], scale), -448.f), 448.f);
                      pk |= (uint32_t)__nv_cvt_float_to_fp8(qv, __NV_SATFINITE, __NV_E4M3) << (8 * b);
                    }
                    wds[j] = pk;
                  }
                  *reinterpret_cast<uint4*>(dst + 16 * i) = make_uint4(wds[0], wds[1], wds[2], wds[3]);
                }
                if (hf == 0) p.hs[orow * (p.n / 128) + t.n0 / 128] = scale;
              }
            } else if (live) {
              const int sp = t.row_start + row;
              const int64_t orow = p.y_rows != nullptr ? (int64_t)__ldg(p.y_rows + sp) : (int64_t)sp;
              uint8_t* dst = reinterpret_cast<uint8_t*>(p.y) + (orow * p.y_stride + t.n0 + 64 * hf) * 2;
#pragma unroll
              for (int i = 0; i < 8; ++i)
                *reinterpret_cast<uint4*>(dst + 16 * i) = *reinterpret_cast<const uint4*>(src + 16 * i);
            }
            named_bar_sync(2, 32 * kF8EpiWarps);     // the tile may be written again
          }
        } else {
          // direct stores (f32 rows, or 16-bit rows whose stride rules out 16-byte stores)
          const int esz = dtype_size(p.y_dtype);
          char* const ybase = reinterpret_cast<char*>(p.y) + (int64_t)n * esz;
          const int64_t ystride_b = p.y_stride * esz;
#pragma unroll
          for (int i = 0; i < 3; ++i) {
            const int col0 = 16 * (3 * i + third);
            if (col0 < t.ncols) {
              int myrow = -1;
              if (lane < 16 && col0 + lane < t.count && !failed) {
                const int sp = t.row_start + col0 + lane;
                myrow = p.y_rows != nullptr ? __ldg(p.y_rows + sp) : sp;
              }
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const int64_t orow = __shfl_sync(0xffffffffu, myrow, j);
                if (orow >= 0) {
                  const float v = acc[16 * i + j] + bias;
                  char* dst = ybase + orow * ystride_b;
                  if (p.y_dtype == HQ_DT_F16) *reinterpret_cast<__half*>(dst) = __float2half_rn(v);
                  else if (p.y_dtype == HQ_DT_BF16) *reinterpret_cast<__nv_bfloat16*>(dst) = __float2bfloat16_rn(v);
                  else *reinterpret_cast<float*>(dst) = v;
                }
              }
            }
          }
        }
      }
    }
  }

  f8_fence_before();
  __syncthreads();
  if (warp == 1) {
    f8_fence_after();
    f8_tmem_dealloc(tmem_base, kF8TmemCols);
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

int32_t launch_fp8_grouped(const Fp8GroupedParams& p_in, cudaStream_t stream) {
  Fp8GroupedParams p = p_in;
  if (!fp8_grouped_supported(p.n, p.k)) return HQ_ERR_SHAPE;
  if (p.expert_bounds != nullptr && p.n_experts > kF8MaxExperts) return HQ_ERR_SHAPE;
  if (p.n_rows <= 0) return HQ_OK;
  CUtensorMap tm_w, tm_wu, tm_x[3];
  const uint64_t wrows = (uint64_t)(p.expert_bounds != nullptr ? p.n_experts : 1) * p.n;
  if (!f8_encode_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.w, (uint64_t)p.k, wrows, (uint64_t)p.k, 128, 128,
                    CU_TENSOR_MAP_SWIZZLE_128B))
    return HQ_ERR_CUDA;
  tm_wu = tm_w;
  if (p.w_up != nullptr && !f8_encode_2d(&tm_wu, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.w_up, (uint64_t)p.k, wrows,
                                         (uint64_t)p.k, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B))
    return HQ_ERR_CUDA;
  const uint32_t box_rows[3] = {48, 96, (uint32_t)kF8Cap};
  for (int i = 0; i < 3; ++i)
    if (!f8_encode_2d(&tm_x[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, p.xq, (uint64_t)p.k, (uint64_t)p.n_rows, (uint64_t)p.k,
                      128, box_rows[i], CU_TENSOR_MAP_SWIZZLE_128B))
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
  // the kernel cuts the token tiles itself; this is only an upper bound on the items, for small calls
  const int64_t n_exp = p.expert_bounds != nullptr ? p.n_experts : 1;
  const int64_t max_tiles = p.n_rows / kF8Cap + n_exp;
  const int64_t items = max_tiles * (p.n / 128);
  const int64_t grid = items < sms ? items : sms;
  // 16-bit rows leave through the transposed tile when every row segment can be written with 16-byte stores
  p.y_tile_ok = p.y != nullptr && p.y_dtype != HQ_DT_F32 && (reinterpret_cast<uintptr_t>(p.y) & 15u) == 0 &&
                (p.y_stride % 8) == 0;
  if (p.spin_limit == 0) p.spin_limit = 1u << 22;
  fp8_grouped_kernel<<<(unsigned)grid, kF8Threads, F8Smem::TOTAL, stream>>>(tm_w, tm_wu, tm_x[0], tm_x[1], tm_x[2], p);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

}  // namespace hq
