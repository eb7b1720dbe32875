// Block-FP8 expert GEMM with FP8 activations on tcgen05 (kind::f8f6f4), nothing converted on the way in.
//
// y[row, n] = sum over 128-column blocks kb of  ws[expert, n/128, kb] * xs[row, kb] *
//             sum_{k in kb} e4m3(X[row, k]) * e4m3(W[expert, n, k])
// W: the reference's e4m3 codes [E, N, K] + f32 128x128 block scales; X: activation rows already quantized
// 1 x 128 (codes + one f32 scale per row and block) and already in expert-sorted order, so the token rows of one
// expert are a plain 2-D box.  Both operands go from HBM to shared memory by TMA (cp.async.bulk.tensor, 128-byte
// swizzle) and from there into the tensor core unchanged; the products of e4m3 values are exact and accumulate
// in f32 in tensor memory.  Because the scales change every 128 columns the accumulation is cut there: each
// 128-column block is multiplied into a fresh tensor-memory buffer (four in rotation) and the epilogue warps
// fold it into register accumulators while the next blocks are being multiplied.
//
// Orientation: tensor-memory lanes = tokens (MMA M = 128, A = the token tile), columns = output features (MMA
// N = 128, B = the weight tile).  The factor of a block, weight-block scale x token scale, is then ONE scalar per
// epilogue thread and block, so folding a block costs one packed FMA per two elements and a single shared load
// (with features on the lanes every element needs its own factor, and the loads for them cost more than the
// arithmetic).  Work item = (token tile of <= 128 rows of one expert, 128 output features); the tiles are cut
// inside the kernel from expert_bounds; the token box that is fetched has 32, 64, 96 or 128 rows, and lane
// quarters without tokens are not drained.
//
// Two modes.  Plain: one pass over K, each thread writes its token's 32 features as 16-byte stores.  Gated: the item
// runs the gate bank's 128 rows over K, parks gate (rounded to f16) in shared memory, runs the up bank's rows of
// the same features over K, applies the gated activation, rounds to f16, quantizes the token's 128 values 1 x 128
// (the four warps that share a token exchange their maxima) and writes e4m3 codes + scale: the {gate | up} matrix
// and the separate activation / quantization pass never touch HBM.
//
// Roles (one persistent CTA per SM, 20 warps): warp 0 issues TMA, warps 1 and 2 issue the MMAs of alternate
// 128-column blocks (one elected lane each), warp 3 builds the factor tables (four blocks at a time, four tables
// in rotation, loads four tables ahead), warps 4-19 are the epilogue: warp w reads tensor-memory lanes
// 32 * (w % 4) .. + 31 (its 32 tokens) and the 32 feature columns 32 * ((w - 4) / 4) .. + 31.  Every wait is
// bounded; a wait that runs out is reported in the status word, the rest of the kernel's waits then poll once,
// nothing more is multiplied or stored, and the kernel reaches its normal exit (tensor memory is always freed).
// No multicast, no peer memory.
#include <cuda.h>
#include <cuda_fp8.h>

#include "hq_common.cuh"
#include "hq_kernels.h"

namespace hq {

// Developer instrumentation, compiled out unless HQ_F8_PROFILE is defined: cycles each role spends in its waits,
// summed over CTAs into g_f8_prof (read back with hq_debug_f8_prof).
#ifdef HQ_F8_PROFILE
__device__ unsigned long long g_f8_prof[16];
#define F8_PROF_BEGIN() const long long prof_t0__ = clock64()
#define F8_PROF_END(idx, cond) do { if (cond) atomicAdd(&g_f8_prof[idx], (unsigned long long)(clock64() - prof_t0__)); } while (0)
#else
#define F8_PROF_BEGIN() do {} while (0)
#define F8_PROF_END(idx, cond) do {} while (0)
#endif

constexpr int kF8Threads = 640;
constexpr int kF8Rows = 128;                             // token rows per tile (MMA M)
#ifdef HQ_F8_STAGES
constexpr int kF8Stages = HQ_F8_STAGES;                // experiment builds only
#else
constexpr int kF8Stages = 5;
#endif
constexpr int kF8WTile = 128 * 128;                      // weight box: 128 rows x 128 bytes
constexpr int kF8XTile = kF8Rows * 128;                  // largest token box
constexpr int kF8StageBytes = kF8WTile + kF8XTile;
constexpr int kF8MaxKB = 64;                             // 128-column blocks per row (K <= 8192)
constexpr int kF8AccBufs = 4;                            // 128-column accumulator buffers in tensor memory
constexpr int kF8TmemCols = 512;
constexpr int kF8FacSlots = 4;                           // factor tables in rotation
constexpr int kF8FacBlocks = 4;                          // 128-column blocks per factor table
constexpr int kF8FacSlotBytes = kF8FacBlocks * kF8Rows * 4;
constexpr int kF8EpiWarps = 16;
constexpr int kF8MaxExperts = 1024;
static_assert(kF8StageBytes % 1024 == 0, "stages stay 1024-byte aligned");

struct F8Smem {
  static constexpr int OFF_FAC = kF8Stages * kF8StageBytes;
  static constexpr int OFF_GATE = OFF_FAC + kF8FacSlots * kF8FacSlotBytes;   // gate values parked between the passes
#ifdef HQ_F8_STREAM_ONLY
  static constexpr int OFF_MAX = OFF_GATE + 16;
#else
  static constexpr int OFF_MAX = OFF_GATE + kF8Rows * 128 * 2;               // [4 column parts][128 tokens] maxima
#endif
  static constexpr int OFF_PREF = OFF_MAX + 4 * kF8Rows * 4;
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
// 32 lanes x 32 consecutive 32-bit columns
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

// Packed f32 pairs: the running sums live in 64-bit registers so that one fma.rn.f32x2 serves two elements
// without any register moves around it.
__device__ __forceinline__ uint64_t f8_pack2(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void f8_unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f8_fma2(uint64_t x, uint64_t f, uint64_t acc) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(x), "l"(f), "l"(acc));
  return r;
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
  int expert, row_start, count, n0;
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
  const int j = tt - pref[lo];
  t.row_start = base + j * kF8Rows;
  t.count = min(kF8Rows, cnt - j * kF8Rows);
  return t;
}

// Walks the (item, pass, chunk of four 128-column blocks) sequence of one CTA, in the order every role follows.
struct F8ChunkCursor {
  int w, pass, c4;
  bool valid;
  F8Item t;
  __device__ __forceinline__ void start(const Fp8GroupedParams& p, const int32_t* pref, int n_exp, int n_nt,
                                        int total) {
    w = blockIdx.x;
    pass = 0;
    c4 = 0;
    valid = w < total;
    if (valid) t = f8_item(p, pref, n_exp, w, n_nt);
  }
  __device__ __forceinline__ void next(const Fp8GroupedParams& p, const int32_t* pref, int n_exp, int n_nt, int total,
                                       int npass, int KB) {
    if (!valid) return;
    if (++c4 < KB / kF8FacBlocks) return;
    c4 = 0;
    if (++pass < npass) return;
    pass = 0;
    w += gridDim.x;
    valid = w < total;
    if (valid) t = f8_item(p, pref, n_exp, w, n_nt);
  }
  // the chunk's token scales (four tokens per lane) and its four weight-block scales
  __device__ __forceinline__ void load(const Fp8GroupedParams& p, int KB, int lane, float4 (&v)[4],
                                       float4& ws4) const {
    const int count = valid ? t.count : 0;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int tok = lane + 32 * r;
      v[r] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (tok < count)
        v[r] = __ldg(reinterpret_cast<const float4*>(p.xs + (int64_t)(t.row_start + tok) * KB + 4 * c4));
    }
    ws4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (valid) {
      const float* wsc = (pass == 0 ? p.w_scales : p.w_up_scales) +
                         ((int64_t)t.expert * p.fp8_nb + t.n0 / 128) * p.fp8_kb;
      ws4 = __ldg(reinterpret_cast<const float4*>(wsc + 4 * c4));
    }
  }
  // Pull the weight bytes of this chunk and the next one of the item's 128 rows into L2, 1 KiB of every row at a
  // time, with one tensor prefetch (map over the bank as 32-bit words, box = 256 words x 128 rows).  The operand
  // boxes that follow take 128 bytes of each row; on their own they open 128 DRAM pages per box.  Called four
  // chunks (sixteen blocks) ahead of the multiply, by one lane.
  __device__ __forceinline__ void prefetch_weights(const Fp8GroupedParams& p, const CUtensorMap* pf_gate,
                                                   const CUtensorMap* pf_up) const {
    if (!valid || (c4 & 1) != 0) return;
    const CUtensorMap* m = pass == 0 ? pf_gate : pf_up;
    const int x = c4 * (kF8FacBlocks * 128 / 4);      // in 32-bit words
    const int y = t.expert * p.n + t.n0;
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(reinterpret_cast<uint64_t>(m)),
                 "r"(x), "r"(y)
                 : "memory");
  }
};

__global__ void __launch_bounds__(kF8Threads, 1)
fp8_grouped_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_wu,
                   const __grid_constant__ CUtensorMap tm_x0, const __grid_constant__ CUtensorMap tm_x1,
                   const __grid_constant__ CUtensorMap tm_x2, const __grid_constant__ CUtensorMap tm_x3,
                   const __grid_constant__ CUtensorMap tm_pf, const __grid_constant__ CUtensorMap tm_pfu,
                   const Fp8GroupedParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  float* fac = reinterpret_cast<float*>(smem + F8Smem::OFF_FAC);
  uint8_t* gate_park = smem + F8Smem::OFF_GATE;
  float* row_max = reinterpret_cast<float*>(smem + F8Smem::OFF_MAX);
  int32_t* pref = reinterpret_cast<int32_t*>(smem + F8Smem::OFF_PREF);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + F8Smem::OFF_BAR);
  uint64_t* empty = full + kF8Stages;
  uint64_t* acc_full = empty + kF8Stages;            // [4] a 128-column block has been multiplied into buffer b
  uint64_t* acc_empty = acc_full + kF8AccBufs;       // [4] ... and has been read out by all epilogue warps
  uint64_t* fac_full = acc_empty + kF8AccBufs;       // [4] a factor table has been written
  uint64_t* fac_empty = fac_full + kF8FacSlots;      // [4] ... and every epilogue warp is done with it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(fac_empty + kF8FacSlots);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_nt = p.n / 128;
  const int KB = p.k / 128;
  const int n_exp = p.expert_bounds != nullptr ? p.n_experts : 1;
  const int npass = p.w_up != nullptr ? 2 : 1;
#ifdef HQ_F8_PROFILE
  const long long prof_kernel_t0 = clock64();
#endif

  // ---- token tiles per expert -> exclusive prefix -------------------------------------------------------
  for (int e = tid; e < n_exp; e += kF8Threads) {
    const int cnt = p.expert_bounds != nullptr ? __ldg(p.expert_bounds + e + 1) - __ldg(p.expert_bounds + e) : p.m;
    pref[e + 1] = (cnt + kF8Rows - 1) / kF8Rows;
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
    if (lane == 0 && p.test_skip_producer != 1) {
      const uint32_t spin = spin_limit;
      int s = 0, round = 0;
      int issued = 0;              // stages handed to the copy engine so far
      bool stop = false;           // a wait ran out: nothing more is issued (the stage may still be in use)
      const int burst = p.load_burst;
      for (int w = blockIdx.x; w < total && !stop; w += gridDim.x) {
        const F8Item t = f8_item(p, pref, n_exp, w, n_nt);
        // the smallest token box that covers the tile (rows past it keep whatever the stage held: they only feed
        // tensor-memory lanes nobody reads)
        const int bsel = (t.count + 31) >> 5;        // 1 .. 4
        const CUtensorMap* mx = bsel == 1 ? &tm_x0 : (bsel == 2 ? &tm_x1 : (bsel == 3 ? &tm_x2 : &tm_x3));
        const uint32_t box_bytes = (uint32_t)bsel * 32u * 128u;
        const int wrow = t.expert * p.n + t.n0;
        for (int pass = 0; pass < npass && !stop; ++pass) {
          const CUtensorMap* mw = pass == 0 ? &tm_w : &tm_wu;
          // `burst` consecutive blocks are requested together, so that every weight row is read burst x 128
          // contiguous bytes at a time (a 128-row box on its own touches 128 DRAM pages for 128 bytes each)
          for (int kb0 = 0; kb0 < KB && !stop; kb0 += burst) {
            int s2 = s, round2 = round;
            for (int b = 0; b < burst; ++b) {
              if (round2 > 0) {
                F8_PROF_BEGIN();
                if (!mbar_wait(&empty[s2], (round2 - 1) & 1, spin)) {
                  report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 710 + s2);
                  stop = true;
                }
                F8_PROF_END(0, true);
              }
              if (stop) break;
              if (++s2 == kF8Stages) {
                s2 = 0;
                ++round2;
              }
            }
            if (stop) break;
            s2 = s;
#ifdef HQ_F8_STREAM_ONLY
            // experiment: test_skip_producer 2 = weights only, 3 = tokens only
            const bool do_w = p.test_skip_producer != 3, do_x = p.test_skip_producer != 2;
#else
            constexpr bool do_w = true, do_x = true;
#endif
            for (int b = 0; b < burst; ++b) {
              uint8_t* stage = smem + s2 * kF8StageBytes;
              mbar_arrive_expect_tx(&full[s2], (do_w ? (uint32_t)kF8WTile : 0u) + (do_x ? box_bytes : 0u));
              if (do_w) f8_tma_2d(stage, mw, (kb0 + b) * 128, wrow, &full[s2]);
              if (++s2 == kF8Stages) s2 = 0;
            }
            s2 = s;
            for (int b = 0; b < burst; ++b) {
              uint8_t* stage = smem + s2 * kF8StageBytes;
              if (do_x) f8_tma_2d(stage + kF8WTile, mx, (kb0 + b) * 128, t.row_start, &full[s2]);
              if (++s2 == kF8Stages) s2 = 0;
            }
            for (int b = 0; b < burst; ++b) {
              if (++s == kF8Stages) {
                s = 0;
                ++round;
              }
            }
            issued += burst;
          }
        }
      }
      // no copy may still be writing this CTA's shared memory when it exits: wait (bounded) for the last copies of
      // every stage.  On the normal path the MMA warps consumed them long ago and these waits return at once.
      for (int j = 0; j < kF8Stages && j < issued; ++j) {
        const int idx = issued - 1 - j;
        if (!mbar_wait(&full[idx % kF8Stages], (idx / kF8Stages) & 1, spin)) break;
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
      const uint32_t idesc = f8_idesc();
      uint32_t spin = spin_limit;
      bool failed = false;
      int blk = 0;      // 128-column blocks so far (buffer = blk % kF8AccBufs, stage = blk % kF8Stages)
      for (int w = blockIdx.x; w < total; w += gridDim.x) {
        for (int i = 0; i < npass * KB; ++i, ++blk) {
          if ((blk & 1) != me) continue;
          const int buf = blk % kF8AccBufs;
          const int s = blk % kF8Stages;
#ifndef HQ_F8_STREAM_ONLY
          if (blk >= kF8AccBufs) {
            F8_PROF_BEGIN();
            if (!mbar_wait(&acc_empty[buf], ((blk / kF8AccBufs) - 1) & 1, spin)) {
              report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 720 + buf);
              spin = 1;
              failed = true;
            }
            F8_PROF_END(1, me == 0);
          }
#endif
          {
            F8_PROF_BEGIN();
            if (!mbar_wait(&full[s], (blk / kF8Stages) & 1, spin)) {
              report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 730 + s);
              spin = 1;
              failed = true;
            }
            F8_PROF_END(2, me == 0);
          }
          if (failed) continue;        // nothing more is multiplied once a wait has run out
#ifdef HQ_F8_STREAM_ONLY
          mbar_arrive(&empty[s]);      // experiment: loads only, nothing is multiplied or drained
          continue;
#endif
          f8_fence_after();
          const uint32_t stage = smem_u32(smem + s * kF8StageBytes);
          // A = the token tile (tensor-memory lanes), B = the weight tile (columns)
          const uint64_t adesc = f8_smem_desc(stage + kF8WTile), bdesc = f8_smem_desc(stage);
          const uint32_t d = tmem_base + (uint32_t)(buf * 128);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)   // 32 k = 32 bytes per instruction: advance the start address by 2 units
            f8_mma(d, adesc + 2 * kk, bdesc + 2 * kk, idesc, kk > 0 ? 1u : 0u);
          {
            F8_PROF_BEGIN();
            f8_commit(&empty[s]);        // the stage is free once these MMAs have read it
            f8_commit(&acc_full[buf]);   // the block's products are complete
            F8_PROF_END(3, me == 0);
          }
        }
      }
    }
    __syncwarp();
#ifdef HQ_F8_STREAM_ONLY
  } else if (warp >= 3) {
    // experiment: idle
#endif
  } else if (warp == 3) {
    // =========================== factor tables ======================================================
    // fac[slot][b][token] = weight-block scale(kb) x token scale(token, kb) for the four blocks kb = 4c + b of
    // chunk c.  Rows are read straight from the scale matrix, one 16-byte load per token and chunk; under load
    // such a read takes microseconds, so the loads of chunk c + 4 are in flight while chunk c is written.
    uint32_t spin = spin_limit;
    constexpr int D = 4;                      // chunks of loads in flight
    F8ChunkCursor pre, cur;                   // the chunk being loaded / being written
    pre.start(p, pref, n_exp, n_nt, total);
    cur = pre;
    float4 v[D][4], ws4[D];
#pragma unroll
    for (int d = 0; d < D; ++d) {
      if (p.l2_prefetch && lane == 0) pre.prefetch_weights(p, &tm_pf, &tm_pfu);
      pre.load(p, KB, lane, v[d], ws4[d]);
      pre.next(p, pref, n_exp, n_nt, total, npass, KB);
    }
    int chunk = 0;
    while (cur.valid) {
#pragma unroll
      for (int d = 0; d < D; ++d) {
        if (cur.valid) {
          const int slot = chunk % kF8FacSlots;
          if (chunk >= kF8FacSlots) {
            F8_PROF_BEGIN();
            if (!mbar_wait_backoff(&fac_empty[slot], ((chunk / kF8FacSlots) - 1) & 1, spin)) {
              if (lane == 0) report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 760 + slot);
              spin = 1;
            }
            F8_PROF_END(6, lane == 0);
          }
          float* dst = fac + slot * (kF8FacBlocks * kF8Rows);
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const int tok = lane + 32 * r;
            dst[tok] = v[d][r].x * ws4[d].x;
            dst[kF8Rows + tok] = v[d][r].y * ws4[d].y;
            dst[2 * kF8Rows + tok] = v[d][r].z * ws4[d].z;
            dst[3 * kF8Rows + tok] = v[d][r].w * ws4[d].w;
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&fac_full[slot]);
          ++chunk;
          cur.next(p, pref, n_exp, n_nt, total, npass, KB);
          if (p.l2_prefetch && lane == 0) pre.prefetch_weights(p, &tm_pf, &tm_pfu);
          pre.load(p, KB, lane, v[d], ws4[d]);
          pre.next(p, pref, n_exp, n_nt, total, npass, KB);
        }
      }
    }
  } else {
    // =========================== epilogue ===========================================================
    const int q = warp & 3;                 // tensor-memory lane quarter this warp may read: tokens 32q .. 32q + 31
    const int part = (warp - 4) >> 2;       // feature columns 32 * part .. + 31 of the tile
    const int tok = 32 * q + lane;          // this thread's token row inside the tile
    uint32_t spin = spin_limit;
    bool failed = false;
    int blk = 0, chunk = 0;
    for (int w = blockIdx.x; w < total; w += gridDim.x) {
      const F8Item t = f8_item(p, pref, n_exp, w, n_nt);
      const bool quarter_live = 32 * q < t.count;      // any token in this warp's lanes
      const bool live = tok < t.count;
      const int n_first = t.n0 + 32 * part;            // first of this thread's 32 output features
      uint64_t acc2[16];                               // 32 running sums as packed pairs
#pragma unroll
      for (int j = 0; j < 16; ++j) acc2[j] = 0ull;
      for (int pass = 0; pass < npass; ++pass) {
        for (int kb = 0; kb < KB; ++kb, ++blk) {
          const int slot = chunk % kF8FacSlots;
          if ((kb & (kF8FacBlocks - 1)) == 0) {
            F8_PROF_BEGIN();
            if (!mbar_wait(&fac_full[slot], (chunk / kF8FacSlots) & 1, spin)) {
              if (lane == 0) report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 740 + slot);
              spin = 1;
              failed = true;
            }
            F8_PROF_END(4, tid == 128);
          }
          const int buf = blk % kF8AccBufs;
          {
            F8_PROF_BEGIN();
            if (!mbar_wait(&acc_full[buf], (blk / kF8AccBufs) & 1, spin)) {
              if (lane == 0) report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 750 + buf);
              spin = 1;
              failed = true;
            }
            F8_PROF_END(5, tid == 128);
          }
          if (!failed && quarter_live) {
            f8_fence_after();
            uint32_t c[32];
            F8_PROF_BEGIN();
            f8_tmem_ld32(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(buf * 128 + 32 * part), c);
            const float f = fac[slot * (kF8FacBlocks * kF8Rows) + (kb & (kF8FacBlocks - 1)) * kF8Rows + tok];
            const uint64_t f2 = f8_pack2(__float_as_uint(f), __float_as_uint(f));
            f8_tmem_ld_wait();
            F8_PROF_END(10, tid == 128);
            f8_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);     // the buffer may be overwritten: values are in registers
#pragma unroll
            for (int j = 0; j < 16; ++j) acc2[j] = f8_fma2(f8_pack2(c[2 * j], c[2 * j + 1]), f2, acc2[j]);
            F8_PROF_END(11, tid == 128);
          } else {
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
          }
          if ((kb & (kF8FacBlocks - 1)) == kF8FacBlocks - 1) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&fac_empty[slot]);
            ++chunk;
          }
        }
        // ---- end of a pass over K: this thread holds its token's 32 features of the tile -------------------
        F8_PROF_BEGIN();
        float acc[32];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          f8_unpack2(acc2[j], acc[2 * j], acc[2 * j + 1]);
          acc2[j] = 0ull;
        }
        const void* bias_p = pass == 0 ? p.bias : p.bias_up;
        if (bias_p != nullptr) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            acc[j] += load_as_float(bias_p, p.bias_dtype, (int64_t)t.expert * p.n + n_first + j);
        }
        if (npass == 2) {
          // gate and up are rounded to f16 where a 16-bit pipeline would store them; the activated value is
          // rounded once more before the quantizer sees it.  Each thread parks its own 32 gate values (64 bytes).
          uint4* park = reinterpret_cast<uint4*>(gate_park + (tok * 128 + 32 * part) * 2);
          if (pass == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              park[i] = make_uint4(pack_half2(acc[8 * i], acc[8 * i + 1]), pack_half2(acc[8 * i + 2], acc[8 * i + 3]),
                                   pack_half2(acc[8 * i + 4], acc[8 * i + 5]), pack_half2(acc[8 * i + 6], acc[8 * i + 7]));
          } else {
            float m = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint4 raw = park[i];
              const __half2* g2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 g = __half22float2(g2[j]);
                const float u0 = __half2float(__float2half_rn(acc[8 * i + 2 * j]));
                const float u1 = __half2float(__float2half_rn(acc[8 * i + 2 * j + 1]));
                const float a0 = __half2float(__float2half_rn(f8_gated(g.x, u0, p.act)));
                const float a1 = __half2float(__float2half_rn(f8_gated(g.y, u1, p.act)));
                acc[8 * i + 2 * j] = a0;
                acc[8 * i + 2 * j + 1] = a1;
                m = fmaxf(m, fmaxf(fabsf(a0), fabsf(a1)));
              }
            }
            // the token's 128 values are spread over the four warps of this lane quarter
            row_max[part * kF8Rows + tok] = m;
            named_bar_sync(2 + q, 128);
            m = fmaxf(fmaxf(row_max[tok], row_max[kF8Rows + tok]),
                      fmaxf(row_max[2 * kF8Rows + tok], row_max[3 * kF8Rows + tok]));
            if (live && !failed) {
              const float scale = m > 0.f ? __fdiv_rn(m, 448.f) : 1e-12f;
              const int64_t orow = t.row_start + tok;
              uint4* dst = reinterpret_cast<uint4*>(p.hq + orow * p.n + n_first);
#pragma unroll
              for (int i = 0; i < 2; ++i) {
                uint32_t wds[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  uint32_t pk = 0;
#pragma unroll
                  for (int b = 0; b < 4; ++b) {
                    const float qv = fminf(fmaxf(__fdiv_rn(acc[16 * i + 4 * j + b], scale), -448.f), 448.f);
                    pk |= (uint32_t)__nv_cvt_float_to_fp8(qv, __NV_SATFINITE, __NV_E4M3) << (8 * b);
                  }
                  wds[j] = pk;
                }
                dst[i] = make_uint4(wds[0], wds[1], wds[2], wds[3]);
              }
              if (part == 0) p.hs[orow * (p.n / 128) + t.n0 / 128] = scale;
            }
            named_bar_sync(2 + q, 128);     // row_max may be written again
          }
        } else if (live && !failed) {
          const int sp = t.row_start + tok;
          const int64_t orow = p.y_rows != nullptr ? (int64_t)__ldg(p.y_rows + sp) : (int64_t)sp;
          if (p.y_dtype == HQ_DT_F32) {
            float* dst = reinterpret_cast<float*>(p.y) + orow * p.y_stride + n_first;
            if (p.y_vec_ok) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                reinterpret_cast<float4*>(dst)[i] = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) dst[j] = acc[j];
            }
          } else {
            uint32_t wds[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (p.y_dtype == HQ_DT_F16) {
                wds[j] = pack_half2(acc[2 * j], acc[2 * j + 1]);
              } else {
                __nv_bfloat162 b = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
                wds[j] = *reinterpret_cast<uint32_t*>(&b);
              }
            }
            uint16_t* dst = reinterpret_cast<uint16_t*>(p.y) + orow * p.y_stride + n_first;
            if (p.y_vec_ok) {
#pragma unroll
              for (int i = 0; i < 4; ++i)
                reinterpret_cast<uint4*>(dst)[i] = make_uint4(wds[4 * i], wds[4 * i + 1], wds[4 * i + 2], wds[4 * i + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                dst[2 * j] = (uint16_t)(wds[j] & 0xFFFFu);
                dst[2 * j + 1] = (uint16_t)(wds[j] >> 16);
              }
            }
          }
        }
        F8_PROF_END(12, tid == 128);
      }
    }
  }

  f8_fence_before();
  __syncthreads();
#ifdef HQ_F8_PROFILE
  if (tid == 0) {
    atomicAdd(&g_f8_prof[8], (unsigned long long)(clock64() - prof_kernel_t0));
    unsigned long long nb = 0;
    for (int w = blockIdx.x; w < total; w += gridDim.x) nb += (unsigned long long)(npass * KB);
    atomicAdd(&g_f8_prof[9], nb);
  }
#endif
  if (warp == 1) {
    f8_fence_after();
    f8_tmem_dealloc(tmem_base, kF8TmemCols);
  }
}

#ifdef HQ_F8_PROFILE
extern "C" int32_t hq_debug_f8_prof(unsigned long long* out_host, int32_t reset) {
  if (cudaMemcpyFromSymbol(out_host, g_f8_prof, sizeof(g_f8_prof)) != cudaSuccess) return HQ_ERR_CUDA;
  if (reset) {
    unsigned long long z[16] = {};
    if (cudaMemcpyToSymbol(g_f8_prof, z, sizeof(z)) != cudaSuccess) return HQ_ERR_CUDA;
  }
  return HQ_OK;
}
#endif

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
bool f8_encode_2d(CUtensorMap* map, CUtensorMapDataType type, const void* base, uint64_t inner, uint64_t rows,
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
  CUtensorMap tm_w, tm_wu, tm_x[4], tm_pf, tm_pfu;
  const uint64_t wrows = (uint64_t)(p.expert_bounds != nullptr ? p.n_experts : 1) * p.n;
  if (!f8_encode_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.w, (uint64_t)p.k, wrows, (uint64_t)p.k, 128, 128,
                    CU_TENSOR_MAP_SWIZZLE_128B))
    return HQ_ERR_CUDA;
  tm_wu = tm_w;
  if (p.w_up != nullptr && !f8_encode_2d(&tm_wu, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.w_up, (uint64_t)p.k, wrows,
                                         (uint64_t)p.k, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B))
    return HQ_ERR_CUDA;
  // prefetch maps: the same banks as 32-bit words, 1 KiB x 128 rows per box (K % 512 == 0: the last box of a row
  // is cut by the tensor bound)
  if (!f8_encode_2d(&tm_pf, CU_TENSOR_MAP_DATA_TYPE_UINT32, p.w, (uint64_t)p.k / 4, wrows, (uint64_t)p.k, 256, 128,
                    CU_TENSOR_MAP_SWIZZLE_NONE))
    return HQ_ERR_CUDA;
  tm_pfu = tm_pf;
  if (p.w_up != nullptr && !f8_encode_2d(&tm_pfu, CU_TENSOR_MAP_DATA_TYPE_UINT32, p.w_up, (uint64_t)p.k / 4, wrows,
                                         (uint64_t)p.k, 256, 128, CU_TENSOR_MAP_SWIZZLE_NONE))
    return HQ_ERR_CUDA;
  for (int i = 0; i < 4; ++i)
    if (!f8_encode_2d(&tm_x[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, p.xq, (uint64_t)p.k, (uint64_t)p.n_rows, (uint64_t)p.k,
                      128, 32u * (uint32_t)(i + 1), CU_TENSOR_MAP_SWIZZLE_128B))
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
  const int64_t max_tiles = p.n_rows / kF8Rows + n_exp;
  const int64_t items = max_tiles * (p.n / 128);
  const int64_t grid = items < sms ? items : sms;
  // a thread writes its token's 32 features as 16-byte stores when every row segment is 16-byte aligned
  p.y_vec_ok = p.y != nullptr && (reinterpret_cast<uintptr_t>(p.y) & 15u) == 0 &&
               (p.y_stride * dtype_size(p.y_dtype)) % 16 == 0;
  if (p.spin_limit == 0) p.spin_limit = 1u << 22;
  if (p.load_burst != 1 && p.load_burst != 2 && p.load_burst != 4) p.load_burst = 2;
  p.l2_prefetch = p.load_burst_prefetch_off ? 0 : 1;
  fp8_grouped_kernel<<<(unsigned)grid, kF8Threads, F8Smem::TOTAL, stream>>>(tm_w, tm_wu, tm_x[0], tm_x[1], tm_x[2],
                                                                            tm_x[3], tm_pf, tm_pfu, p);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

}  // namespace hq
