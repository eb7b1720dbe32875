// MXFP4 expert GEMM on the block-scaled tensor-core path: tcgen05.mma kind::mxf8f6f4 with .block_scale.
//
// y[row, n] = sum over 32-element blocks b of  2^(sx[row, b] - 127) * 2^(sw[expert, n, b] - 127) *
//             sum_{k in b} e4m3(X[row, k]) * e2m1(W[expert, n, k])
// W: MXFP4Layer's bytes as they are (hanzo-quant/src/mxfp4/mod.rs:29-41: blocks [E, N, K/2], low nibble = even k;
// scales [E, N, K/32] e8m0) -- the nibbles are never expanded: TMA copies them with the 16-packed-4-bit tensor-map
// type, which spreads every 8 bytes of nibbles over a 16-byte slot of shared memory, the form the MMA reads for a
// 4-bit operand.  X: activation rows quantized to MXFP8 (e4m3 codes + one e8m0 scale per 32 elements), already in
// expert-sorted order.  The e8m0 scale factors of both operands sit in tensor memory and are applied by the MMA
// per 32-element block, so the f32 accumulator in tensor memory runs over the whole K and is drained once per tile.
//
// Orientation: tensor-memory lanes = tokens (MMA M = 128, A = the token tile), columns = output features (MMA
// N = 128, B = the weight tile).  Where the scale factors have to be (found by a probe on this part, one MMA with
// distinct values in every cell): for row r of A, lane r, column sfa + r / 32, byte a_sf_id; for column n of B,
// column sfb + n / 32, lane n % 32 of EVERY lane quarter (each quarter reads its own copy), byte b_sf_id.  The four
// "scale" warps (one per lane quarter) write them from registers with tcgen05.st: one word per token (its four
// blocks of the 128-wide K stage) and four words per lane for the 128 features.
//
// Work item = (token tile of <= 128 rows of one expert, 128 weight rows); token tiles are cut inside the kernel
// from expert_bounds.  Epilogues: plain (bias, rows out in f32 / f16 / bf16) or gated for interleaved gate/up rows
// (gpt-oss: row 2i = gate_i, 2i + 1 = up_i): bias, activation, then the MXFP8 quantizer of the 64 results per
// thread (two 32-element blocks), written as codes + scales for the down projection.
//
// Roles (one persistent CTA per SM, 16 warps): warp 0 issues TMA, warp 1 issues the MMAs (one lane; the stages of a
// tile accumulate into one buffer, so they must be issued in order), warps 4-7 write scale factors, warps 8-15
// drain finished tiles, two per lane quarter with 64 columns each (two accumulator buffers, so a drain overlaps the
// next tile's MMAs).  Every wait is
// bounded; after a time-out the remaining waits poll once, nothing more is multiplied or stored and the kernel
// reaches its normal exit.  No multicast, no peer memory.
#include <cuda.h>
#include <cuda_fp8.h>

#include "hq_common.cuh"
#include "hq_kernels.h"

namespace hq {

bool f8_encode_2d(CUtensorMap* map, CUtensorMapDataType type, const void* base, uint64_t inner, uint64_t rows,
                  uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle swz);

// Developer instrumentation, compiled out unless HQ_MX_PROFILE is defined: cycles each role spends in its waits,
// summed over CTAs into g_mx_prof (read back with hq_debug_mx_prof).
#ifdef HQ_MX_PROFILE
__device__ unsigned long long g_mx_prof[16];
#define MX_PROF_BEGIN() const long long prof_t0__ = clock64()
#define MX_PROF_END(idx, cond) do { if (cond) atomicAdd(&g_mx_prof[idx], (unsigned long long)(clock64() - prof_t0__)); } while (0)
#else
#define MX_PROF_BEGIN() do {} while (0)
#define MX_PROF_END(idx, cond) do {} while (0)
#endif

constexpr int kMxThreads = 512;
constexpr int kMxEpiWarps = 8;                           // two per lane quarter, 64 columns each
constexpr int kMxMaxStages = 6;                          // shared-memory stages (fewer when K is large, see below)
constexpr int kMxTile = 128 * 128;                       // one operand box in shared memory: 128 rows x 128 bytes
constexpr int kMxStageBytes = 2 * kMxTile;
constexpr int kMxAccBufs = 2;
constexpr int kMxSfBase = 256;                           // tensor-memory column of the first scale-factor slot
constexpr int kMxTmemCols = 512;                         // (one slot of 8 columns per stage)
constexpr int kMxMaxExperts = 1024;
constexpr int kMxSmemLimit = 227 * 1024;

// Shared memory, in order: the stages; four strips for the e8m0 scale bytes of a work item (token rows and weight
// rows, two items in rotation; a strip holds the item's 128 rows x K/32 bytes as they lie in memory, starting at
// the 16-byte boundary below the first byte); the tile prefix; the epilogue warps' bias strips; the barriers.
struct MxSmem {
  static constexpr int PREF_BYTES = (kMxMaxExperts + 1) * 4 + 12;
  static constexpr int BIAS_BYTES = kMxEpiWarps * 64 * 4;
  static constexpr int N_BAR = 3 * kMxMaxStages + 2 * kMxAccBufs + 4;
  static constexpr int FIXED = PREF_BYTES + BIAS_BYTES + N_BAR * 8 + 16 + 1024;
  __host__ __device__ static int strip(int k) { return (128 * (k / 32) + 32 + 15) & ~15; }
  __host__ __device__ static int stages(int k) {
    const int s = (kMxSmemLimit - FIXED - 4 * strip(k)) / kMxStageBytes;
    return s > kMxMaxStages ? kMxMaxStages : s;
  }
  __host__ __device__ static int total(int k) { return FIXED + 4 * strip(k) + stages(k) * kMxStageBytes; }
};
static_assert(MxSmem::PREF_BYTES % 16 == 0, "the strips behind the prefix stay 16-byte aligned");

__device__ __forceinline__ void mx_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void mx_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void mx_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mx_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa,
                                       uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %6, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mx_tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
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

// K-major operand tile of 128-byte rows, 128-byte swizzle, 8-row groups 1024 bytes apart, descriptor version 1
__device__ __forceinline__ uint64_t mx_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFFu);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Block-scaled instruction descriptor: b_sf_id [4,6), a format [7,10) = e4m3 (0), b format [10,13) = e2m1 (5),
// N >> 3 [17,23), scale format ue8m0 [23], M >> 4 [24,29), a_sf_id [29,31); both operands K-major, f32 accumulate.
__device__ __forceinline__ uint32_t mx_idesc(int sf_id) {
  return ((uint32_t)sf_id << 4) | (0u << 7) | (5u << 10) | ((uint32_t)(128 >> 3) << 17) | (1u << 23) |
         ((uint32_t)(128 >> 4) << 24) | ((uint32_t)sf_id << 29);
}

__device__ __forceinline__ void mx_tma_2d(void* dst_smem, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
          "r"(smem_u32(dst_smem)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

// four consecutive scale bytes (shared memory, 2-byte aligned) as one word; `have` of them exist (2 or 4), the rest
// read as 127 (2^0) -- they belong to K blocks whose products are never issued
__device__ __forceinline__ uint32_t mx_scale_word(const uint8_t* p, int have) {
  const uint32_t lo = *reinterpret_cast<const uint16_t*>(p);
  const uint32_t hi = have > 2 ? (uint32_t) * reinterpret_cast<const uint16_t*>(p + 2) : 0x7F7Fu;
  return lo | (hi << 16);
}

// [lo, hi): the whole 16-byte units that cover the byte range [b0, b1) of a tensor of `size` bytes without reaching
// past its end (hi is cut back to the last whole unit inside the tensor; the bytes behind it are copied by hand)
struct MxRange {
  int64_t lo, hi;
};
__device__ __forceinline__ MxRange mx_range(int64_t b0, int64_t b1, int64_t size) {
  MxRange r;
  r.lo = b0 & ~(int64_t)15;
  r.hi = min((b1 + 15) & ~(int64_t)15, size & ~(int64_t)15);
  if (r.hi < r.lo) r.hi = r.lo;
  return r;
}

__device__ __forceinline__ float mx_gated(float g, float u, const hq_act_args& a) {
  if (a.act == HQ_ACT_GPTOSS) {
    g = fminf(g, a.limit);
    u = fminf(fmaxf(u, -a.limit), a.limit);
    return (u + 1.f) * __fdividef(g, 1.f + __expf(-a.alpha * g));
  }
  if (a.has_limit) {
    g = fminf(g, a.limit);
    u = fminf(fmaxf(u, -a.limit), a.limit);
  }
  return __fdividef(g, 1.f + __expf(-g)) * u;
}

// MXFP8 (OCP microscaling, e4m3 elements): shared exponent = floor(log2(amax)) - 8 (e4m3's largest power of two is
// 2^8), stored biased by 127 and kept inside 0..254; an all-zero block gets 127.  Elements are scaled by 2^-e and
// converted with saturation at +-448.
__device__ __forceinline__ int mx_shared_exp(float amax) {
  if (!(amax > 0.f)) return 127;
  const int e = (int)((__float_as_uint(amax) >> 23) & 0xFFu) - 127;      // floor(log2) of a normal number
  return min(max(e - 8 + 127, 0), 254);
}
__device__ __forceinline__ float mx_exp_to_inv_scale(int e) {              // 2^-(e - 127), e in 0..254
  return __uint_as_float((uint32_t)(254 - e) << 23);
}

struct MxItem {
  int expert, row_start, count, n0;
};
__device__ __forceinline__ MxItem mx_item(const MxGroupedParams& p, const int32_t* pref, int n_exp, int w, int n_nt) {
  MxItem t;
  const int tt = w / n_nt;
  t.n0 = (w - tt * n_nt) * 128;
  int lo = 0, hi = n_exp - 1;
  while (lo < hi) {
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
  t.row_start = base + j * 128;
  t.count = min(128, cnt - j * 128);
  return t;
}

__global__ void __launch_bounds__(kMxThreads, 1)
mx_grouped_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_wtail,
                  const __grid_constant__ CUtensorMap tm_x, const MxGroupedParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int NS = MxSmem::stages(p.k);
  const int strip = MxSmem::strip(p.k);
  uint8_t* sc = smem + NS * kMxStageBytes;          // scale strips: [item parity][token rows | weight rows]
  int32_t* pref = reinterpret_cast<int32_t*>(sc + 4 * strip);
  float* bias_sm = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(pref) + MxSmem::PREF_BYTES);
  uint64_t* full = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(bias_sm) + MxSmem::BIAS_BYTES);
  uint64_t* empty = full + kMxMaxStages;
  uint64_t* sf_full = empty + kMxMaxStages;         // the stage's scale factors are in tensor memory (`empty` also
                                                    // says that the MMAs which read them are done)
  uint64_t* acc_full = sf_full + kMxMaxStages;      // [2] a tile's accumulation is complete
  uint64_t* acc_empty = acc_full + kMxAccBufs;      // [2] ... and has been drained
  uint64_t* sc_full = acc_empty + kMxAccBufs;       // [2] an item's scale bytes are in their strips
  uint64_t* sc_empty = sc_full + 2;                 // [2] ... and the scale warps are done with them
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sc_empty + 2);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_nt = (p.n + 127) / 128;
  const int KS = (p.k + 127) / 128;                 // K stages; the last one may hold 32, 64 or 96 elements
  const int k_tail = p.k - (KS - 1) * 128;          // elements of the last stage (32 .. 128)
  const int n_exp = p.expert_bounds != nullptr ? p.n_experts : 1;
  const int sb = p.k / 32;                          // scale bytes per row
#ifdef HQ_MX_PROFILE
  const long long prof_kernel_t0 = clock64();
#endif

  for (int e = tid; e < n_exp; e += kMxThreads) {
    const int cnt = p.expert_bounds != nullptr ? __ldg(p.expert_bounds + e + 1) - __ldg(p.expert_bounds + e) : p.m;
    pref[e + 1] = (cnt + 127) / 128;
  }
  if (tid == 0) {
    pref[0] = 0;
    for (int s = 0; s < kMxMaxStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
      mbar_init(&sf_full[s], 4);
    }
    for (int b = 0; b < kMxAccBufs; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], kMxEpiWarps);
      mbar_init(&sc_full[b], 1);
      mbar_init(&sc_empty[b], 4);
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
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(kMxTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  mx_fence_before();
  __syncthreads();
  mx_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total = pref[n_exp] * n_nt;
  const uint32_t spin_limit = p.spin_limit;

  if (warp == 0) {
    // =========================== TMA issuer =========================================================
    if (lane == 0 && p.test_skip_producer != 1) {
      int s = 0, round = 0;
      int issued = 0;              // stages handed to the copy engine so far
      int itemc = 0;               // items so far (scale strips of parity itemc & 1)
      bool stop = false;           // a wait ran out: nothing more is issued (the target may still be in use)
      const int64_t xs_bytes = p.n_rows * sb, ws_bytes = (int64_t)n_exp * p.n * sb;
      for (int w = blockIdx.x; w < total && !stop; w += gridDim.x, ++itemc) {
        const MxItem t = mx_item(p, pref, n_exp, w, n_nt);
        const int wrow = t.expert * p.n + t.n0;
        // ---- the item's scale bytes: two contiguous byte ranges, copied in whole 16-byte units ----
        {
          const int par = itemc & 1;
          if (itemc >= 2 && !mbar_wait(&sc_empty[par], ((itemc >> 1) - 1) & 1, spin_limit)) {
            report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 880 + par);
            stop = true;
            break;
          }
          uint8_t* da = sc + (2 * par) * strip;
          uint8_t* db = da + strip;
          const int64_t a0 = (int64_t)t.row_start * sb, a1 = a0 + (int64_t)t.count * sb;
          const int64_t b0 = (int64_t)wrow * sb, b1 = b0 + (int64_t)min(128, p.n - t.n0) * sb;
          const MxRange ra = mx_range(a0, a1, xs_bytes), rb = mx_range(b0, b1, ws_bytes);
          // the last bytes of a tensor whose size is not a multiple of 16 are copied by hand (at most 15)
          for (int64_t b = max(ra.hi, a0); b < a1; ++b) da[b - ra.lo] = p.xs[b];
          for (int64_t b = max(rb.hi, b0); b < b1; ++b) db[b - rb.lo] = p.w_scales[b];
          mbar_arrive_expect_tx(&sc_full[par], (uint32_t)((ra.hi - ra.lo) + (rb.hi - rb.lo)));
          if (ra.hi > ra.lo) bulk_g2s(da, p.xs + ra.lo, (uint32_t)(ra.hi - ra.lo), &sc_full[par]);
          if (rb.hi > rb.lo) bulk_g2s(db, p.w_scales + rb.lo, (uint32_t)(rb.hi - rb.lo), &sc_full[par]);
        }
        for (int ks = 0; ks < KS; ++ks) {
          {
            MX_PROF_BEGIN();
            if (round > 0 && !mbar_wait(&empty[s], (round - 1) & 1, spin_limit)) {
              report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 810 + s);
              stop = true;
              break;
            }
            MX_PROF_END(0, true);
          }
          uint8_t* stage = smem + s * kMxStageBytes;
          // the copy engine reports the bytes it read: the packed nibbles (half a byte per element), not the
          // 16-byte slots they are spread over in shared memory
          mbar_arrive_expect_tx(&full[s], (uint32_t)(kMxTile + kMxTile / 2));
          mx_tma_2d(stage, &tm_x, ks * 128, t.row_start, &full[s]);
          // a K that is not a multiple of 128 ends in a stage of its own tensor map (the packed 4-bit map type
          // needs a row length that is a multiple of 128 elements)
          if (ks == KS - 1 && k_tail != 128) mx_tma_2d(stage + kMxTile, &tm_wtail, 0, wrow, &full[s]);
          else mx_tma_2d(stage + kMxTile, &tm_w, ks * 128, wrow, &full[s]);
          ++issued;
          if (++s == NS) {
            s = 0;
            ++round;
          }
        }
      }
      // no copy may still be writing this CTA's shared memory when it exits: wait (bounded) for the last copies of
      // every stage and strip.  On the normal path they were consumed long ago and these waits return at once.
      for (int j = 0; j < NS && j < issued; ++j) {
        const int idx = issued - 1 - j;
        if (!mbar_wait(&full[idx % NS], (idx / NS) & 1, spin_limit)) break;
      }
      for (int j = 0; j < 2 && j < itemc; ++j) {
        const int idx = itemc - 1 - j;
        if (!mbar_wait(&sc_full[idx & 1], (idx >> 1) & 1, spin_limit)) break;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // =========================== MMA issuer =========================================================
    if (lane == 0) {
      uint32_t spin = spin_limit;
      bool failed = false;
      int s = 0, round = 0;        // shared-memory stage (= scale-factor slot) and how often the ring has wrapped
      int tile = 0;
      for (int w = blockIdx.x; w < total; w += gridDim.x, ++tile) {
        const int buf = tile & 1;
        if (tile >= kMxAccBufs) {
          MX_PROF_BEGIN();
          if (!mbar_wait(&acc_empty[buf], ((tile >> 1) - 1) & 1, spin)) {
            report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 820 + buf);
            spin = 1;
            failed = true;
          }
          MX_PROF_END(1, true);
        }
        const uint32_t d = tmem_base + (uint32_t)(buf * 128);
        for (int ks = 0; ks < KS; ++ks, s = (s + 1 == NS ? 0 : s + 1), round += (s == 0)) {
          const int slot = s;
          {
            MX_PROF_BEGIN();
            if (!mbar_wait(&full[s], round & 1, spin)) {
              report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 830 + s);
              spin = 1;
              failed = true;
            }
            MX_PROF_END(2, true);
          }
          {
            MX_PROF_BEGIN();
            if (!mbar_wait(&sf_full[slot], round & 1, spin)) {
              report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 840 + slot);
              spin = 1;
              failed = true;
            }
            MX_PROF_END(3, true);
          }
          if (failed) continue;
          MX_PROF_BEGIN();
          mx_fence_after();
          const uint32_t stage = smem_u32(smem + s * kMxStageBytes);
          const uint64_t adesc = mx_smem_desc(stage), bdesc = mx_smem_desc(stage + kMxTile);
          const uint32_t sfa = tmem_base + (uint32_t)(kMxSfBase + 8 * slot), sfb = sfa + 4;
          const int n_mma = (ks == KS - 1) ? k_tail / 32 : 4;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            if (kk < n_mma) mx_mma(d, adesc + 2 * kk, bdesc + 2 * kk, mx_idesc(kk), sfa, sfb, (ks | kk) != 0 ? 1u : 0u);
          mx_commit(&empty[s]);
          if (ks == KS - 1) mx_commit(&acc_full[buf]);
          MX_PROF_END(4, true);
        }
      }
    }
    __syncwarp();
  } else if (warp >= 4 && warp < 8) {
    // =========================== scale factors ======================================================
    // Per K stage and lane quarter q: one word for this thread's token (its four e8m0 bytes of the stage) into
    // column sfa + q, four words for the features 32 j + lane into columns sfb + j.  The bytes come from the
    // item's strips in shared memory (the copy warp fetched them one item ahead).
    const int q = warp - 4;
    const int tok = 32 * q + lane;
    uint32_t spin = spin_limit;
    bool failed = false;
    int s = 0, round = 0, itemc = 0;
    for (int w = blockIdx.x; w < total; w += gridDim.x, ++itemc) {
      const MxItem t = mx_item(p, pref, n_exp, w, n_nt);
      const int par = itemc & 1;
      if (!mbar_wait(&sc_full[par], (itemc >> 1) & 1, spin)) {
        if (lane == 0) report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 870 + par);
        spin = 1;
        failed = true;
      }
      const uint8_t* sa = sc + (2 * par) * strip + (int)(((int64_t)t.row_start * sb) & 15) + tok * sb;
      const uint8_t* sw = sc + (2 * par + 1) * strip + (int)((((int64_t)t.expert * p.n + t.n0) * sb) & 15) + lane * sb;
      const bool a_live = tok < t.count && !failed;
      bool b_live[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) b_live[j] = t.n0 + 32 * j + lane < p.n && !failed;
      for (int ks = 0; ks < KS; ++ks) {
        if (round > 0) {
          MX_PROF_BEGIN();
          if (!mbar_wait(&empty[s], (round - 1) & 1, spin)) {
            if (lane == 0) report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 850 + s);
            spin = 1;
            failed = true;
          }
          MX_PROF_END(5, q == 0 && lane == 0);
        }
        mx_fence_after();
        MX_PROF_BEGIN();
        const int have = (ks == KS - 1) ? k_tail / 32 : 4;
        const uint32_t wa = a_live ? mx_scale_word(sa + 4 * ks, have) : 0x7F7F7F7Fu;
        uint32_t wb[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) wb[j] = b_live[j] ? mx_scale_word(sw + 32 * j * sb + 4 * ks, have) : 0x7F7F7F7Fu;
        const uint32_t base = tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(kMxSfBase + 8 * s);
        asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(base + q), "r"(wa) : "memory");
        asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(base + 4), "r"(wb[0]),
                     "r"(wb[1]), "r"(wb[2]), "r"(wb[3])
                     : "memory");
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        mx_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sf_full[s]);
        MX_PROF_END(6, q == 0 && lane == 0);
        if (++s == NS) {
          s = 0;
          ++round;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sc_empty[par]);
    }
  } else if (warp >= 8) {
    // =========================== epilogue ===========================================================
    // Two warps per lane quarter; each owns 64 of the tile's 128 columns.  The 64 bias values of those columns are
    // staged in a strip of shared memory of the warp's own (no barrier with the other warps).
    const int q = warp & 3;                  // lane quarter: tokens 32q .. 32q + 31
    const int half = (warp - 8) >> 2;        // columns 64 half .. 64 half + 63 of the tile
    const int tok = 32 * q + lane;
    float* bsm = bias_sm + (warp - 8) * 64;
    uint32_t spin = spin_limit;
    bool failed = false;
    const bool gated = p.act.act != HQ_ACT_NONE;
    const bool has_bias = p.bias != nullptr;
    int tile = 0;
    for (int w = blockIdx.x; w < total; w += gridDim.x, ++tile) {
      const MxItem t = mx_item(p, pref, n_exp, w, n_nt);
      const int buf = tile & 1;
      const int n_first = t.n0 + 64 * half;
      const bool cols_live = n_first < p.n;
      if (has_bias && cols_live) {
        const int64_t b0 = (int64_t)t.expert * p.n + n_first;
        bsm[lane] = n_first + lane < p.n ? load_as_float(p.bias, p.bias_dtype, b0 + lane) : 0.f;
        bsm[lane + 32] = n_first + lane + 32 < p.n ? load_as_float(p.bias, p.bias_dtype, b0 + lane + 32) : 0.f;
      }
      __syncwarp();
      {
        MX_PROF_BEGIN();
        if (!mbar_wait(&acc_full[buf], (tile >> 1) & 1, spin)) {
          if (lane == 0) report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 860 + buf);
          spin = 1;
          failed = true;
        }
        MX_PROF_END(7, warp == 8 && lane == 0);
      }
      mx_fence_after();
      MX_PROF_BEGIN();
      const bool live = tok < t.count && !failed;
      const int64_t srow = t.row_start + tok;
      if (cols_live && 32 * q < t.count && !failed) {
        uint32_t c[64];
        const uint32_t taddr = tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(buf * 128 + 64 * half);
        mx_tmem_ld32(taddr, *reinterpret_cast<uint32_t(*)[32]>(&c[0]));
        mx_tmem_ld32(taddr + 32, *reinterpret_cast<uint32_t(*)[32]>(&c[32]));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (has_bias) {
#pragma unroll
          for (int j = 0; j < 64; j += 4) {
            const float4 b = *reinterpret_cast<const float4*>(bsm + j);
            c[j] = __float_as_uint(__uint_as_float(c[j]) + b.x);
            c[j + 1] = __float_as_uint(__uint_as_float(c[j + 1]) + b.y);
            c[j + 2] = __float_as_uint(__uint_as_float(c[j + 2]) + b.z);
            c[j + 3] = __float_as_uint(__uint_as_float(c[j + 3]) + b.w);
          }
        }
        if (live && gated) {
          // interleaved rows: columns 2i / 2i + 1 are gate_i / up_i, so 64 columns give 32 results = one MXFP8 block
          float m = 0.f;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float a = mx_gated(__uint_as_float(c[2 * j]), __uint_as_float(c[2 * j + 1]), p.act);
            c[j] = __float_as_uint(a);
            m = fmaxf(m, fabsf(a));
          }
          const int i_first = n_first / 2;               // first intermediate feature of these 32 results
          if (p.hq == nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (i_first + j < p.h_width)
                store_from_float(p.y, p.y_dtype, srow * p.y_stride + i_first + j, __uint_as_float(c[j]));
          } else {
            const int e = mx_shared_exp(m);
            const float inv = mx_exp_to_inv_scale(e);
            uint32_t wds[8];
#pragma unroll
            for (int g4 = 0; g4 < 8; ++g4) {
              const uint32_t lo = __nv_cvt_float2_to_fp8x2(
                  make_float2(__uint_as_float(c[4 * g4]) * inv, __uint_as_float(c[4 * g4 + 1]) * inv), __NV_SATFINITE,
                  __NV_E4M3);
              const uint32_t hi = __nv_cvt_float2_to_fp8x2(
                  make_float2(__uint_as_float(c[4 * g4 + 2]) * inv, __uint_as_float(c[4 * g4 + 3]) * inv),
                  __NV_SATFINITE, __NV_E4M3);
              wds[g4] = lo | (hi << 16);
            }
            uint4* dst = reinterpret_cast<uint4*>(p.hq + srow * p.h_width + i_first);
            dst[0] = make_uint4(wds[0], wds[1], wds[2], wds[3]);
            dst[1] = make_uint4(wds[4], wds[5], wds[6], wds[7]);
            p.hs[srow * (p.h_width / 32) + i_first / 32] = (uint8_t)e;
          }
        } else if (live) {
          const int64_t orow = p.y_rows != nullptr ? (int64_t)__ldg(p.y_rows + srow) : srow;
          if (p.y_vec_ok && n_first + 64 <= p.n) {
            // 64 consecutive values of one row: 128 (16-bit) or 256 (f32) contiguous bytes in 16-byte stores
            if (p.y_dtype == HQ_DT_F32) {
              float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.y) + orow * p.y_stride + n_first);
#pragma unroll
              for (int j = 0; j < 16; ++j)
                dst[j] = make_float4(__uint_as_float(c[4 * j]), __uint_as_float(c[4 * j + 1]),
                                     __uint_as_float(c[4 * j + 2]), __uint_as_float(c[4 * j + 3]));
            } else {
              uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.y) + orow * p.y_stride + n_first);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                uint32_t pk[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  const float lo = __uint_as_float(c[8 * j + 2 * u]), hi = __uint_as_float(c[8 * j + 2 * u + 1]);
                  if (p.y_dtype == HQ_DT_F16) {
                    const __half2 h2 = __floats2half2_rn(lo, hi);
                    pk[u] = *reinterpret_cast<const uint32_t*>(&h2);
                  } else {
                    const __nv_bfloat162 b2 = __floats2bfloat162_rn(lo, hi);
                    pk[u] = *reinterpret_cast<const uint32_t*>(&b2);
                  }
                }
                dst[j] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 64; ++j)
              if (n_first + j < p.n)
                store_from_float(p.y, p.y_dtype, orow * p.y_stride + n_first + j, __uint_as_float(c[j]));
          }
        }
      }
      mx_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
      MX_PROF_END(10, warp == 8 && lane == 0);
    }
  }

  mx_fence_before();
  __syncthreads();
#ifdef HQ_MX_PROFILE
  if (tid == 0) {
    atomicAdd(&g_mx_prof[8], (unsigned long long)(clock64() - prof_kernel_t0));
    unsigned long long nb = 0;
    for (int w = blockIdx.x; w < total; w += gridDim.x) nb += (unsigned long long)KS;
    atomicAdd(&g_mx_prof[9], nb);
  }
#endif
  if (warp == 1) {
    mx_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kMxTmemCols) : "memory");
  }
}

#ifdef HQ_MX_PROFILE
extern "C" int32_t hq_debug_mx_prof(unsigned long long* out_host, int32_t reset) {
  if (cudaMemcpyFromSymbol(out_host, g_mx_prof, sizeof(g_mx_prof)) != cudaSuccess) return HQ_ERR_CUDA;
  if (reset) {
    unsigned long long z[16] = {};
    if (cudaMemcpyToSymbol(g_mx_prof, z, sizeof(z)) != cudaSuccess) return HQ_ERR_CUDA;
  }
  return HQ_OK;
}
#endif

// ---- MXFP8 row quantizer: rows looked up through row_map (token order -> expert-sorted order) ---------------
// One warp per (row, 512-element span): a lane owns 8 consecutive elements in each half of the span (both loads
// issued before anything is used), a 32-element block is 4 lanes.
__device__ __forceinline__ void mx_load8(const void* x, int dtype, int64_t i, float (&v)[8]) {
  if (dtype == HQ_DT_F32) {
    const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + i);
    const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + i + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    const uint4 t = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(x) + i);
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (dtype == HQ_DT_BF16) {
        v[2 * j] = __uint_as_float(w[j] << 16);
        v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
      } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
        v[2 * j] = f.x;
        v[2 * j + 1] = f.y;
      }
    }
  }
}

__global__ void __launch_bounds__(256) mxfp8_quant_rows_kernel(const void* __restrict__ x, int dtype, int64_t x_stride,
                                                               const int32_t* __restrict__ row_map,
                                                               const int32_t* __restrict__ n_valid, int64_t n_rows,
                                                               int k, int vec_ok, uint8_t* __restrict__ codes,
                                                               uint8_t* __restrict__ scales) {
  const int spans = (k + 511) / 512;
  const int64_t item = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int64_t limit = n_valid != nullptr ? min((int64_t)*n_valid, n_rows) : n_rows;
  if (item >= limit * spans) return;
  const int lane = threadIdx.x & 31;
  const int64_t row = item / spans;
  const int span = (int)(item - row * spans);
  const int64_t src_row = row_map != nullptr ? (int64_t)row_map[row] : row;
  float v[2][8];
  bool in[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int c0 = span * 512 + j * 256 + lane * 8;
    in[j] = c0 < k;                                   // k is a multiple of 32, so a lane's 8 elements are all in or out
    if (in[j] && vec_ok) {
      mx_load8(x, dtype, src_row * x_stride + c0, v[j]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[j][i] = in[j] ? load_as_float(x, dtype, src_row * x_stride + c0 + i) : 0.f;
    }
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[j][i]));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
    if (!in[j]) continue;
    const int e = mx_shared_exp(m);
    const float inv = mx_exp_to_inv_scale(e);
    uint32_t packed[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[j][4 * h] * inv, v[j][4 * h + 1] * inv), __NV_SATFINITE,
                                                   __NV_E4M3);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[j][4 * h + 2] * inv, v[j][4 * h + 3] * inv),
                                                   __NV_SATFINITE, __NV_E4M3);
      packed[h] = lo | (hi << 16);
    }
    const int c0 = span * 512 + j * 256 + lane * 8;
    *reinterpret_cast<uint2*>(codes + row * k + c0) = make_uint2(packed[0], packed[1]);
    if ((lane & 3) == 0) scales[row * (k / 32) + c0 / 32] = (uint8_t)e;
  }
}

int32_t launch_mxfp8_quant_rows(const void* x, int x_dtype, int64_t x_stride, const int32_t* row_map,
                                const int32_t* n_valid, int64_t n_rows, int64_t k, uint8_t* codes, uint8_t* scales,
                                cudaStream_t stream) {
  const int64_t items = n_rows * ((k + 511) / 512);
  if (items == 0) return HQ_OK;
  // 16-byte loads need an aligned base and row pitch; otherwise elements are loaded one at a time
  const int esz = dtype_size(x_dtype);
  const int vec_ok = (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (x_stride * esz) % 16 == 0 ? 1 : 0;
  mxfp8_quant_rows_kernel<<<(unsigned)((items + 7) / 8), 256, 0, stream>>>(x, x_dtype, x_stride, row_map, n_valid,
                                                                           n_rows, (int)k, vec_ok, codes, scales);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

// K % 64 == 0: whole 32-element blocks, 32-byte row stride of the packed nibbles, 2-byte aligned scale rows
// ... and a K whose scale strips leave room for at least two stages
bool mx_grouped_supported(int64_t n, int64_t k) {
  return k % 64 == 0 && k >= 128 && n >= 1 && k <= 16384 && MxSmem::stages((int)k) >= 2;
}

int32_t launch_mx_grouped(const MxGroupedParams& p_in, cudaStream_t stream) {
  MxGroupedParams p = p_in;
  if (!mx_grouped_supported(p.n, p.k)) return HQ_ERR_SHAPE;
  if (p.expert_bounds != nullptr && p.n_experts > kMxMaxExperts) return HQ_ERR_SHAPE;
  if (p.n_rows <= 0) return HQ_OK;
  // the packed 4-bit tensor-map type wants a 32-byte aligned base and row stride
  if ((reinterpret_cast<uintptr_t>(p.w) & 31u) != 0) return HQ_ERR_ALIGN;
  CUtensorMap tm_w, tm_wtail, tm_x;
  const uint64_t wrows = (uint64_t)(p.expert_bounds != nullptr ? p.n_experts : 1) * p.n;
  const uint64_t k_main = (uint64_t)(p.k / 128) * 128;
  const uint64_t wstride = (uint64_t)p.k / 2;
  if (k_main > 0 && !f8_encode_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, p.w, k_main, wrows, wstride, 128, 128,
                                  CU_TENSOR_MAP_SWIZZLE_128B))
    return HQ_ERR_CUDA;
  tm_wtail = tm_w;
  if (k_main != (uint64_t)p.k) {
    // the last 32 / 64 / 96 elements of every row: a map of its own whose rows are 128 elements long; what it
    // reads past the row's end meets zero activations (the bank needs 64 readable bytes after its last row)
    const uint8_t* tail = reinterpret_cast<const uint8_t*>(p.w) + k_main / 2;
    if (!f8_encode_2d(&tm_wtail, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, tail, 128, wrows, wstride, 128, 128,
                      CU_TENSOR_MAP_SWIZZLE_128B))
      return HQ_ERR_CUDA;
  }
  if (!f8_encode_2d(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.xq, (uint64_t)p.k, (uint64_t)p.n_rows, (uint64_t)p.k, 128,
                    128, CU_TENSOR_MAP_SWIZZLE_128B))
    return HQ_ERR_CUDA;
  static bool attr_done[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return HQ_ERR_CUDA;
  if (dev < 64 && !attr_done[dev]) {
    if (cudaFuncSetAttribute(mx_grouped_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMxSmemLimit) !=
        cudaSuccess)
      return HQ_ERR_CUDA;
    attr_done[dev] = true;
  }
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  const int64_t n_exp = p.expert_bounds != nullptr ? p.n_experts : 1;
  const int64_t items = (p.n_rows / 128 + n_exp) * ((p.n + 127) / 128);
  const int64_t grid = items < sms ? items : sms;
  if (p.spin_limit == 0) p.spin_limit = 1u << 22;
  p.y_vec_ok = p.y != nullptr && (reinterpret_cast<uintptr_t>(p.y) & 15u) == 0 &&
               (p.y_stride * dtype_size(p.y_dtype)) % 16 == 0;
  mx_grouped_kernel<<<(unsigned)grid, kMxThreads, MxSmem::total(p.k), stream>>>(tm_w, tm_wtail, tm_x, p);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

}  // namespace hq
