// Decode-regime quantized mat-vec (1..8 activation rows per work item), dense
// and expert-indexed, for block-FP8 and MXFP4 weights (Q8_0 and Q4_K have a kernel
// of their own in hq_gemv_int8.cu and are only dispatched from here).
//
// HBM-bound: every weight byte is read once, straight from the reference's
// device layout.  Persistent CTAs (one per SM) walk work items of 16 output rows.
// Two producer warps stream each item's row segments (>= 2 KiB per bulk async
// copy -- smaller copies cannot keep HBM busy) into a shared-memory ring with
// mbarrier completion; thirteen consumer warps split K thirteen ways, decode the
// blocks in registers into f16 MMA fragments (e4m3 and e2m1 by hardware conversion)
// and multiply them against the (<= 8) activation rows with m16n8k16 warp MMAs,
// f32 accumulation, one scale FMA per 32-element block.
// The thirteen partial sums of an item are handed through shared memory (two
// buffers, mbarrier hand-off, no CTA-wide barrier) to a warp of its own that adds
// them in a fixed order and writes the outputs, so results are bit-reproducible.
//
// Algorithmic bytes per launch: N*K*bits/8 (weights) + M*K*sizeof(x) + M*N*sizeof(y).
#include "hq_gemv_shared.cuh"

namespace hq {

constexpr int kConsumerWarps = 13;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kProducerWarps = 2;   // a bulk-copy instruction holds its warp ~50 cycles per active lane: split the rows
constexpr int kGemvThreads = kConsumerThreads + 32 * (kProducerWarps + 1);   // + producers + the reducing warp
constexpr uint32_t kSpinLimit = 1u << 22;

// shared-memory plan of one launch (computed on the host)
struct GemvLayout {
  int nstage;       // ring stages
  int xs_rows;      // activation rows staged (rows beyond read as zero)
  int xk;           // activation columns per epoch
  int xk_sub;       // columns per register prefetch
  int x_bytes;
  int off_x, off_red, off_bar, total;
};

// ---- per-format geometry ----------------------------------------------------
template <int FMT>
struct FmtTraits;
template <>
struct FmtTraits<HQ_FMT_FP8_BLOCK> {
  static constexpr int kGran = 128;
  __host__ __device__ static constexpr int seg_bytes(int kc) { return kc; }
  __host__ __device__ static int64_t row_bytes(int64_t k) { return k; }
};
template <>
struct FmtTraits<HQ_FMT_MXFP4> {
  static constexpr int kGran = 32;
  __host__ __device__ static constexpr int seg_bytes(int kc) { return kc / 2; }
  __host__ __device__ static int64_t row_bytes(int64_t k) { return k / 2; }
};

__host__ __device__ constexpr int seg_pitch(int seg) {
  // rows of a stage sit `pitch` bytes apart; pitch/4 == 4 (mod 8) spreads the 8 row
  // groups of a warp over all 32 banks for the 32-bit fragment loads
  return ((seg / 4) % 8 == 4) ? seg : seg + 16;
}

template <int FMT, int KC>
struct GemvStage {
  static constexpr int RT = 16;
  static constexpr int SEG = FmtTraits<FMT>::seg_bytes(KC);
  static constexpr int PITCH = seg_pitch(SEG);
  static constexpr int STAGE_BYTES = RT * PITCH;
};
constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 227 * 1024;

// ---- activation staging -----------------------------------------------------
// The (<= 8) activation rows of a work item are staged as f16 in shared memory, kXK columns at a time, in
// fragment order.  Raw bytes are fetched one epoch ahead into registers (16 bytes per group).
constexpr int kMaxXGroups = 9;

struct XPrefetch {
  uint4 v[kMaxXGroups];
};

__device__ __forceinline__ void x_prefetch(XPrefetch& pf, const GemvParams& p, int row0, int nrows, int k0,
                                           int k_len, int tid) {
  const int esz = dtype_size(p.x_dtype);
  const int epg = 16 / esz;              // elements per 16-byte group
  const int gpr = k_len / epg;           // groups per activation row in this epoch
  const int ngroups = nrows * gpr;
#pragma unroll
  for (int i = 0; i < kMaxXGroups; ++i) {
    const int it = i * kConsumerThreads + tid;
    if (it < ngroups) {
      const int col = it / gpr;
      const int kk = (it - col * gpr) * epg;
      const int64_t xr = p.x_rows ? (int64_t)p.x_rows[row0 + col] : (int64_t)(row0 + col);
      const char* src = (const char*)p.x + (xr * p.x_stride + k0 + kk) * esz;
      pf.v[i] = __ldg(reinterpret_cast<const uint4*>(src));
    }
  }
}

__device__ __forceinline__ void x_commit(const XPrefetch& pf, const GemvParams& p, int nrows, int k_len, int tid,
                                         __half* xs, int XP) {
  const int esz = dtype_size(p.x_dtype);
  const int epg = 16 / esz;
  const int gpr = k_len / epg;
  const int ngroups = nrows * gpr;
#pragma unroll
  for (int i = 0; i < kMaxXGroups; ++i) {
    const int it0 = i * kConsumerThreads;
    if (it0 < ngroups) {  // uniform across the block
      const int it = it0 + tid;
      const bool ok = it < ngroups;
      float f[8];
      int col = 0, kk = 0;
      if (ok) {
        col = it / gpr;
        kk = (it - col * gpr) * epg;
        const uint4 raw = pf.v[i];
        if (p.x_dtype == HQ_DT_F32) {
          f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y);
          f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
          f[4] = f[5] = f[6] = f[7] = 0.f;
        } else if (p.x_dtype == HQ_DT_BF16) {
          f[0] = __uint_as_float(raw.x << 16); f[1] = __uint_as_float(raw.x & 0xFFFF0000u);
          f[2] = __uint_as_float(raw.y << 16); f[3] = __uint_as_float(raw.y & 0xFFFF0000u);
          f[4] = __uint_as_float(raw.z << 16); f[5] = __uint_as_float(raw.z & 0xFFFF0000u);
          f[6] = __uint_as_float(raw.w << 16); f[7] = __uint_as_float(raw.w & 0xFFFF0000u);
        } else {
          const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 t = __half22float2(h[j]);
            f[2 * j] = t.x; f[2 * j + 1] = t.y;
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = 0.f;
      }
      // round to f16 (what the MMA sees)
      __half hv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) hv[j] = __float2half_rn(f[j]);
      if (ok) {
        __half* dst = xs + col * XP + kk;
        if (epg == 8) {
          *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(hv);
        } else {
          *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(hv);
        }
      }
    }
  }
}

// ---- block decoders: one "unit" of k for 16 rows x 8 activation columns -----
// Fragment ownership: lane = 4*g + t.  A-fragment rows g and g+8, B-fragment
// column g.  Accumulator: acc[0],acc[1] = (row g, cols 2t,2t+1); acc[2],acc[3] = row g+8.
// Every decoder is split into a load half (shared-memory reads only, issued
// back to back for several units) and a compute half, so the reads of the
// next unit are in flight while the MMAs of this one run.

__device__ __forceinline__ void e4m3x4_to_f16x4(uint32_t v, uint32_t& lo, uint32_t& hi) {
  asm("{\n"
      ".reg .b16 l, h;\n"
      "mov.b32 {l, h}, %2;\n"
      "cvt.rn.f16x2.e4m3x2 %0, l;\n"
      "cvt.rn.f16x2.e4m3x2 %1, h;\n"
      "}\n"
      : "=r"(lo), "=r"(hi)
      : "r"(v));
}

// block-FP8 and MXFP4: unit = 32 elements.
struct B32Regs {
  uint32_t a0, a1, b0, b1;
  uint2 x0, x1;
};
__device__ __forceinline__ void fp8_load(B32Regs& r, uint32_t rowA, uint32_t rowB, uint32_t xs_g, int unit, int t,
                                         bool xv) {
  const uint32_t qo = 32u * unit + 4u * t;
  r.a0 = lds32<0>(rowA + qo); r.a1 = lds32<16>(rowA + qo);
  r.b0 = lds32<0>(rowB + qo); r.b1 = lds32<16>(rowB + qo);
  const uint32_t xo = xs_g + (32u * unit + 4u * t) * 2u;
  r.x0 = xv ? lds64<0>(xo) : make_uint2(0u, 0u);
  r.x1 = xv ? lds64<32>(xo) : make_uint2(0u, 0u);
}
__device__ __forceinline__ void fp8_compute(float (&acc)[4], const B32Regs& r, float scale) {
  float blk[4];
  uint32_t al, ah, bl, bh;
  e4m3x4_to_f16x4(r.a0, al, ah);
  e4m3x4_to_f16x4(r.b0, bl, bh);
  mma_f16_16816_c(blk, al, bl, ah, bh, r.x0.x, r.x0.y, 0.f, 0.f, 0.f, 0.f);
  e4m3x4_to_f16x4(r.a1, al, ah);
  e4m3x4_to_f16x4(r.b1, bl, bh);
  mma_f16_16816(blk, al, bl, ah, bh, r.x1.x, r.x1.y);
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i] = fmaf(scale, blk[i], acc[i]);
}

// four bytes of e2m1 nibble pairs (low nibble = even element = low half) -> four f16x2 by hardware conversion
__device__ __forceinline__ void e2m1x8_to_f16x8(uint32_t w, uint32_t (&h)[4]) {
  asm("{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "mov.b32 {b0, b1, b2, b3}, %4;\n"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n"
      "}\n"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
      : "r"(w));
}
// MXFP4: one 32-element block = 16 bytes; lane t owns bytes 4t..4t+3 (elements 8t..8t+7).
__device__ __forceinline__ void mx_load(B32Regs& r, uint32_t rowA, uint32_t rowB, uint32_t xs_g, int unit, int t,
                                        bool xv) {
  const uint32_t qo = 16u * unit + 4u * t;
  r.a0 = lds32(rowA + qo);
  r.b0 = lds32(rowB + qo);
  const uint32_t xo = xs_g + (32u * unit + 8u * t) * 2u;
  r.x0 = xv ? lds64<0>(xo) : make_uint2(0u, 0u);
  r.x1 = xv ? lds64<8>(xo) : make_uint2(0u, 0u);
}
__device__ __forceinline__ void mx_compute(float (&acc)[4], const B32Regs& r, float sA, float sB) {
  float blk[4];
  uint32_t a[4], b[4];
  e2m1x8_to_f16x8(r.a0, a);
  e2m1x8_to_f16x8(r.b0, b);
  mma_f16_16816_c(blk, a[0], b[0], a[1], b[1], r.x0.x, r.x0.y, 0.f, 0.f, 0.f, 0.f);
  mma_f16_16816(blk, a[2], b[2], a[3], b[3], r.x1.x, r.x1.y);
  acc[0] = fmaf(sA, blk[0], acc[0]);
  acc[1] = fmaf(sA, blk[1], acc[1]);
  acc[2] = fmaf(sB, blk[2], acc[2]);
  acc[3] = fmaf(sB, blk[3], acc[3]);
}

// ---- the kernel --------------------------------------------------------------
// Persistent: each CTA walks work items (activation-row group y, 16-row output tile) with a stride of
// gridDim.x; the producer warp keeps the weight ring full across item boundaries.
template <int FMT, int KC>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_kernel(const GemvParams p, const GemvLayout lay) {
  using L = GemvStage<FMT, KC>;
  using F = FmtTraits<FMT>;
  constexpr int WK = kConsumerWarps;
  constexpr int RT = L::RT;
  const int NSTAGE = lay.nstage;
  extern __shared__ __align__(128) uint8_t smem[];

  const int n_rt = (p.n + RT - 1) / RT;
  const int n_y = p.tiles != nullptr ? p.tile_count[0] : (p.m + 7) / 8;
  const int total = n_y * n_rt;
  // Item walk: dense calls stride through the items; expert-indexed calls take a contiguous run each, so
  // consecutive items of a CTA share their activation rows (one expert tile) and are staged once.
  const bool runs = p.tiles != nullptr;
  const int per = runs ? (total + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  const int w_begin = runs ? (int)blockIdx.x * per : (int)blockIdx.x;
  const int w_end = runs ? min(total, w_begin + per) : total;
  const int w_step = runs ? 1 : (int)gridDim.x;
  if (w_begin >= w_end) return;
  const int kXK = lay.xk;          // activation columns staged per epoch (whole chunks)
  const int xk_sub = lay.xk_sub;   // columns one register prefetch covers
  const int n_super = (p.k + kXK - 1) / kXK;

  uint64_t* full = reinterpret_cast<uint64_t*>(smem + lay.off_bar);
  uint64_t* empty = full + kMaxStages;
  uint64_t* red_full = empty + kMaxStages;   // [2] partial sums of an item are all written
  uint64_t* red_free = red_full + 2;     // [2] ... and have been consumed
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < NSTAGE; ++s) {
      mbar_init(&full[s], kProducerWarps);
      mbar_init(&empty[s], kConsumerWarps);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&red_full[b], kConsumerWarps);
      mbar_init(&red_free[b], 1);
    }
    fence_barrier_init();
  }
  // zero the activation buffer once: rows beyond an item's row count must read as zero
  for (int i = tid; i < lay.x_bytes / 16; i += kGemvThreads)
    reinterpret_cast<uint4*>(smem + lay.off_x)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();

  const int64_t row_bytes = F::row_bytes(p.k);
  const int nchunk = (p.k + KC - 1) / KC;

  if (warp >= kConsumerWarps && warp < kConsumerWarps + kProducerWarps) {
    // ================= producer warps: stream weight row segments ===============
    const int pw = warp - kConsumerWarps;
    constexpr int RPP = RT / kProducerWarps;    // rows per producer warp
    uint32_t spin = kSpinLimit;
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    int s = 0, round = 0;
    for (int w = w_begin; w < w_end; w += w_step) {
      const WorkItem wi = get_item<RT>(p, w, n_rt);
      if (wi.nrows <= 0) continue;
      const int rows_valid = min(RT, p.n - wi.n0);
      const int my_rows = max(0, min(RPP, rows_valid - pw * RPP));
      for (int chunk = 0; chunk < nchunk; ++chunk) {
        const int kc_len = min(KC, p.k - chunk * KC);
        const uint32_t bytes = (uint32_t)F::seg_bytes(kc_len);
        for (int bank = 0; bank < p.n_banks; ++bank) {
          if (round > 0) {
            if (!mbar_wait_backoff(&empty[s], (round - 1) & 1, spin)) {
              // give up waiting but keep the control flow intact: results are invalid and flagged
              if (lane == 0) report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 100 + s);
              spin = 1;
            }
          }
          const uint8_t* wsrc = reinterpret_cast<const uint8_t*>(bank == 0 ? p.w : p.w_up) +
                                (int64_t)wi.expert * p.w_expert_stride + (int64_t)(wi.n0 + pw * RPP) * row_bytes +
                                (int64_t)F::seg_bytes(chunk * KC);
          if (lane == 0) mbar_arrive_expect_tx(&full[s], bytes * (uint32_t)my_rows);
          __syncwarp();
          uint8_t* dst = smem + s * L::STAGE_BYTES + pw * RPP * L::PITCH;
          if (lane < my_rows)
            bulk_g2s_hint(dst + lane * L::PITCH, wsrc + (int64_t)lane * row_bytes, bytes, &full[s], policy);
          if (++s == NSTAGE) {
            s = 0;
            ++round;
          }
        }
      }
    }
    return;
  }

  const int g = lane >> 2, t = lane & 3;
  float* red = reinterpret_cast<float*>(smem + lay.off_red);   // [2 buffers][banks][warps][4][32]

  if (warp == kConsumerWarps + kProducerWarps) {
    // ================= reducing warp: adds the K-split partial sums in warp order and writes ==========
    uint32_t spin = kSpinLimit;
    int item = 0;
    for (int w = w_begin; w < w_end; w += w_step) {
      const WorkItem wi = get_item<RT>(p, w, n_rt);
      if (wi.nrows <= 0) continue;
      const int rb = item & 1;
      const float* rbuf = red + rb * (p.n_banks * kConsumerWarps * 4 * 32);
      bool failed = false;
      if (!mbar_wait_backoff(&red_full[rb], (item >> 1) & 1, spin)) {
        if (lane == 0) report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 310 + rb);
        spin = 1;
        failed = true;                 // nothing is stored for an item whose partial sums never arrived
      }
      float v[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int b = 0; b < 2; ++b)
        if (b < p.n_banks) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < kConsumerWarps; ++j) sum += rbuf[((b * kConsumerWarps + j) * 4 + i) * 32 + lane];
            v[b][i] = sum;
          }
        }
      __syncwarp();
      if (lane == 0) mbar_arrive(&red_free[rb]);
      // rows of this lane: n0 + g (+8); columns 2t, 2t+1
      gemv_store_item(p, wi, g, 2 * t, !failed, v);
      ++item;
    }
    return;
  }

  // ================= consumer warps ============================================
  const int wk = warp;
  __half* xs = reinterpret_cast<__half*>(smem + lay.off_x);
  const int XP = lay.xk + 16;                 // f16 elements per staged activation row
  const bool xv = g < lay.xs_rows;            // activation rows beyond the staged ones are zero
  const uint32_t xs_g = smem_u32(xs) + (uint32_t)(xv ? g : 0) * XP * 2u;

  XPrefetch pf;
  bool pf_valid = false;
  int staged_y = -1;        // activation rows currently in shared memory (valid when n_super == 1)
  int staged_rows = 0;
  {
    const WorkItem w0 = get_item<RT>(p, w_begin, n_rt);
    if (w0.nrows > 0) {
      x_prefetch(pf, p, w0.row0, w0.nrows, 0, min(xk_sub, p.k), tid);
      pf_valid = true;
    }
  }

  uint32_t spin = kSpinLimit;
  int s = 0, it = 0, item = 0;
  uint32_t phase = 0;
  for (int w = w_begin; w < w_end; w += w_step) {
    const WorkItem wi = get_item<RT>(p, w, n_rt);
    if (wi.nrows <= 0) continue;
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    for (int sc = 0; sc < n_super; ++sc) {
      const int k_base = sc * kXK;
      const int k_len = min(kXK, p.k - k_base);
      if (n_super > 1 || wi.y != staged_y) {
        // ---- stage this epoch's activations (all consumer warps) ----------------------------------
        if (!pf_valid) x_prefetch(pf, p, wi.row0, wi.nrows, k_base, min(xk_sub, k_len), tid);
        named_bar_sync(1, kConsumerThreads);       // everyone is done reading the previous epoch
        // rows left over from an earlier item with more rows than this one must read as zero
        for (int i = tid; i < (staged_rows - wi.nrows) * (XP / 8); i += kConsumerThreads)
          reinterpret_cast<uint4*>(xs + wi.nrows * XP)[i] = make_uint4(0, 0, 0, 0);
        staged_rows = wi.nrows;
        x_commit(pf, p, wi.nrows, min(xk_sub, k_len), tid, xs, XP);
        for (int sub = xk_sub; sub < k_len; sub += xk_sub) {   // f32 input: second half, fetched now
          x_prefetch(pf, p, wi.row0, wi.nrows, k_base + sub, min(xk_sub, k_len - sub), tid);
          x_commit(pf, p, wi.nrows, min(xk_sub, k_len - sub), tid, xs + sub, XP);
        }
        staged_y = wi.y;
        pf_valid = false;
        // fetch the next epoch's activations while this one is being consumed
        if (sc + 1 < n_super) {
          x_prefetch(pf, p, wi.row0, wi.nrows, k_base + kXK, min(xk_sub, p.k - k_base - kXK), tid);
          pf_valid = true;
        } else if (w + w_step < w_end) {
          const WorkItem nx = get_item<RT>(p, w + w_step, n_rt);
          if (nx.nrows > 0 && (n_super > 1 || nx.y != wi.y)) {
            x_prefetch(pf, p, nx.row0, nx.nrows, 0, min(xk_sub, p.k), tid);
            pf_valid = true;
          }
        }
        named_bar_sync(1, kConsumerThreads);
      }
      const int c0 = k_base / KC, c1 = (k_base + k_len + KC - 1) / KC;
      for (int chunk = c0; chunk < c1; ++chunk) {
        const int kc_len = min(KC, p.k - chunk * KC);
        const int kx = chunk * KC - k_base;      // offset of this chunk inside the staged activations
#pragma unroll
        for (int bank = 0; bank < 2; ++bank) {
          if (bank >= p.n_banks) break;
          if (!mbar_wait(&full[s], phase, spin)) {
            // bounded wait ran out: flag it and carry on (every warp still reaches every barrier)
            if (lane == 0) report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 200 + s);
            spin = 1;
          }
          ++it;
          // the units of a stage do not divide evenly among the warps: rotate who gets the extra one
          const int wrot = (wk + it) % WK;
          const uint32_t rowA = smem_u32(smem + s * L::STAGE_BYTES) + (uint32_t)g * L::PITCH;
          const uint32_t rowB = rowA + 8u * L::PITCH;
          const uint32_t xs_c = xs_g + 2u * kx;
          float(&a)[4] = acc[bank];
          if (FMT == HQ_FMT_FP8_BLOCK) {
            const int nunits = kc_len / 32;
            const float* fsc = reinterpret_cast<const float*>(bank == 0 ? p.scales : p.scales_up) +
                               (int64_t)wi.expert * p.scale_expert_stride +
                               (int64_t)(wi.n0 / 128) * ((p.k + 127) / 128);
            int u = wrot;
            for (; u + WK < nunits; u += 2 * WK) {
              B32Regs r0, r1;
              fp8_load(r0, rowA, rowB, xs_c, u, t, xv);
              fp8_load(r1, rowA, rowB, xs_c, u + WK, t, xv);
              const float s0 = __ldg(fsc + (chunk * KC + 32 * u) / 128);
              const float s1 = __ldg(fsc + (chunk * KC + 32 * (u + WK)) / 128);
              fp8_compute(a, r0, s0);
              fp8_compute(a, r1, s1);
            }
            if (u < nunits) {
              B32Regs r0;
              fp8_load(r0, rowA, rowB, xs_c, u, t, xv);
              fp8_compute(a, r0, __ldg(fsc + (chunk * KC + 32 * u) / 128));
            }
          } else {
            const int nunits = kc_len / 32;
            const int kb_row = p.k / 32;
            const uint8_t* msc = reinterpret_cast<const uint8_t*>(bank == 0 ? p.scales : p.scales_up) +
                                 (int64_t)wi.expert * p.scale_expert_stride + chunk * (KC / 32);
            const uint8_t* mA = msc + (int64_t)min(wi.n0 + g, p.n - 1) * kb_row;
            const uint8_t* mB = msc + (int64_t)min(wi.n0 + g + 8, p.n - 1) * kb_row;
            for (int u = wrot; u < nunits; u += WK) {
              B32Regs r0;
              mx_load(r0, rowA, rowB, xs_c, u, t, xv);
              // 2^(e-127) with the reference's bit trick (e = 0 decodes to 0)
              const float sA = __uint_as_float((uint32_t)__ldg(mA + u) << 23);
              const float sB = __uint_as_float((uint32_t)__ldg(mB + u) << 23);
              mx_compute(a, r0, sA, sB);
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&empty[s]);
          if (++s == NSTAGE) {
            s = 0;
            phase ^= 1u;
          }
        }
      }
    }

    // ---- hand the K-split partials to the reducing warp (two buffers) ----------------------------------
    const int rb = item & 1;
    float* rbuf = red + rb * (p.n_banks * kConsumerWarps * 4 * 32);
    if (item >= 2) {
      if (!mbar_wait(&red_free[rb], ((item >> 1) - 1) & 1, spin)) {
        if (lane == 0) report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 300 + rb);
        spin = 1;
      }
    }
#pragma unroll
    for (int b = 0; b < 2; ++b)
      if (b < p.n_banks) {
#pragma unroll
        for (int i = 0; i < 4; ++i) rbuf[((b * kConsumerWarps + warp) * 4 + i) * 32 + lane] = acc[b][i];
      }
    __syncwarp();
    if (lane == 0) mbar_arrive(&red_full[rb]);
    ++item;
  }
}

// ---- host launcher ------------------------------------------------------------
template <int FMT, int KC>
static int32_t launch_cfg(const GemvParams& p, int n_y_max, int max_rows, cudaStream_t stream) {
  using L = GemvStage<FMT, KC>;
  using F = FmtTraits<FMT>;
  static_assert((L::PITCH / 4) % 8 == 4, "row pitch must spread banks");
  static_assert(F::seg_bytes(KC) >= 2048, "bulk copies below 2 KiB cannot saturate HBM");
  // Shared-memory plan: stage as many activation columns as leave at least four ring stages (the whole K when
  // it fits -- then a persistent CTA converts its activations once), give every remaining byte to the ring.
  GemvLayout lay{};
  const int esz = dtype_size(p.x_dtype);
  const int k_round = (p.k + KC - 1) / KC * KC;
  const int candidates[3] = {k_round, 8192 < k_round ? (8192 / KC * KC) : k_round, 4096 < k_round ? 4096 : k_round};
  for (int c = 0; c < 3; ++c) {
    lay.xk = candidates[c];
    lay.xs_rows = max_rows;
    lay.x_bytes = lay.xs_rows * (lay.xk + 16) * 2;
    const int red_bytes = 2 * p.n_banks * kConsumerWarps * 4 * 32 * 4;
    const int bar_bytes = (2 * kMaxStages + 4) * 8 + 16;
    const int fixed = lay.x_bytes + red_bytes + bar_bytes;
    int nst = (kSmemBudget - fixed) / L::STAGE_BYTES;
    if (nst > kMaxStages) nst = kMaxStages;
    lay.nstage = nst;
    lay.off_x = nst * L::STAGE_BYTES;
    lay.off_red = lay.off_x + lay.x_bytes;
    lay.off_bar = lay.off_red + red_bytes;
    lay.total = lay.off_bar + bar_bytes;
    if (nst >= 4) break;
  }
  if (lay.nstage < 2) return HQ_ERR_SHAPE;
  // columns one register prefetch can hold (kMaxXGroups groups of 16 bytes per thread), in whole 256-column steps
  int sub = (kMaxXGroups * kConsumerThreads * 16) / (lay.xs_rows * esz) / 256 * 256;
  lay.xk_sub = sub < lay.xk ? sub : lay.xk;
  auto kern = gemv_kernel<FMT, KC>;
  static bool attr_done[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return HQ_ERR_CUDA;
  if (dev < 64 && !attr_done[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget) != cudaSuccess)
      return HQ_ERR_CUDA;
    attr_done[dev] = true;
  }
  const int64_t items = (int64_t)n_y_max * ((p.n + L::RT - 1) / L::RT);
  const int64_t grid = items < sm_count() ? items : sm_count();
  if (grid <= 0) return HQ_OK;
  kern<<<(unsigned)grid, kGemvThreads, lay.total, stream>>>(p, lay);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

int32_t launch_gemv(const GemvParams& p, int n_y_max, cudaStream_t stream) {
  // most activation rows any work item of this launch can have
  const int max_rows = p.tiles != nullptr ? 8 : (p.m < 8 ? p.m : 8);
  // chunk sizes keep every bulk copy (one row segment) at 2 KiB or more
  switch (p.format) {
    case HQ_FMT_Q8_0:
    case HQ_FMT_Q4_K: return launch_gemv_int8(p, n_y_max, max_rows, stream);   // integer-MMA kernel
    case HQ_FMT_FP8_BLOCK:
      // one or two activation rows: the FP8 warp-MMA kernel (weights unconverted), for shapes whose 16-row items
      // stay inside one weight-scale block
      if (max_rows <= 2 && p.k % 256 == 0 && p.n % 16 == 0) return launch_gemv_int8(p, n_y_max, max_rows, stream);
      return launch_cfg<HQ_FMT_FP8_BLOCK, 2048>(p, n_y_max, max_rows, stream);
    case HQ_FMT_MXFP4: return launch_cfg<HQ_FMT_MXFP4, 4096>(p, n_y_max, max_rows, stream);
    case HQ_FMT_Q6_K:
    case HQ_FMT_Q5_K:
    case HQ_FMT_Q4_0:
    case HQ_FMT_Q5_0:
    case HQ_FMT_Q4_1:
    case HQ_FMT_Q5_1:
    case HQ_FMT_Q2_K:
    case HQ_FMT_Q3_K: return launch_gemv_ggml_mma(p, n_y_max, stream);
    default: return HQ_ERR_FORMAT;
  }
}

}  // namespace hq
