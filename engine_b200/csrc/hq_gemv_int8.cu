// Decode-regime mat-vec (1..8 activation rows per work item), dense and expert-indexed, for the formats whose
// codes a narrow warp MMA takes as they lie in memory: GGUF Q8_0 and Q4_K on the integer MMA, block-FP8 (one or
// two rows) on the FP8 MMA.  The description below follows Q8_0; the Q4_K and FP8 specifics are at their group
// routines (q4k_group, fp8_group).
//
// HBM-bound: every weight byte is read once, straight from the 34-byte blocks {f16 d, int8 q[32]}.
// What limits such a kernel on the SM side is the number of instructions spent per weight byte, so the
// int8 codes are never converted: they go into the integer warp MMA (m16n8k32, s8 x s8 -> s32) exactly as
// they lie in the block.  The activations are made to fit instead: each 128-element group of an
// activation row is written as x ~= s * (h + l / 256) with int8 h and l (s a power of two; 256 h + l is x / s
// rounded to 16-bit fixed point, so the error is below max|x| / 32000 per element), and h and l occupy separate MMA columns.
// One MMA then yields the exact integer dot products of one block for all rows and columns; they leave
// the accumulator as floats through a bias constant (no conversion instruction), are multiplied by the
// block's d, summed over the four blocks of a group and scaled once by the group's activation scale.
//
// Layout of the work: persistent CTAs (one per SM) walk items of 16 output rows.  Two producer warps stream
// the item's row segments (2176 bytes = 64 blocks per bulk async copy; copies below 2 KiB cannot keep HBM
// busy) into a shared-memory ring with mbarrier completion.  The consumer warps each take groups of
// four blocks (136 bytes, 8-byte aligned) of every stage, so the misaligned block payloads are fetched
// with a fixed pattern of 8- and 4-byte loads and four funnel shifts per row.  Within an MMA the k order
// is free as long as both operands agree: lane t owns payload bytes 8t..8t+7 of a block, and reads the
// same eight positions of the staged activations with one 8-byte load.  Partial sums of the K slices
// meet in shared memory and are added in warp order by a warp of their own: results are
// bit-reproducible.
//
// Algorithmic bytes per launch: N*K*34/32 (weights) + M*K*sizeof(x) + M*N*sizeof(y).
#include "hq_gemv_shared.cuh"

namespace hq {

#ifndef HQ_Q8_GROUPS_PER_WARP
#define HQ_Q8_GROUPS_PER_WARP 2
#endif
constexpr int kQ8GroupsPerWarp = HQ_Q8_GROUPS_PER_WARP;   // 128-element groups a warp takes from every stage
constexpr int kQ8Warps = 16 / kQ8GroupsPerWarp;  // consumer warps
constexpr int kQ8Consumers = kQ8Warps * 32;
constexpr int kQ8Producers = 2;                  // producer warps: a bulk-copy instruction holds its warp for ~50
                                                 // cycles per active lane, so the 16 row copies of a stage are
                                                 // split over two warps
constexpr int kQ8Threads = kQ8Consumers + 32 * (kQ8Producers + 1);   // + producers + the reducing warp
constexpr int kQ8RT = 16;

// Stage geometry per format.  A stage holds KC columns of 16 weight rows = 16 groups of GK columns; a group is
// the unit a consumer warp works on (Q8_0: four 34-byte blocks = 136 bytes; Q4_K: one 144-byte super-block)
// and the unit that shares one activation step.  Row segments (one bulk copy each) are >= 2 KiB; the row
// pitch in a stage is = 32 (mod 128) so 8-byte loads of 4 rows x 4 lanes cover all banks.
template <int FMT>
struct I8Traits;
template <>
struct I8Traits<HQ_FMT_Q8_0> {
  static constexpr int KC = 2048, GK = 128, GROUP_BYTES = 136;
  static constexpr int SEG = KC / 32 * 34, PITCH = SEG + 32, STAGE_BYTES = kQ8RT * PITCH;
  __host__ __device__ static constexpr int64_t row_bytes(int64_t k) { return k / 32 * 34; }
  static constexpr bool kSubSums = false;
};
template <>
struct I8Traits<HQ_FMT_Q4_K> {
  static constexpr int KC = 4096, GK = 256, GROUP_BYTES = 144;
  static constexpr int SEG = KC / 256 * 144, PITCH = SEG + 32, STAGE_BYTES = kQ8RT * PITCH;
  __host__ __device__ static constexpr int64_t row_bytes(int64_t k) { return k / 256 * 144; }
  static constexpr bool kSubSums = true;     // per 32-element sub-block sums of the staged bytes (the min term)
};
constexpr int kQ8MaxStages = 8;
constexpr int kQ8SmemBudget = 227 * 1024 - 256;   // dynamic part; a few static words come on top
constexpr int kQ8XGroups = 8;                    // 16-byte registers a thread prefetches activations into
constexpr uint32_t kQ8Spin = 1u << 22;
constexpr int kQ8Magic = 0x4B400000;             // 1.5 * 2^23 as f32 bits: magic + n reads as 12582912.f + n
template <>
struct I8Traits<HQ_FMT_FP8_BLOCK> {
  // e4m3 codes, one byte per weight: a 128-column group is 128 bytes and shares one weight-block scale
  static constexpr int KC = 2048, GK = 128, GROUP_BYTES = 128;
  static constexpr int SEG = KC, PITCH = SEG + 32, STAGE_BYTES = kQ8RT * PITCH;
  __host__ __device__ static constexpr int64_t row_bytes(int64_t k) { return k; }
  static constexpr bool kSubSums = false;
};
static_assert(I8Traits<HQ_FMT_Q8_0>::SEG >= 2048 && I8Traits<HQ_FMT_Q8_0>::SEG % 16 == 0, "bulk copy size");
static_assert(I8Traits<HQ_FMT_Q4_K>::SEG >= 2048 && I8Traits<HQ_FMT_Q4_K>::SEG % 16 == 0, "bulk copy size");
static_assert(I8Traits<HQ_FMT_Q8_0>::PITCH % 128 == 32 && I8Traits<HQ_FMT_Q4_K>::PITCH % 128 == 32, "row pitch");
static_assert(I8Traits<HQ_FMT_Q8_0>::KC / I8Traits<HQ_FMT_Q8_0>::GK == 16 && I8Traits<HQ_FMT_Q4_K>::KC / I8Traits<HQ_FMT_Q4_K>::GK == 16, "16 groups per stage");

// shared-memory plan of one launch (computed on the host)
struct Q8Layout {
  int nstage;
  int ncols;        // staged int8 columns: 8 = (h, l) of <= 4 activation rows, 16 = (h, l) of <= 8
  int xk;           // activation columns staged per epoch (whole stages)
  int xk_sub;       // columns one register prefetch covers
  int xpitch;       // bytes between staged columns, = 32 (mod 128)
  int x_bytes;
  int off_x, off_sx, off_xs, off_red, off_bar, total;   // off_xs: Q4_K sub-block sums [group][column][16]
  int kslices;            // K slices worked by different CTAs (1 = a CTA covers the whole K)
  int slice_k;            // activation columns per slice: a multiple of 256 (the last slice may be shorter)
  int32_t* counters;      // split K: arrivals per item stream (zero between launches)
  float* partials;        // split K: [item][slice][bank][4][32] partial sums
};

__device__ __forceinline__ void mma_s8_16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1, int c) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c));
}

// the same shape with e4m3 operands and f32 accumulation (D += A.B)
__device__ __forceinline__ void mma_e4m3_16832(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Programmatic dependent launch: the kernel after this one in the stream may start its CTAs as ours retire (and
// this kernel may have been started that way): everything that does not depend on the previous kernel -- barrier
// set-up, the first weight stages -- then overlaps its tail.  Whatever reads activations, the scratch or
// dispatch tables, or writes outputs, first waits for the previous kernel to have completed.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// two f32 lanes per instruction (sm_100): the accumulator pairs of one weight row share every factor
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ uint64_t f2_pack_bits(int lo, int hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

// ---- activation staging ---------------------------------------------------------------------
// Raw activations are fetched one epoch ahead into registers, eight elements per item (16 bytes of f16 / bf16,
// 32 bytes of f32), then every GK-element group of a row is quantized by the GK/8 lanes that hold it.
struct Q8XPrefetch {
  uint4 v[kQ8XGroups];
};

__device__ __forceinline__ void q8_x_prefetch(Q8XPrefetch& pf, const GemvParams& p, int row0, int nrows, int k0,
                                              int k_len, int tid) {
  const bool wide = p.x_dtype == HQ_DT_F32;
  const int ipr = k_len >> 3;            // items per activation row in this epoch
  const int nitems = nrows * ipr;
  const int per_thread = wide ? kQ8XGroups / 2 : kQ8XGroups;
#pragma unroll
  for (int i = 0; i < kQ8XGroups; ++i) {
    const int it = i * kQ8Consumers + tid;
    if (i < per_thread && it < nitems) {
      const int col = it / ipr;
      const int kk = (it - col * ipr) << 3;
      const int64_t xr = p.x_rows ? (int64_t)p.x_rows[row0 + col] : (int64_t)(row0 + col);
      const char* src = (const char*)p.x + (xr * p.x_stride + k0 + kk) * (wide ? 4 : 2);
      if (wide) {
        pf.v[(2 * i) % kQ8XGroups] = __ldg(reinterpret_cast<const uint4*>(src));
        pf.v[(2 * i + 1) % kQ8XGroups] = __ldg(reinterpret_cast<const uint4*>(src) + 1);
      } else {
        pf.v[i] = __ldg(reinterpret_cast<const uint4*>(src));
      }
    }
  }
}

// k_len is a multiple of 256, so a warp never straddles two activation rows and is valid or idle as a whole.
// xq: staged int8 columns of this epoch (column c at xq + c * xpitch), already offset to the sub-range;
// sx: step table [group][ncols] f32, xs: sub-block sums [group][ncols][16] bytes, likewise offset.
template <int GK, bool SUBSUMS>
__device__ __forceinline__ void q8_x_commit(const Q8XPrefetch& pf, const GemvParams& p, int nrows, int k_len, int tid,
                                            uint8_t* xq, int xpitch, float* sx, uint8_t* xs, int ncols) {
  const bool wide = p.x_dtype == HQ_DT_F32;
  const int ipr = k_len >> 3;
  const int nitems = nrows * ipr;
  const int per_thread = wide ? kQ8XGroups / 2 : kQ8XGroups;
  const int l_off = ncols >> 1;          // column of the low byte relative to the high byte
#pragma unroll
  for (int i = 0; i < kQ8XGroups; ++i) {
    const int it = i * kQ8Consumers + tid;
    if (i < per_thread && it < nitems) {   // uniform across the warp
      const int col = it / ipr;
      const int kk = (it - col * ipr) << 3;
      float f[8];
      if (wide) {
        const uint4 r0 = pf.v[(2 * i) % kQ8XGroups], r1 = pf.v[(2 * i + 1) % kQ8XGroups];
        f[0] = __uint_as_float(r0.x); f[1] = __uint_as_float(r0.y);
        f[2] = __uint_as_float(r0.z); f[3] = __uint_as_float(r0.w);
        f[4] = __uint_as_float(r1.x); f[5] = __uint_as_float(r1.y);
        f[6] = __uint_as_float(r1.z); f[7] = __uint_as_float(r1.w);
      } else if (p.x_dtype == HQ_DT_BF16) {
        const uint4 raw = pf.v[i];
        f[0] = __uint_as_float(raw.x << 16); f[1] = __uint_as_float(raw.x & 0xFFFF0000u);
        f[2] = __uint_as_float(raw.y << 16); f[3] = __uint_as_float(raw.y & 0xFFFF0000u);
        f[4] = __uint_as_float(raw.z << 16); f[5] = __uint_as_float(raw.z & 0xFFFF0000u);
        f[6] = __uint_as_float(raw.w << 16); f[7] = __uint_as_float(raw.w & 0xFFFF0000u);
      } else {
        const uint4 raw = pf.v[i];
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 t = __half22float2(h[j]);
          f[2 * j] = t.x; f[2 * j + 1] = t.y;
        }
      }
      // largest magnitude as an integer maximum of the sign-cleared bits: NaN and infinity order above every
      // finite value, so either makes the group's step non-finite instead of vanishing in an fmax
      uint32_t abits = 0u;
#pragma unroll
      for (int j = 0; j < 8; ++j) abits = max(abits, __float_as_uint(f[j]) & 0x7FFFFFFFu);
      abits = max(abits, __shfl_xor_sync(0xffffffffu, abits, 1));
      abits = max(abits, __shfl_xor_sync(0xffffffffu, abits, 2));
      abits = max(abits, __shfl_xor_sync(0xffffffffu, abits, 4));
      abits = max(abits, __shfl_xor_sync(0xffffffffu, abits, 8));
      if (GK == 256) abits = max(abits, __shfl_xor_sync(0xffffffffu, abits, 16));
      const float amax = __uint_as_float(abits);
      // The step s is the power of two at or above amax / 127 (not below 2^-100), so x / s and the products
      // with s are exact: an activation that is a small multiple of s (a one-hot row, say) passes through
      // without any rounding.  Non-finite input must not turn into a finite output: its step is a NaN.
      const bool finite = abits < 0x7F800000u;
      const uint32_t tb = __float_as_uint(fmaxf(amax / 127.f, 7.888609052e-31f));
      const float s = finite ? __uint_as_float((tb + 0x007FFFFFu) & 0x7F800000u) : __int_as_float(0x7fc00000);
      const float inv256 = (finite && abits != 0u) ? 256.f / s : 0.f;
      // x / s as 16-bit fixed point u = rint(256 x / s) + 128 = 256 h + (l + 128): h is the high byte, the low
      // byte is l in offset binary
      uint32_t u[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) u[j] = (uint32_t)__float2int_rn(fmaf(f[j], inv256, 128.f));
      uint32_t hq[2], lq[2];
#pragma unroll
      for (int w2 = 0; w2 < 2; ++w2) {
        const uint32_t p01 = __byte_perm(u[4 * w2], u[4 * w2 + 1], 0x5140);      // bytes l0 l1 h0 h1
        const uint32_t p23 = __byte_perm(u[4 * w2 + 2], u[4 * w2 + 3], 0x5140);
        hq[w2] = __byte_perm(p01, p23, 0x7632);
        lq[w2] = __byte_perm(p01, p23, 0x5410) ^ 0x80808080u;
      }
      uint8_t* dh = xq + col * xpitch + kk;
      uint8_t* dl = dh + l_off * xpitch;
      *reinterpret_cast<uint2*>(dh) = make_uint2(hq[0], hq[1]);
      *reinterpret_cast<uint2*>(dl) = make_uint2(lq[0], lq[1]);
      if ((kk & (GK - 1)) == 0) {
        float* d = sx + (kk / GK) * ncols + col;
        d[0] = s;
        d[l_off] = s * (1.f / 256.f);
      }
      if (SUBSUMS) {
        // sums of the staged bytes over each 32-element sub-block (4 lanes), written as 32 a + b with int8 a
        // and b in 0..31, for the integer dot product with the sub-block minima
        int sh = 0, sl = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          sh += (int)u[j] >> 8;
          sl += (int)(u[j] & 0xFFu) - 128;
        }
        sh += __shfl_xor_sync(0xffffffffu, sh, 1);
        sl += __shfl_xor_sync(0xffffffffu, sl, 1);
        sh += __shfl_xor_sync(0xffffffffu, sh, 2);
        sl += __shfl_xor_sync(0xffffffffu, sl, 2);
        if ((kk & 31) == 0) {
          const int j = (kk & 255) >> 5;
          uint8_t* e = xs + ((kk >> 8) * ncols + col) * 16 + j;
          e[0] = (uint8_t)(sh >> 5);
          e[8] = (uint8_t)(sh & 31);
          e[l_off * 16] = (uint8_t)(sl >> 5);
          e[l_off * 16 + 8] = (uint8_t)(sl & 31);
        }
      }
    }
  }
}

// Staging for block-FP8 weights: the e4m3 weight codes go into the FP8 warp MMA as they are, so the activations
// become e4m3 as well -- three terms per value, x / s ~= t1 + t2 / 16 + t3 / 256 with s a power of two at or above
// max|x| / 448 over the 128-element group (12 significant bits: error below max|x| / 2^13 of the group).  The
// terms occupy separate columns, `tstride` = 2 columns apart (at most two activation rows share the column set).
__device__ __forceinline__ uint32_t f32x4_to_e4m3x4(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
  return (uint32_t)lo | ((uint32_t)hi << 16);
}
__device__ __forceinline__ void e4m3x4_to_f32x4(uint32_t v, float (&f)[4]) {
  uint32_t lo, hi;
  asm("{\n"
      ".reg .b16 l, h;\n"
      "mov.b32 {l, h}, %2;\n"
      "cvt.rn.f16x2.e4m3x2 %0, l;\n"
      "cvt.rn.f16x2.e4m3x2 %1, h;\n"
      "}\n"
      : "=r"(lo), "=r"(hi)
      : "r"(v));
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}

__device__ __forceinline__ void fp8_x_commit(const Q8XPrefetch& pf, const GemvParams& p, int nrows, int k_len, int tid,
                                             uint8_t* xq, int xpitch, float* sx, int ncols, int tstride) {
  const bool wide = p.x_dtype == HQ_DT_F32;
  const int ipr = k_len >> 3;
  const int nitems = nrows * ipr;
  const int per_thread = wide ? kQ8XGroups / 2 : kQ8XGroups;
#pragma unroll
  for (int i = 0; i < kQ8XGroups; ++i) {
    const int it = i * kQ8Consumers + tid;
    if (i < per_thread && it < nitems) {   // uniform across the warp
      const int col = it / ipr;
      const int kk = (it - col * ipr) << 3;
      float f[8];
      if (wide) {
        const uint4 r0 = pf.v[(2 * i) % kQ8XGroups], r1 = pf.v[(2 * i + 1) % kQ8XGroups];
        f[0] = __uint_as_float(r0.x); f[1] = __uint_as_float(r0.y);
        f[2] = __uint_as_float(r0.z); f[3] = __uint_as_float(r0.w);
        f[4] = __uint_as_float(r1.x); f[5] = __uint_as_float(r1.y);
        f[6] = __uint_as_float(r1.z); f[7] = __uint_as_float(r1.w);
      } else if (p.x_dtype == HQ_DT_BF16) {
        const uint4 raw = pf.v[i];
        f[0] = __uint_as_float(raw.x << 16); f[1] = __uint_as_float(raw.x & 0xFFFF0000u);
        f[2] = __uint_as_float(raw.y << 16); f[3] = __uint_as_float(raw.y & 0xFFFF0000u);
        f[4] = __uint_as_float(raw.z << 16); f[5] = __uint_as_float(raw.z & 0xFFFF0000u);
        f[6] = __uint_as_float(raw.w << 16); f[7] = __uint_as_float(raw.w & 0xFFFF0000u);
      } else {
        const uint4 raw = pf.v[i];
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 t = __half22float2(h[j]);
          f[2 * j] = t.x; f[2 * j + 1] = t.y;
        }
      }
      uint32_t abits = 0u;
#pragma unroll
      for (int j = 0; j < 8; ++j) abits = max(abits, __float_as_uint(f[j]) & 0x7FFFFFFFu);
      abits = max(abits, __shfl_xor_sync(0xffffffffu, abits, 1));
      abits = max(abits, __shfl_xor_sync(0xffffffffu, abits, 2));
      abits = max(abits, __shfl_xor_sync(0xffffffffu, abits, 4));
      abits = max(abits, __shfl_xor_sync(0xffffffffu, abits, 8));
      const float amax = __uint_as_float(abits);
      const bool finite = abits < 0x7F800000u;
      const uint32_t tb = __float_as_uint(fmaxf(amax / 448.f, 7.888609052e-31f));
      const float s = finite ? __uint_as_float((tb + 0x007FFFFFu) & 0x7F800000u) : __int_as_float(0x7fc00000);
      const float inv = (finite && abits != 0u) ? 1.f / s : 0.f;
      uint32_t t1[2], t2[2], t3[2];
#pragma unroll
      for (int w2 = 0; w2 < 2; ++w2) {
        float v[4], d[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = f[4 * w2 + j] * inv;
        t1[w2] = f32x4_to_e4m3x4(v[0], v[1], v[2], v[3]);
        e4m3x4_to_f32x4(t1[w2], d);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = (v[j] - d[j]) * 16.f;
        t2[w2] = f32x4_to_e4m3x4(v[0], v[1], v[2], v[3]);
        e4m3x4_to_f32x4(t2[w2], d);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = (v[j] - d[j]) * 16.f;
        t3[w2] = f32x4_to_e4m3x4(v[0], v[1], v[2], v[3]);
      }
      uint8_t* d1 = xq + col * xpitch + kk;
      *reinterpret_cast<uint2*>(d1) = make_uint2(t1[0], t1[1]);
      *reinterpret_cast<uint2*>(d1 + tstride * xpitch) = make_uint2(t2[0], t2[1]);
      *reinterpret_cast<uint2*>(d1 + 2 * tstride * xpitch) = make_uint2(t3[0], t3[1]);
      if ((kk & 127) == 0) {
        float* dsx = sx + (kk >> 7) * ncols + col;
        dsx[0] = s;
        dsx[tstride] = s * (1.f / 16.f);
        dsx[2 * tstride] = s * (1.f / 256.f);
      }
    }
  }
}

// one 128-column group of e4m3 weights x 16 rows x NCS column sets: four MMAs accumulate in f32 (the weight-block
// scale `ws` is the same for all 16 rows and the whole group), then one FMA per accumulator with ws x the column's
// activation step
template <int NCS>
__device__ __forceinline__ void fp8_group(float (&acc)[NCS][4], uint32_t pa, uint32_t pb, uint32_t xq,
                                          uint32_t cs_stride, uint32_t sx, float ws) {
  const uint2 a0 = lds64<0>(pa), a1 = lds64<32>(pa), a2 = lds64<64>(pa), a3 = lds64<96>(pa);
  const uint2 b0 = lds64<0>(pb), b1 = lds64<32>(pb), b2 = lds64<64>(pb), b3 = lds64<96>(pb);
  uint2 xb[NCS][4];
  uint2 sxv[NCS];
#pragma unroll
  for (int c = 0; c < NCS; ++c) {
    const uint32_t xc = xq + c * cs_stride;
    xb[c][0] = lds64<0>(xc); xb[c][1] = lds64<32>(xc); xb[c][2] = lds64<64>(xc); xb[c][3] = lds64<96>(xc);
    sxv[c] = lds64(sx + 32u * c);
  }
#pragma unroll
  for (int c = 0; c < NCS; ++c) {
    float d[4] = {0.f, 0.f, 0.f, 0.f};
    mma_e4m3_16832(d, a0.x, b0.x, a0.y, b0.y, xb[c][0].x, xb[c][0].y);
    mma_e4m3_16832(d, a1.x, b1.x, a1.y, b1.y, xb[c][1].x, xb[c][1].y);
    mma_e4m3_16832(d, a2.x, b2.x, a2.y, b2.y, xb[c][2].x, xb[c][2].y);
    mma_e4m3_16832(d, a3.x, b3.x, a3.y, b3.y, xb[c][3].x, xb[c][3].y);
    const float s0 = ws * __uint_as_float(sxv[c].x), s1 = ws * __uint_as_float(sxv[c].y);
    acc[c][0] = fmaf(d[0], s0, acc[c][0]);
    acc[c][1] = fmaf(d[1], s1, acc[c][1]);
    acc[c][2] = fmaf(d[2], s0, acc[c][2]);
    acc[c][3] = fmaf(d[3], s1, acc[c][3]);
  }
}

// ---- one group: four blocks x 16 weight rows x NCS column sets --------------------------------
// Fragment ownership: lane = 4*g + t.  A rows g and g+8; B column g of each column set; accumulator
// element 0, 1 = (row g, columns 2t, 2t+1), element 2, 3 = row g+8.
//   pa, pb : shared addresses of the group in rows g and g+8, plus 8t
//   da, db : the same without the 8t (block headers)
//   xq     : shared address of staged column g at this group's first element, plus 8t
//   cs_stride : bytes between column sets (8 staged columns)
//   sx     : shared address of this group's scale-table row, plus 8t bytes (columns 2t, 2t+1)
template <int NCS>
__device__ __forceinline__ void q8_group(float (&acc)[NCS][4], uint32_t pa, uint32_t pb, uint32_t da, uint32_t db,
                                         uint32_t xq, uint32_t cs_stride, uint32_t sx) {
  // ---- all shared loads first ----
  const uint2 a0 = lds64<0>(pa);   const uint32_t a0x = lds32<8>(pa);
  const uint32_t a1l = lds32<36>(pa), a1h = lds32<40>(pa);
  const uint32_t a2x = lds32<68>(pa); const uint2 a2 = lds64<72>(pa);
  const uint2 a3 = lds64<104>(pa);
  const uint2 b0 = lds64<0>(pb);   const uint32_t b0x = lds32<8>(pb);
  const uint32_t b1l = lds32<36>(pb), b1h = lds32<40>(pb);
  const uint32_t b2x = lds32<68>(pb); const uint2 b2 = lds64<72>(pb);
  const uint2 b3 = lds64<104>(pb);
  uint2 xb[NCS][4];
  uint2 sxv[NCS];
#pragma unroll
  for (int c = 0; c < NCS; ++c) {
    const uint32_t xc = xq + c * cs_stride;
    xb[c][0] = lds64<0>(xc); xb[c][1] = lds64<32>(xc); xb[c][2] = lds64<64>(xc); xb[c][3] = lds64<96>(xc);
    sxv[c] = lds64(sx + 32u * c);
  }
  uint32_t dA[4], dB[4];
  dA[0] = lds16<0>(da); dA[1] = lds16<34>(da); dA[2] = lds16<68>(da); dA[3] = lds16<102>(da);
  dB[0] = lds16<0>(db); dB[1] = lds16<34>(db); dB[2] = lds16<68>(db); dB[3] = lds16<102>(db);

  // ---- block payloads: lane t owns bytes 8t..8t+7 of each block (payloads start at 2, 36, 70, 104) ----
  uint32_t alo[4], ahi[4], blo[4], bhi[4];
  alo[0] = __funnelshift_r(a0.x, a0.y, 16); ahi[0] = __funnelshift_r(a0.y, a0x, 16);
  alo[1] = a1l;                             ahi[1] = a1h;
  alo[2] = __funnelshift_r(a2x, a2.x, 16);  ahi[2] = __funnelshift_r(a2.x, a2.y, 16);
  alo[3] = a3.x;                            ahi[3] = a3.y;
  blo[0] = __funnelshift_r(b0.x, b0.y, 16); bhi[0] = __funnelshift_r(b0.y, b0x, 16);
  blo[1] = b1l;                             bhi[1] = b1h;
  blo[2] = __funnelshift_r(b2x, b2.x, 16);  bhi[2] = __funnelshift_r(b2.x, b2.y, 16);
  blo[3] = b3.x;                            bhi[3] = b3.y;
  uint64_t fA[4], fB[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float a = half_bits_to_float(dA[j]), b = half_bits_to_float(dB[j]);
    fA[j] = f2_pack(a, a);
    fB[j] = f2_pack(b, b);
  }
  const uint64_t unbias = f2_pack(-12582912.f, -12582912.f);
#pragma unroll
  for (int c = 0; c < NCS; ++c) {
    uint64_t tmpA = 0ull, tmpB = 0ull;     // (row g, columns 2t, 2t+1) and (row g+8, ...)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int d[4];
      mma_s8_16832(d, alo[j], blo[j], ahi[j], bhi[j], xb[c][j].x, xb[c][j].y, kQ8Magic);
      // |sum| <= 32 * 128 * 127 < 2^22, so the biased word is an exact float
      tmpA = f2_fma(fA[j], f2_add(f2_pack_bits(d[0], d[1]), unbias), tmpA);
      tmpB = f2_fma(fB[j], f2_add(f2_pack_bits(d[2], d[3]), unbias), tmpB);
    }
    const uint64_t s01 = f2_pack_bits((int)sxv[c].x, (int)sxv[c].y);
    uint64_t accA = f2_pack(acc[c][0], acc[c][1]), accB = f2_pack(acc[c][2], acc[c][3]);
    accA = f2_fma(tmpA, s01, accA);
    accB = f2_fma(tmpB, s01, accB);
    f2_unpack(accA, acc[c][0], acc[c][1]);
    f2_unpack(accB, acc[c][2], acc[c][3]);
  }
}

// ---- Q4_K: one super-block (256 weights) x 16 weight rows x NCS column sets ---------------------------
// y = d * sum_j sc_j * (q_j . x_j) - dmin * sum_j m_j * sum(x_j) over the eight 32-element sub-blocks j.  The
// 4-bit codes enter the integer MMA as bytes 0..15 (a mask and a shift, no conversion); the 6-bit sub-block
// scales multiply the integer block sums with integer multiply-adds, so one conversion to float per output
// serves the whole super-block; the minima meet the staged sub-block sums of the activations in two more MMAs
// (k = sub-block index).  Nibble bytes 32c..32c+31 hold sub-block 2c in their low and 2c+1 in their high
// nibbles; lane t owns bytes 8t..8t+7 of each 32-byte chunk.
//   pa, pb : shared addresses of the super-block in rows g and g+8, plus 8t;  da, db : the same without 8t
//   xq     : shared address of staged column g at this group's first element, plus 8t
//   sx     : shared address of this group's step-table row, plus 8t bytes (columns 2t, 2t+1)
//   xs     : shared address of this group's sub-block sums for column g, plus 4 (t & 1)
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void mma_s8_16832_acc(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NCS>
__device__ __forceinline__ void q4k_group(float (&acc)[NCS][4], uint32_t pa, uint32_t pb, uint32_t da, uint32_t db,
                                          uint32_t xq, uint32_t cs_stride, uint32_t sx, uint32_t xs,
                                          uint32_t xs_cs_stride, int t) {
  // ---- all shared loads first ----
  const uint4 hA = lds128(da), hB = lds128(db);     // {d | dmin, 12 bytes of 6-bit scales and minima}
  uint2 qA[4], qB[4];
  qA[0] = lds64<16>(pa); qA[1] = lds64<48>(pa); qA[2] = lds64<80>(pa); qA[3] = lds64<112>(pa);
  qB[0] = lds64<16>(pb); qB[1] = lds64<48>(pb); qB[2] = lds64<80>(pb); qB[3] = lds64<112>(pb);
  uint2 xb[NCS][8];
  uint2 sxv[NCS];
  uint32_t xsa[NCS], xsb[NCS];
#pragma unroll
  for (int c = 0; c < NCS; ++c) {
    const uint32_t xc = xq + c * cs_stride;
    xb[c][0] = lds64<0>(xc);   xb[c][1] = lds64<32>(xc);  xb[c][2] = lds64<64>(xc);  xb[c][3] = lds64<96>(xc);
    xb[c][4] = lds64<128>(xc); xb[c][5] = lds64<160>(xc); xb[c][6] = lds64<192>(xc); xb[c][7] = lds64<224>(xc);
    sxv[c] = lds64(sx + 32u * c);
    xsa[c] = lds32<0>(xs + c * xs_cs_stride);
    xsb[c] = lds32<8>(xs + c * xs_cs_stride);
  }
  // ---- 6-bit scales and minima, four to a word (sub-blocks 0-3 and 4-7) ----
  uint32_t scA[2], scB[2], mnA[2], mnB[2];
  scA[0] = hA.y & 0x3F3F3F3Fu; mnA[0] = hA.z & 0x3F3F3F3Fu;
  scA[1] = (hA.w & 0x0F0F0F0Fu) | ((hA.y >> 2) & 0x30303030u);
  mnA[1] = ((hA.w >> 4) & 0x0F0F0F0Fu) | ((hA.z >> 2) & 0x30303030u);
  scB[0] = hB.y & 0x3F3F3F3Fu; mnB[0] = hB.z & 0x3F3F3F3Fu;
  scB[1] = (hB.w & 0x0F0F0F0Fu) | ((hB.y >> 2) & 0x30303030u);
  mnB[1] = ((hB.w >> 4) & 0x0F0F0F0Fu) | ((hB.z >> 2) & 0x30303030u);
  // ---- nibbles to bytes ----
  uint32_t aL[4][2], aH[4][2], bL[4][2], bH[4][2];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    aL[c][0] = qA[c].x & 0x0F0F0F0Fu; aL[c][1] = qA[c].y & 0x0F0F0F0Fu;
    aH[c][0] = (qA[c].x >> 4) & 0x0F0F0F0Fu; aH[c][1] = (qA[c].y >> 4) & 0x0F0F0F0Fu;
    bL[c][0] = qB[c].x & 0x0F0F0F0Fu; bL[c][1] = qB[c].y & 0x0F0F0F0Fu;
    bH[c][0] = (qB[c].x >> 4) & 0x0F0F0F0Fu; bH[c][1] = (qB[c].y >> 4) & 0x0F0F0F0Fu;
  }
  const float dA = half_bits_to_float(hA.x), nA = half_bits_to_float(hA.x >> 16);
  const float dB = half_bits_to_float(hB.x), nB = half_bits_to_float(hB.x >> 16);
  // the minima as the A operand of the sub-block-sum MMAs: k = sub-block index (8 of the 32 k slots used)
  const uint32_t mA = t == 0 ? mnA[0] : (t == 1 ? mnA[1] : 0u);
  const uint32_t mB = t == 0 ? mnB[0] : (t == 1 ? mnB[1] : 0u);
#pragma unroll
  for (int c = 0; c < NCS; ++c) {
    int isum[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int ch = j >> 1;
      int d[4];
      if (j & 1) mma_s8_16832(d, aH[ch][0], bH[ch][0], aH[ch][1], bH[ch][1], xb[c][j].x, xb[c][j].y, 0);
      else       mma_s8_16832(d, aL[ch][0], bL[ch][0], aL[ch][1], bL[ch][1], xb[c][j].x, xb[c][j].y, 0);
      const int sa = (int)((scA[j >> 2] >> (8 * (j & 3))) & 0xFFu);
      const int sb = (int)((scB[j >> 2] >> (8 * (j & 3))) & 0xFFu);
      isum[0] += sa * d[0];
      isum[1] += sa * d[1];
      isum[2] += sb * d[2];
      isum[3] += sb * d[3];
    }
    // |isum| <= 8 * 63 * 32 * 15 * 128 < 2^31
    int ma[4] = {0, 0, 0, 0}, mb[4] = {0, 0, 0, 0};
    mma_s8_16832_acc(ma, mA, mB, 0u, 0u, xsa[c], 0u);
    mma_s8_16832_acc(mb, mA, mB, 0u, 0u, xsb[c], 0u);
    const float s0 = __uint_as_float(sxv[c].x), s1 = __uint_as_float(sxv[c].y);
    const float v0 = dA * (float)isum[0] - nA * (float)(32 * ma[0] + mb[0]);
    const float v1 = dA * (float)isum[1] - nA * (float)(32 * ma[1] + mb[1]);
    const float v2 = dB * (float)isum[2] - nB * (float)(32 * ma[2] + mb[2]);
    const float v3 = dB * (float)isum[3] - nB * (float)(32 * ma[3] + mb[3]);
    acc[c][0] = fmaf(v0, s0, acc[c][0]);
    acc[c][1] = fmaf(v1, s1, acc[c][1]);
    acc[c][2] = fmaf(v2, s0, acc[c][2]);
    acc[c][3] = fmaf(v3, s1, acc[c][3]);
  }
}

// ---- the kernel ------------------------------------------------------------------------------------
// NCS = column sets per block: 1 when every work item has at most 4 activation rows (columns 0-3 hold the
// leading terms, 4-7 the remainders), 2 for up to 8 rows (set 0 = leading terms, set 1 = remainders).
template <int FMT, int NCS>
__global__ void __launch_bounds__(kQ8Threads, 1) gemv_int8_kernel(const GemvParams p, const Q8Layout lay) {
  using T = I8Traits<FMT>;
  constexpr int WK = kQ8Warps;
  constexpr int RT = kQ8RT;
  constexpr int KC = T::KC;
  const int NSTAGE = lay.nstage;
  extern __shared__ __align__(128) uint8_t smem[];

  pdl_launch_dependents();
  if (p.tiles != nullptr) pdl_wait();    // the item list itself comes from the previous kernel
  const int n_rt = (p.n + RT - 1) / RT;
  const int n_y = p.tiles != nullptr ? p.tile_count[0] : (p.m + 7) / 8;
  const int total = n_y * n_rt;
  // Split K: neighbouring CTAs take the K slices of one item, so each keeps only its slice of the activations
  // staged (once, for every item it meets) and the slices of an item finish at about the same time.
  const int S = lay.kslices;
  const int R = gridDim.x / S;                 // item streams
  const int r0 = blockIdx.x / S;
  const int slice = blockIdx.x - r0 * S;
  // Item walk: dense calls stride through the items (neighbouring CTAs read neighbouring rows); expert-indexed
  // calls take a contiguous run each, so consecutive items of a CTA share their activation rows (one expert
  // tile) and are staged once instead of once per item.
  const bool runs = p.tiles != nullptr;
  const int per = runs ? (total + R - 1) / R : 0;
  const int w_begin = runs ? r0 * per : r0;
  const int w_end = runs ? min(total, w_begin + per) : total;
  const int w_step = runs ? 1 : R;
  if (r0 >= R || w_begin >= w_end) return;
  const int k_lo = min(p.k, slice * lay.slice_k), k_hi = min(p.k, k_lo + lay.slice_k);
  const int nchunk = (k_hi - k_lo + KC - 1) / KC;     // stages of this slice; the last one may be short
  const int kXK = lay.xk;
  const int xk_sub = lay.xk_sub;
  const int n_super = (k_hi - k_lo + kXK - 1) / kXK;

  uint64_t* full = reinterpret_cast<uint64_t*>(smem + lay.off_bar);
  uint64_t* empty = full + kQ8MaxStages;
  uint64_t* red_full = empty + kQ8MaxStages;   // [2] partial sums of an item are all written
  uint64_t* red_free = red_full + 2;           // [2] ... and have been consumed
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < NSTAGE; ++s) {
      mbar_init(&full[s], kQ8Producers);
      mbar_init(&empty[s], WK);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&red_full[b], WK);
      mbar_init(&red_free[b], 1);
    }
    fence_barrier_init();
  }
  // zero the staged activations once: columns beyond an item's row count must read as zero
  for (int i = tid; i < lay.x_bytes / 16; i += kQ8Threads)
    reinterpret_cast<uint4*>(smem + lay.off_x)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();

  const int64_t row_bytes = T::row_bytes(p.k);

  if (warp >= WK && warp < WK + kQ8Producers) {
    // ================= producer warps: stream weight row segments ================================
    const int pw = warp - WK;
    constexpr int RPP = RT / kQ8Producers;      // rows per producer warp
    uint32_t spin = kQ8Spin;
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    int s = 0, round = 0;
    for (int w = w_begin; w < w_end; w += w_step) {
      const WorkItem wi = get_item<RT>(p, w, n_rt);
      if (wi.nrows <= 0) continue;
      const int rows_valid = min(RT, p.n - wi.n0);
      const int my_rows = max(0, min(RPP, rows_valid - pw * RPP));
      for (int chunk = 0; chunk < nchunk; ++chunk) {
        const int kc_len = min(KC, k_hi - (k_lo + chunk * KC));
        const uint32_t bytes = (uint32_t)T::row_bytes(kc_len);
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
                                T::row_bytes(k_lo + chunk * KC);
          if (lane == 0) mbar_arrive_expect_tx(&full[s], bytes * (uint32_t)my_rows);
          __syncwarp();
          uint8_t* dst = smem + s * T::STAGE_BYTES + pw * RPP * T::PITCH;
          if (lane < my_rows)
            bulk_g2s_hint(dst + lane * T::PITCH, wsrc + (int64_t)lane * row_bytes, bytes, &full[s], policy);
          if (++s == NSTAGE) {
            s = 0;
            ++round;
          }
        }
      }
    }
  }

  float* red = reinterpret_cast<float*>(smem + lay.off_red);   // [2 buffers][banks][warps][4][32]
  const int g = lane >> 2, t = lane & 3;

  if (warp == WK + kQ8Producers) {
    // ================= reducing warp: adds the K-split partial sums in warp order and writes ======
    pdl_wait();
    uint32_t spin = kQ8Spin;
    int item = 0;
    for (int w = w_begin; w < w_end; w += w_step) {
      const WorkItem wi = get_item<RT>(p, w, n_rt);
      if (wi.nrows <= 0) continue;
      const int rb = item & 1;
      const float* rbuf = red + rb * (p.n_banks * WK * 4 * 32);
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
            for (int j = 0; j < WK; ++j) sum += rbuf[((b * WK + j) * 4 + i) * 32 + lane];
            if (NCS == 1 && FMT == HQ_FMT_FP8_BLOCK) {
              // two-row layout of the three e4m3 terms: columns 2, 3 and 4, 5 sit one and two lanes further on
              const float s1 = __shfl_down_sync(0xffffffffu, sum, 1), s2 = __shfl_down_sync(0xffffffffu, sum, 2);
              sum += s1 + s2;
            } else if (NCS == 1) {
              // four-row layout: the remainder columns 4..7 sit two lanes further on
              sum += __shfl_down_sync(0xffffffffu, sum, 2);
            }
            v[b][i] = sum;
          }
        }
      __syncwarp();
      if (lane == 0) mbar_arrive(&red_free[rb]);
      if (S > 1) {
        // split K: the slice sums of an item meet in global memory and are added when the kernel ends
        const int nb = p.n_banks;
        float* mine = lay.partials + ((int64_t)w * S + slice) * (nb * 128);
#pragma unroll
        for (int b = 0; b < 2; ++b)
          if (b < nb) {
#pragma unroll
            for (int i = 0; i < 4; ++i) __stcg(mine + (b * 4 + i) * 32 + lane, v[b][i]);
          }
      } else {
        gemv_store_item(p, wi, g, 2 * t, !failed && (NCS > 1 || t < (FMT == HQ_FMT_FP8_BLOCK ? 1 : 2)), v);
      }
      ++item;
    }
  }

  if (warp < WK) {
  pdl_wait();
  // ================= consumer warps ================================================================
  uint8_t* xq = smem + lay.off_x;
  float* sx = reinterpret_cast<float*>(smem + lay.off_sx);
  const int xpitch = lay.xpitch;
  const int ncols = lay.ncols;
  const uint32_t cs_stride = 8u * (uint32_t)xpitch;
  // terms an activation is split into, and the column distance between them: two int8 terms half the staged
  // columns apart, or three e4m3 terms 2 columns apart (block-FP8 runs with one column set, at most two rows)
  constexpr int kTerms = FMT == HQ_FMT_FP8_BLOCK ? 3 : 2;
  const int tstride = FMT == HQ_FMT_FP8_BLOCK ? 2 : (ncols >> 1);
  // this lane's staged column (column g of every set), its group within a stage, its scale-table columns
  const uint32_t xq_lane = smem_u32(xq) + (uint32_t)g * xpitch + (uint32_t)T::GK * warp + 8u * t;
  const uint32_t sx_lane = smem_u32(sx) + (uint32_t)warp * ncols * 4u + 8u * t;
  uint8_t* xsub = smem + lay.off_xs;     // Q4_K: sub-block sums [group][column][16]
  const uint32_t xs_lane = smem_u32(xsub) + ((uint32_t)warp * ncols + g) * 16u + 4u * (t & 1);

  Q8XPrefetch pf;
  bool pf_valid = false;
  int staged_y = -1;        // activation rows currently staged (valid when n_super == 1)
  int staged_rows = 0;
  {
    const WorkItem w0 = get_item<RT>(p, w_begin, n_rt);
    if (w0.nrows > 0) {
      q8_x_prefetch(pf, p, w0.row0, w0.nrows, k_lo, min(xk_sub, k_hi - k_lo), tid);
      pf_valid = true;
    }
  }

  uint32_t spin = kQ8Spin;
  int s = 0, item = 0;
  uint32_t phase = 0;
  for (int w = w_begin; w < w_end; w += w_step) {
    const WorkItem wi = get_item<RT>(p, w, n_rt);
    if (wi.nrows <= 0) continue;
    float acc[2][NCS][4];
#pragma unroll
    for (int b = 0; b < 2; ++b)
#pragma unroll
      for (int c = 0; c < NCS; ++c)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[b][c][i] = 0.f;
    for (int sc = 0; sc < n_super; ++sc) {
      const int k_base = k_lo + sc * kXK;
      const int k_len = min(kXK, k_hi - k_base);
      if (n_super > 1 || wi.y != staged_y) {
        // ---- stage this epoch's activations (all consumer warps) ----------------------------------
        if (!pf_valid) q8_x_prefetch(pf, p, wi.row0, wi.nrows, k_base, min(xk_sub, k_len), tid);
        named_bar_sync(1, kQ8Consumers);       // everyone is done reading the previous epoch
        // columns left over from an earlier item with more rows than this one must read as zero
        if (staged_rows > wi.nrows) {
          const int per_col = xpitch / 16;
          const int stale = staged_rows - wi.nrows;
          for (int i = tid; i < kTerms * stale * per_col; i += kQ8Consumers) {
            const int term = i / (stale * per_col);
            const int j = i - term * (stale * per_col);
            const int col = wi.nrows + j / per_col + term * tstride;
            reinterpret_cast<uint4*>(xq + col * xpitch)[j % per_col] = make_uint4(0, 0, 0, 0);
          }
        }
        staged_rows = wi.nrows;
        auto commit = [&](int len, int sub) {
          if (FMT == HQ_FMT_FP8_BLOCK)
            fp8_x_commit(pf, p, wi.nrows, len, tid, xq + sub, xpitch, sx + (sub / T::GK) * ncols, ncols, tstride);
          else
            q8_x_commit<T::GK, T::kSubSums>(pf, p, wi.nrows, len, tid, xq + sub, xpitch, sx + (sub / T::GK) * ncols,
                                            xsub + (sub / T::GK) * ncols * 16, ncols);
        };
        commit(min(xk_sub, k_len), 0);
        for (int sub = xk_sub; sub < k_len; sub += xk_sub) {   // wide input: the rest is fetched now
          q8_x_prefetch(pf, p, wi.row0, wi.nrows, k_base + sub, min(xk_sub, k_len - sub), tid);
          commit(min(xk_sub, k_len - sub), sub);
        }
        staged_y = wi.y;
        pf_valid = false;
        // fetch the next epoch's activations while this one is being consumed
        if (sc + 1 < n_super) {
          q8_x_prefetch(pf, p, wi.row0, wi.nrows, k_base + kXK, min(xk_sub, k_hi - k_base - kXK), tid);
          pf_valid = true;
        } else if (w + w_step < w_end) {
          const WorkItem nx = get_item<RT>(p, w + w_step, n_rt);
          if (nx.nrows > 0 && (n_super > 1 || nx.y != wi.y)) {
            q8_x_prefetch(pf, p, nx.row0, nx.nrows, k_lo, min(xk_sub, k_hi - k_lo), tid);
            pf_valid = true;
          }
        }
        named_bar_sync(1, kQ8Consumers);
      }
      // stages of this epoch, counted from the slice's first column (an epoch is a whole number of stages)
      const int c0 = (k_base - k_lo) / KC, c1 = (k_base - k_lo + k_len + KC - 1) / KC;
      for (int chunk = c0; chunk < c1; ++chunk) {
        const int k_chunk = k_lo + chunk * KC;
        const int ngroups = min(KC, k_hi - k_chunk) / T::GK;   // groups in this stage
        const uint32_t kx = (uint32_t)(k_chunk - k_base);      // offset of the stage inside the staged activations
#pragma unroll
        for (int bank = 0; bank < 2; ++bank) {
          if (bank >= p.n_banks) break;
          // block-FP8: the 128 x 128 weight-block scales of this warp's groups, fetched before the wait for the stage
          float wsv[kQ8GroupsPerWarp];
          if (FMT == HQ_FMT_FP8_BLOCK) {
            const float* fsc = reinterpret_cast<const float*>(bank == 0 ? p.scales : p.scales_up) +
                               (int64_t)wi.expert * p.scale_expert_stride +
                               (int64_t)(wi.n0 / 128) * ((p.k + 127) / 128) + k_chunk / 128;
#pragma unroll
            for (int gi = 0; gi < kQ8GroupsPerWarp; ++gi) {
              const int grp = warp + gi * WK;
              wsv[gi] = grp < ngroups ? __ldg(fsc + grp) : 0.f;
            }
          }
          if (!mbar_wait(&full[s], phase, spin)) {
            // bounded wait ran out: flag it and carry on (every warp still reaches every barrier)
            if (lane == 0) report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 200 + s);
            spin = 1;
          }
#pragma unroll
          for (int gi = 0; gi < kQ8GroupsPerWarp; ++gi) {
            const int grp = warp + gi * WK;
            if (grp < ngroups) {
              const uint32_t da = smem_u32(smem + s * T::STAGE_BYTES) + (uint32_t)g * T::PITCH +
                                  (uint32_t)T::GROUP_BYTES * grp;
              const uint32_t db = da + 8u * T::PITCH;
              const uint32_t gq = kx / T::GK + gi * WK;      // group index inside the staged activations, less `warp`
              if (FMT == HQ_FMT_Q8_0) {
                q8_group<NCS>(acc[bank], da + 8u * t, db + 8u * t, da, db, xq_lane + gq * T::GK, cs_stride,
                              sx_lane + gq * (uint32_t)ncols * 4u);
              } else if (FMT == HQ_FMT_FP8_BLOCK) {
                fp8_group<NCS>(acc[bank], da + 8u * t, db + 8u * t, xq_lane + gq * T::GK, cs_stride,
                               sx_lane + gq * (uint32_t)ncols * 4u, wsv[gi]);
              } else {
                q4k_group<NCS>(acc[bank], da + 8u * t, db + 8u * t, da, db, xq_lane + gq * T::GK, cs_stride,
                               sx_lane + gq * (uint32_t)ncols * 4u, xs_lane + gq * (uint32_t)ncols * 16u, 128u, t);
              }
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
    float* rbuf = red + rb * (p.n_banks * WK * 4 * 32);
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
        for (int i = 0; i < 4; ++i)
        {
          float sum = acc[b][0][i];
#pragma unroll
          for (int c = 1; c < NCS; ++c) sum += acc[b][c][i];
          rbuf[((b * WK + warp) * 4 + i) * 32 + lane] = sum;
        }
      }
    __syncwarp();
    if (lane == 0) mbar_arrive(&red_full[rb]);
    ++item;
  }
  }   // consumer warps

  if (S > 1) {
    // ---- split K: whichever CTA of an item stream finishes last adds the slice sums of the stream's items, in
    // slice order (so the result does not depend on who that is), and leaves the counter at zero ---------------
    __shared__ int last_flag;
    pdl_wait();
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      const int old = atomicAdd(lay.counters + r0, 1);
      last_flag = old == S - 1;
      if (last_flag) lay.counters[r0] = 0;
    }
    __syncthreads();
    if (last_flag) {
      __threadfence();
      const int nb = p.n_banks;
      int idx = 0;
      for (int w = w_begin; w < w_end; w += w_step, ++idx) {
        if (idx % (kQ8Threads / 32) != warp) continue;
        const WorkItem wi = get_item<RT>(p, w, n_rt);
        if (wi.nrows <= 0) continue;
        const float* all = lay.partials + (int64_t)w * S * (nb * 128);
        float v[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int b = 0; b < 2; ++b)
          if (b < nb) {
            // every load of a bank is issued before the first sum needs one (at most eight slices)
            float part[8][4];
#pragma unroll
            for (int sl = 0; sl < 8; ++sl)
#pragma unroll
              for (int i = 0; i < 4; ++i)
                part[sl][i] = sl < S ? __ldcg(all + (sl * nb + b) * 128 + i * 32 + lane) : 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              float sum = 0.f;
#pragma unroll
              for (int sl = 0; sl < 8; ++sl) sum += part[sl][i];   // slice order; absent slices add +0
              v[b][i] = sum;
            }
          }
        gemv_store_item(p, wi, g, 2 * t, NCS > 1 || t < (FMT == HQ_FMT_FP8_BLOCK ? 1 : 2), v);
      }
    }
  }
}

// ---- host launcher -----------------------------------------------------------------------------
// Split K when K is too long for a CTA to keep its activations staged beside at least four ring stages: a CTA
// that covers the whole K would then have to stage them again for every item.  The slices are equal runs of
// 256-column steps.  Among two to eight slices the plan takes the one with the smallest estimated time, in
// units of one column streamed for one item: the items of the busiest stream times (columns of a slice + a
// fixed cost per item), plus the staging of the slice's activations before the first item.  Both constants are
// fitted to measurements of 14336-column layers with 4096 rows (four slices: 17 us, two: 18 us, seven: 21 us).
// Shorter K stays unsplit -- the meeting of the slice sums costs a few microseconds.
struct Q8Split {
  int kslices, slice_k;
  int64_t counter_bytes, bytes;
};
constexpr int kQ8ItemCostK = 2048;   // fixed cost of an item, in columns
constexpr int kQ8StageCost = 2;       // staging a slice's activations, per column, against streaming it for one item
template <int FMT>
static int q8_fixed_bytes(int ncols, int xk, int n_banks) {
  using T = I8Traits<FMT>;
  return ncols * (xk + 32) + (xk / T::GK) * ncols * 4 + (T::kSubSums ? (xk / T::GK) * ncols * 16 : 0) +
         2 * n_banks * kQ8Warps * 4 * 32 * 4 + (2 * kQ8MaxStages + 4) * 8 + 16;
}
template <int FMT>
static int q8_ring_stages(int ncols, int xk, int n_banks) {
  return (kQ8SmemBudget - q8_fixed_bytes<FMT>(ncols, xk, n_banks)) / I8Traits<FMT>::STAGE_BYTES;
}
template <int FMT>
static Q8Split q8_split_plan(int64_t n, int64_t k, int64_t n_y, int n_banks, bool expert_indexed, int ncols) {
  constexpr int KC = I8Traits<FMT>::KC;
  Q8Split sp{};
  const int nchunk = (int)((k + KC - 1) / KC);
  const int64_t items = n_y * ((n + kQ8RT - 1) / kQ8RT);
  sp.kslices = 1;
  sp.slice_k = nchunk * KC;
  if (expert_indexed || nchunk < 2 || q8_ring_stages<FMT>(ncols, nchunk * KC, n_banks) >= 4) return sp;
  const int sms = sm_count();
  int64_t best = -1;
  for (int s = 2; s <= 8; ++s) {
    const int slice_k = (int)(((k + s - 1) / s + 255) / 256 * 256);
    const int slices = (int)((k + slice_k - 1) / slice_k);
    if (slices != s && s != 8) continue;                 // the same plan as a smaller s
    const bool fits = q8_ring_stages<FMT>(ncols, (slice_k + KC - 1) / KC * KC, n_banks) >= 4;
    if (!fits && s != 8) continue;                       // eight slices are the fallback whatever they leave
    const int64_t streams = sms / slices > 0 ? sms / slices : 1;
    const int64_t busiest = (items + streams - 1) / streams;
    const int64_t cost = busiest * (slice_k + kQ8ItemCostK) + kQ8StageCost * slice_k;
    if (best < 0 || cost < best) {
      best = cost;
      sp.kslices = slices;
      sp.slice_k = slice_k;
    }
  }
  sp.counter_bytes = 1024;     // one arrival counter per item stream (at most one stream per SM)
  sp.bytes = sp.counter_bytes + items * sp.kslices * n_banks * 512;
  return sp;
}

int64_t gemv_int8_workspace_bytes(int format, int64_t n, int64_t k, int64_t m) {
  if (format == HQ_FMT_Q8_0) return q8_split_plan<HQ_FMT_Q8_0>(n, k, (m + 7) / 8, 1, false, m > 4 ? 16 : 8).bytes;
  if (format == HQ_FMT_Q4_K) return q8_split_plan<HQ_FMT_Q4_K>(n, k, (m + 7) / 8, 1, false, m > 4 ? 16 : 8).bytes;
  if (format == HQ_FMT_FP8_BLOCK && k % 256 == 0 && n % 16 == 0 && m <= 2)
    return q8_split_plan<HQ_FMT_FP8_BLOCK>(n, k, 1, 1, false, 8).bytes;
  return 0;
}

template <int FMT, int NCS>
static int32_t launch_q8_cfg(const GemvParams& p, int n_y_max, int max_rows, cudaStream_t stream) {
  using T = I8Traits<FMT>;
  Q8Layout lay{};
  lay.ncols = 8 * NCS;
  Q8Split sp = q8_split_plan<FMT>(p.n, p.k, n_y_max, p.n_banks, p.tiles != nullptr, lay.ncols);
  if (sp.kslices > 1 && (p.workspace == nullptr || p.workspace_bytes < sp.bytes)) {
    sp.kslices = 1;                      // no scratch from the caller: every CTA covers the whole K
    sp.slice_k = (int)((p.k + T::KC - 1) / T::KC) * T::KC;
  }
  lay.kslices = sp.kslices;
  lay.slice_k = sp.slice_k;
  if (sp.kslices > 1) {
    lay.counters = reinterpret_cast<int32_t*>(p.workspace);
    lay.partials = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p.workspace) + sp.counter_bytes);
  }
  // Shared-memory plan: stage as many activation columns as leave at least four ring stages (the CTA's whole
  // K range when it fits -- then a persistent CTA quantizes its activations once), give every remaining byte
  // to the ring.
  const int esz = dtype_size(p.x_dtype);
  const int k_round = (sp.slice_k + T::KC - 1) / T::KC * T::KC;
  const int candidates[3] = {k_round, 8192 < k_round ? 8192 : k_round, 4096 < k_round ? 4096 : k_round};
  for (int c = 0; c < 3; ++c) {
    lay.xk = candidates[c];
    lay.xpitch = lay.xk + 32;
    lay.x_bytes = lay.ncols * lay.xpitch;
    const int sx_bytes = (lay.xk / T::GK) * lay.ncols * 4;
    const int xs_bytes = T::kSubSums ? (lay.xk / T::GK) * lay.ncols * 16 : 0;
    const int red_bytes = 2 * p.n_banks * kQ8Warps * 4 * 32 * 4;
    const int bar_bytes = (2 * kQ8MaxStages + 4) * 8 + 16;
    const int fixed = lay.x_bytes + sx_bytes + xs_bytes + red_bytes + bar_bytes;
    int nst = (kQ8SmemBudget - fixed) / T::STAGE_BYTES;
    if (nst > kQ8MaxStages) nst = kQ8MaxStages;
    lay.nstage = nst;
    lay.off_x = nst * T::STAGE_BYTES;
    lay.off_sx = lay.off_x + lay.x_bytes;
    lay.off_xs = lay.off_sx + sx_bytes;
    lay.off_red = lay.off_xs + xs_bytes;
    lay.off_bar = lay.off_red + red_bytes;
    lay.total = lay.off_bar + bar_bytes;
    if (nst >= 4) break;
  }
  if (lay.nstage < 2) return HQ_ERR_SHAPE;
  // columns one register prefetch can hold, in whole 256-column steps
  const int sub = (kQ8XGroups * kQ8Consumers * 16) / (max_rows * esz) / 256 * 256;   // 16 bytes per register
  lay.xk_sub = sub < lay.xk ? sub : lay.xk;
  auto kern = gemv_int8_kernel<FMT, NCS>;
  static bool attr_done[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return HQ_ERR_CUDA;
  if (dev < 64 && !attr_done[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kQ8SmemBudget) != cudaSuccess)
      return HQ_ERR_CUDA;
    attr_done[dev] = true;
  }
  const int64_t items = (int64_t)n_y_max * ((p.n + kQ8RT - 1) / kQ8RT);
  int64_t streams = sm_count() / sp.kslices;
  if (streams < 1) streams = 1;
  if (streams > items) streams = items;
  const int64_t grid = streams * sp.kslices;
  if (grid <= 0) return HQ_OK;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kQ8Threads);
  cfg.dynamicSmemBytes = (size_t)lay.total;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, p, lay) == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

int32_t launch_gemv_int8(const GemvParams& p, int n_y_max, int max_rows, cudaStream_t stream) {
  if (p.k % 256 != 0) return HQ_ERR_SHAPE;   // row segments must stay 16-byte aligned for the bulk copies
  if (p.format == HQ_FMT_FP8_BLOCK && p.n % 16 != 0) return HQ_ERR_SHAPE;   // a 16-row item shares one weight-block scale
  if (p.format == HQ_FMT_Q8_0)
    return max_rows > 4 ? launch_q8_cfg<HQ_FMT_Q8_0, 2>(p, n_y_max, max_rows, stream)
                        : launch_q8_cfg<HQ_FMT_Q8_0, 1>(p, n_y_max, max_rows, stream);
  if (p.format == HQ_FMT_Q4_K)
    return max_rows > 4 ? launch_q8_cfg<HQ_FMT_Q4_K, 2>(p, n_y_max, max_rows, stream)
                        : launch_q8_cfg<HQ_FMT_Q4_K, 1>(p, n_y_max, max_rows, stream);
  // block-FP8: three e4m3 terms per activation, so one column set holds two rows.  More rows would take three
  // MMAs per block, and the warp-level FP8 MMA is slow enough on this part that the f16 decoder then wins
  // (measured 2.0 against 3.7 TB/s at 4 rows): the caller sends those there.
  if (p.format == HQ_FMT_FP8_BLOCK && max_rows <= 2) return launch_q8_cfg<HQ_FMT_FP8_BLOCK, 1>(p, n_y_max, max_rows, stream);
  return HQ_ERR_FORMAT;
}

}  // namespace hq
