// Decode-regime quantized mat-vec (1..8 activation rows per work item), dense
// and expert-indexed, for Q8_0, Q4_K, block-FP8 and MXFP4 weights.
//
// HBM-bound: every weight byte is read once, straight from the reference's
// device layout.  One CTA owns a tile of RT = 16*WR output rows and walks K in
// chunks.  A producer warp streams each chunk's row segments into a shared
// memory ring with bulk async copies (TMA, mbarrier completion); eight consumer
// warps decode the blocks in registers into f16 MMA fragments -- integer codes
// become f16 *subnormals* with a couple of logic ops, the power-of-two factor
// is folded into the block scale -- and multiply them against the (<= 8)
// activation rows with m16n8k16 warp MMAs, f32 accumulation, one scale FMA per
// 32-element block.  Partial sums of warps that split K are reduced through
// shared memory in a fixed order, so results are bit-reproducible.
//
// Algorithmic bytes per launch: N*K*bits/8 (weights) + M*K*sizeof(x) + M*N*sizeof(y).
#include "hq_common.cuh"
#include "hq_kernels.h"

namespace hq {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kGemvThreads = kConsumerThreads + 32;
constexpr uint32_t kSpinLimit = 1u << 22;

// ---- per-format geometry ----------------------------------------------------
template <int FMT>
struct FmtTraits;
template <>
struct FmtTraits<HQ_FMT_Q8_0> {
  static constexpr int kGran = 256;  // K granularity that keeps row segments 16-byte aligned
  static constexpr bool kPermX = true;
  static constexpr bool kNeedXsum = true;
  __host__ __device__ static constexpr int seg_bytes(int kc) { return kc / 32 * 34; }
  __host__ __device__ static int64_t row_bytes(int64_t k) { return k / 32 * 34; }
};
template <>
struct FmtTraits<HQ_FMT_Q4_K> {
  static constexpr int kGran = 256;
  static constexpr bool kPermX = true;
  static constexpr bool kNeedXsum = true;
  __host__ __device__ static constexpr int seg_bytes(int kc) { return kc / 256 * 144; }
  __host__ __device__ static int64_t row_bytes(int64_t k) { return k / 256 * 144; }
};
template <>
struct FmtTraits<HQ_FMT_FP8_BLOCK> {
  static constexpr int kGran = 128;
  static constexpr bool kPermX = false;
  static constexpr bool kNeedXsum = false;
  __host__ __device__ static constexpr int seg_bytes(int kc) { return kc; }
  __host__ __device__ static int64_t row_bytes(int64_t k) { return k; }
};
template <>
struct FmtTraits<HQ_FMT_MXFP4> {
  static constexpr int kGran = 32;
  static constexpr bool kPermX = false;
  static constexpr bool kNeedXsum = false;
  __host__ __device__ static constexpr int seg_bytes(int kc) { return kc / 2; }
  __host__ __device__ static int64_t row_bytes(int64_t k) { return k / 2; }
};

__host__ __device__ constexpr int seg_pitch(int seg) {
  // rows of a stage sit `pitch` bytes apart; pitch/4 == 4 (mod 8) spreads the 8 row
  // groups of a warp over all 32 banks for the 32-bit fragment loads
  return ((seg / 4) % 8 == 4) ? seg : seg + 16;
}

template <int FMT, int WR, int KC, int NSTAGE>
struct GemvSmem {
  static constexpr int RT = 16 * WR;
  static constexpr int SEG = FmtTraits<FMT>::seg_bytes(KC);
  static constexpr int PITCH = seg_pitch(SEG);
  static constexpr int STAGE_BYTES = RT * PITCH;
  static constexpr int XP = KC + 16;  // f16 elements per activation row in shared memory
  static constexpr int OFF_X = NSTAGE * STAGE_BYTES;
  static constexpr int X_BYTES = 2 * 8 * XP * 2;
  static constexpr int OFF_XSUM = OFF_X + X_BYTES;
  static constexpr int XSUM_BYTES = 2 * (KC / 32) * 8 * 4;
  static constexpr int OFF_MSC = OFF_XSUM + XSUM_BYTES;
  static constexpr int MSC_BYTES = (FMT == HQ_FMT_MXFP4) ? 2 * 2 * RT * (KC / 32) : 0;  // [buf][bank][row][block]
  static constexpr int OFF_FSC = OFF_MSC + ((MSC_BYTES + 15) / 16) * 16;
  static constexpr int FSC_BYTES = (FMT == HQ_FMT_FP8_BLOCK) ? 512 * 4 : 0;
  static constexpr int OFF_RED = OFF_FSC + FSC_BYTES;
  static constexpr int RED_BYTES = kConsumerWarps * 32 * 4 * 4 * 2;  // two banks
  static constexpr int OFF_BAR = OFF_RED + RED_BYTES;
  static constexpr int TOTAL = OFF_BAR + 2 * NSTAGE * 8 + 16;
};

// ---- activation staging -----------------------------------------------------
// Raw activation bytes are fetched one chunk ahead into registers (16 bytes per
// group), then converted to f16 and written to shared memory in fragment order.
constexpr int kMaxXGroups = 8;

struct XPrefetch {
  uint4 v[kMaxXGroups];
};

template <int KC>
__device__ __forceinline__ void x_prefetch(XPrefetch& pf, const GemvParams& p, const int32_t* x_rows, int row0,
                                           int nrows, int k0, int kc_len, int tid) {
  const int esz = dtype_size(p.x_dtype);
  const int epg = 16 / esz;              // elements per 16-byte group
  const int gpr = kc_len / epg;          // groups per activation row in this chunk
  const int ngroups = nrows * gpr;
#pragma unroll
  for (int i = 0; i < kMaxXGroups; ++i) {
    const int it = i * kConsumerThreads + tid;
    if (it < ngroups) {
      const int col = it / gpr;
      const int kk = (it - col * gpr) * epg;
      const int64_t xr = x_rows ? (int64_t)x_rows[row0 + col] : (int64_t)(row0 + col);
      const char* src = (const char*)p.x + (xr * p.x_stride + k0 + kk) * esz;
      pf.v[i] = __ldg(reinterpret_cast<const uint4*>(src));
    }
  }
}

template <bool PERM, bool XSUM, int KC>
__device__ __forceinline__ void x_commit(const XPrefetch& pf, const GemvParams& p, int nrows, int kc_len, int tid,
                                         __half* xs, float* xsum) {
  constexpr int XP = KC + 16;
  const int esz = dtype_size(p.x_dtype);
  const int epg = 16 / esz;
  const int gpr = kc_len / epg;
  const int ngroups = nrows * gpr;
  const int lpb = 32 / epg;  // lanes that share one 32-element block
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
      // round to f16 (what the MMA sees); sums below use the rounded values
      __half hv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) hv[j] = __float2half_rn(f[j]);
      if (XSUM) {
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) s += __half2float(hv[j]);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        if (lpb == 8) s += __shfl_xor_sync(0xffffffffu, s, 4);
        if (ok && (tid % lpb) == 0) xsum[(kk / 32) * 8 + col] = s;
      }
      if (ok) {
        __half* dst = xs + col * XP + kk;
        if (PERM) {  // within each group of four: order 0,2,1,3 (fragment pairs are (b0,b2),(b1,b3))
          __half t1 = hv[1]; hv[1] = hv[2]; hv[2] = t1;
          __half t5 = hv[5]; hv[5] = hv[6]; hv[6] = t5;
        }
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

// Q8_0: unit = one 32-element block (34 bytes, 2-byte aligned in the ring).
__device__ __forceinline__ void unit_q8_0(float (&acc)[4], uint32_t rowA, uint32_t rowB, uint32_t xs_g,
                                          uint32_t xsum_t, int unit, int t) {
  const uint32_t off = 34u * unit;
  const float dA = half_bits_to_float(lds16(rowA + off));
  const float dB = half_bits_to_float(lds16(rowB + off));
  const uint32_t q = off + 2u + 4u * t;
  const uint32_t al = q & ~3u;
  const uint32_t sh = (q & 3u) * 8u;
  const uint32_t a_lo = __funnelshift_r(lds32(rowA + al), lds32(rowA + al + 4), sh) ^ 0x80808080u;
  const uint32_t a_hi = __funnelshift_r(lds32(rowA + al + 16), lds32(rowA + al + 20), sh) ^ 0x80808080u;
  const uint32_t b_lo = __funnelshift_r(lds32(rowB + al), lds32(rowB + al + 4), sh) ^ 0x80808080u;
  const uint32_t b_hi = __funnelshift_r(lds32(rowB + al + 16), lds32(rowB + al + 20), sh) ^ 0x80808080u;
  float blk[4] = {0.f, 0.f, 0.f, 0.f};
  const uint32_t xo = xs_g + (32u * unit + 4u * t) * 2u;
  uint2 xb = lds64(xo);
  mma_f16_16816(blk, a_lo & 0x00FF00FFu, b_lo & 0x00FF00FFu, (a_lo >> 8) & 0x00FF00FFu, (b_lo >> 8) & 0x00FF00FFu,
                xb.x, xb.y);
  xb = lds64(xo + 32u);
  mma_f16_16816(blk, a_hi & 0x00FF00FFu, b_hi & 0x00FF00FFu, (a_hi >> 8) & 0x00FF00FFu, (b_hi >> 8) & 0x00FF00FFu,
                xb.x, xb.y);
  // codes were fed as (q+128) * 2^-24: value = d * (2^24 * blk - 128 * sum(x))
  const uint2 xs2 = lds64(xsum_t + 32u * unit);
  const float sx0 = __uint_as_float(xs2.x), sx1 = __uint_as_float(xs2.y);
  const float sA = dA * 16777216.f, sB = dB * 16777216.f;
  acc[0] = fmaf(sA, blk[0], fmaf(-128.f * dA, sx0, acc[0]));
  acc[1] = fmaf(sA, blk[1], fmaf(-128.f * dA, sx1, acc[1]));
  acc[2] = fmaf(sB, blk[2], fmaf(-128.f * dB, sx0, acc[2]));
  acc[3] = fmaf(sB, blk[3], fmaf(-128.f * dB, sx1, acc[3]));
}

// Q4_K: unit = 64 elements = sub-blocks (2c, 2c+1) of a super-block; they share 32 nibble bytes.
__device__ __forceinline__ void q4k_scale_min(uint32_t row_sb, int j, float& sc, float& mn) {
  // 12 scale bytes at +4: 6-bit (scale, min) pairs, the GGML get_scale_min_k4 packing
  const uint32_t w0 = lds32(row_sb + 4), w1 = lds32(row_sb + 8), w2 = lds32(row_sb + 12);
  uint32_t s, m;
  if (j < 4) {
    s = (w0 >> (8 * j)) & 63u;
    m = (w1 >> (8 * j)) & 63u;
  } else {
    const int jj = j - 4;
    s = ((w2 >> (8 * jj)) & 0xFu) | (((w0 >> (8 * jj + 6)) & 3u) << 4);
    m = ((w2 >> (8 * jj + 4)) & 0xFu) | (((w1 >> (8 * jj + 6)) & 3u) << 4);
  }
  sc = (float)s;
  mn = (float)m;
}

__device__ __forceinline__ void unit_q4_k(float (&acc)[4], uint32_t rowA, uint32_t rowB, uint32_t xs_g,
                                          uint32_t xsum_t, int unit, int t) {
  const int sb = unit >> 2, c = unit & 3;
  const uint32_t sbA = rowA + 144u * sb, sbB = rowB + 144u * sb;
  const uint32_t dmA = lds32(sbA), dmB = lds32(sbB);
  const float dA = half_bits_to_float(dmA), mA = half_bits_to_float(dmA >> 16);
  const float dB = half_bits_to_float(dmB), mB = half_bits_to_float(dmB >> 16);
  const uint32_t qo = 16u + 32u * c + 4u * t;
  const uint32_t a0 = lds32(sbA + qo), a1 = lds32(sbA + qo + 16);
  const uint32_t b0 = lds32(sbB + qo), b1 = lds32(sbB + qo + 16);
  const uint32_t xo = xs_g + (256u * sb + 64u * c + 4u * t) * 2u;
#pragma unroll
  for (int hi = 0; hi < 2; ++hi) {
    // low nibbles -> sub-block 2c (codes * 2^-24), high nibbles -> 2c+1 (codes * 2^-20)
    const uint32_t mask = hi ? 0x00F000F0u : 0x000F000Fu;
    float blk[4] = {0.f, 0.f, 0.f, 0.f};
    uint2 xb = lds64(xo + hi * 64u);
    mma_f16_16816(blk, a0 & mask, b0 & mask, (a0 >> 8) & mask, (b0 >> 8) & mask, xb.x, xb.y);
    xb = lds64(xo + hi * 64u + 32u);
    mma_f16_16816(blk, a1 & mask, b1 & mask, (a1 >> 8) & mask, (b1 >> 8) & mask, xb.x, xb.y);
    const int j = 2 * c + hi;
    float scA, mnA, scB, mnB;
    q4k_scale_min(sbA, j, scA, mnA);
    q4k_scale_min(sbB, j, scB, mnB);
    const float pw = hi ? 1048576.f : 16777216.f;
    const uint2 xs2 = lds64(xsum_t + 32u * (8u * sb + j));
    const float sx0 = __uint_as_float(xs2.x), sx1 = __uint_as_float(xs2.y);
    const float fA = dA * scA * pw, fB = dB * scB * pw;
    const float gA = -(mA * mnA), gB = -(mB * mnB);
    acc[0] = fmaf(fA, blk[0], fmaf(gA, sx0, acc[0]));
    acc[1] = fmaf(fA, blk[1], fmaf(gA, sx1, acc[1]));
    acc[2] = fmaf(fB, blk[2], fmaf(gB, sx0, acc[2]));
    acc[3] = fmaf(fB, blk[3], fmaf(gB, sx1, acc[3]));
  }
}

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

// block-FP8: unit = 32 elements; the 128x128 scale of the row tile is applied per unit.
__device__ __forceinline__ void unit_fp8(float (&acc)[4], uint32_t rowA, uint32_t rowB, uint32_t xs_g, int unit,
                                         int t, float scale) {
  const uint32_t qo = 32u * unit + 4u * t;
  const uint32_t a0 = lds32(rowA + qo), a1 = lds32(rowA + qo + 16);
  const uint32_t b0 = lds32(rowB + qo), b1 = lds32(rowB + qo + 16);
  float blk[4] = {0.f, 0.f, 0.f, 0.f};
  uint32_t al, ah, bl, bh;
  const uint32_t xo = xs_g + (32u * unit + 4u * t) * 2u;
  uint2 xb = lds64(xo);
  e4m3x4_to_f16x4(a0, al, ah);
  e4m3x4_to_f16x4(b0, bl, bh);
  mma_f16_16816(blk, al, bl, ah, bh, xb.x, xb.y);
  xb = lds64(xo + 32u);
  e4m3x4_to_f16x4(a1, al, ah);
  e4m3x4_to_f16x4(b1, bl, bh);
  mma_f16_16816(blk, al, bl, ah, bh, xb.x, xb.y);
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i] = fmaf(scale, blk[i], acc[i]);
}

// e2m1 nibble pair (one byte: low nibble = even element) -> f16x2 holding value * 2^-14:
// f16 bits = sign<<15 | (exp,mant)<<9.
__device__ __forceinline__ uint32_t e2m1_byte_to_f16x2(uint32_t byte) {
  const uint32_t lo = byte & 0xFu, hi = (byte >> 4) & 0xFu;
  const uint32_t hl = ((lo & 7u) << 9) | ((lo & 8u) << 12);
  const uint32_t hh = ((hi & 7u) << 9) | ((hi & 8u) << 12);
  return hl | (hh << 16);
}

// MXFP4: unit = one 32-element block (16 bytes); e8m0 scale bytes staged per chunk in shared memory.
__device__ __forceinline__ void unit_mxfp4(float (&acc)[4], uint32_t rowA, uint32_t rowB, uint32_t xs_g, int unit,
                                           int t, float sA, float sB) {
  const uint32_t qo = 16u * unit + 4u * t;
  const uint32_t a = lds32(rowA + qo), b = lds32(rowB + qo);
  float blk[4] = {0.f, 0.f, 0.f, 0.f};
  const uint32_t xo = xs_g + (32u * unit + 8u * t) * 2u;
  uint2 xb = lds64(xo);
  mma_f16_16816(blk, e2m1_byte_to_f16x2(a), e2m1_byte_to_f16x2(b), e2m1_byte_to_f16x2(a >> 8),
                e2m1_byte_to_f16x2(b >> 8), xb.x, xb.y);
  xb = lds64(xo + 8u);
  mma_f16_16816(blk, e2m1_byte_to_f16x2(a >> 16), e2m1_byte_to_f16x2(b >> 16), e2m1_byte_to_f16x2(a >> 24),
                e2m1_byte_to_f16x2(b >> 24), xb.x, xb.y);
  acc[0] = fmaf(sA, blk[0], acc[0]);
  acc[1] = fmaf(sA, blk[1], acc[1]);
  acc[2] = fmaf(sB, blk[2], acc[2]);
  acc[3] = fmaf(sB, blk[3], acc[3]);
}

__device__ __forceinline__ float gated(float g, float u, const hq_act_args& a) {
  if (a.act == HQ_ACT_GPTOSS) {
    g = fminf(g, a.limit);
    u = fminf(fmaxf(u, -a.limit), a.limit);
    const float glu = g / (1.f + expf(-a.alpha * g));
    return (u + 1.f) * glu;
  }
  if (a.has_limit) {
    g = fminf(g, a.limit);
    u = fminf(fmaxf(u, -a.limit), a.limit);
  }
  return (g / (1.f + expf(-g))) * u;
}

// ---- the kernel --------------------------------------------------------------
template <int FMT, int WR, int KC, int NSTAGE>
__global__ void __launch_bounds__(kGemvThreads, 2) gemv_kernel(const GemvParams p) {
  using L = GemvSmem<FMT, WR, KC, NSTAGE>;
  using F = FmtTraits<FMT>;
  constexpr int WK = kConsumerWarps / WR;
  constexpr int RT = L::RT;
  extern __shared__ __align__(128) uint8_t smem[];

  // ---- which work item -------------------------------------------------------
  int expert = 0, row0 = 0, nrows = 0;
  if (p.tiles != nullptr) {
    const int n_items = p.tile_count[0];
    if ((int)blockIdx.y >= n_items) return;
    expert = p.tiles[2 * blockIdx.y];
    row0 = p.tiles[2 * blockIdx.y + 1];
    nrows = min(8, p.expert_bounds[expert + 1] - row0);
  } else {
    row0 = 8 * blockIdx.y;
    nrows = min(8, p.m - row0);
  }
  if (nrows <= 0) return;
  const int n0 = blockIdx.x * RT;
  const int rows_valid = min(RT, p.n - n0);
  const int nchunk = (p.k + KC - 1) / KC;
  const int nitems = nchunk * p.n_banks;

  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* empty = full + NSTAGE;
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < NSTAGE; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kConsumerWarps);
    }
    fence_barrier_init();
  }
  // zero both activation buffers once: rows >= nrows stay zero for the whole kernel
  for (int i = tid; i < L::X_BYTES / 16; i += kGemvThreads)
    reinterpret_cast<uint4*>(smem + L::OFF_X)[i] = make_uint4(0, 0, 0, 0);
  if (FMT == HQ_FMT_FP8_BLOCK) {
    // the row tile lies inside one 128-row scale block: cache its scale row
    const int kb = (p.k + 127) / 128;
    float* fsc = reinterpret_cast<float*>(smem + L::OFF_FSC);
    for (int b = 0; b < p.n_banks; ++b) {
      const float* src = reinterpret_cast<const float*>(b == 0 ? p.scales : p.scales_up) +
                         (int64_t)expert * p.scale_expert_stride + (int64_t)(n0 / 128) * kb;
      for (int i = tid; i < kb; i += kGemvThreads) fsc[b * 256 + i] = src[i];
    }
  }
  __syncthreads();

  const int64_t row_bytes = F::row_bytes(p.k);

  if (warp == kConsumerWarps) {
    // ================= producer warp: stream weight row segments ===============
    uint32_t spin = kSpinLimit;
    for (int it = 0; it < nitems; ++it) {
      const int s = it % NSTAGE;
      if (it >= NSTAGE) {
        if (!mbar_wait(&empty[s], ((it / NSTAGE) - 1) & 1, spin)) {
          // give up waiting but keep the control flow intact: results are invalid and flagged
          if (lane == 0) report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 100 + s);
          spin = 1;
        }
      }
      const int chunk = it / p.n_banks, bank = it - chunk * p.n_banks;
      const int kc_len = min(KC, p.k - chunk * KC);
      const uint32_t bytes = (uint32_t)F::seg_bytes(kc_len);
      const uint8_t* wsrc = reinterpret_cast<const uint8_t*>(bank == 0 ? p.w : p.w_up) +
                            (int64_t)expert * p.w_expert_stride + (int64_t)n0 * row_bytes +
                            (int64_t)F::seg_bytes(chunk * KC);
      if (lane == 0) mbar_arrive_expect_tx(&full[s], bytes * (uint32_t)rows_valid);
      __syncwarp();
      uint8_t* dst = smem + s * L::STAGE_BYTES;
      for (int r = lane; r < rows_valid; r += 32)
        bulk_g2s(dst + r * L::PITCH, wsrc + (int64_t)r * row_bytes, bytes, &full[s]);
    }
    return;
  }

  // ================= consumer warps ============================================
  const int wr = warp / WK, wk = warp % WK;
  const int g = lane >> 2, t = lane & 3;
  float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
  __half* xs_base = reinterpret_cast<__half*>(smem + L::OFF_X);
  float* xsum_base = reinterpret_cast<float*>(smem + L::OFF_XSUM);
  uint8_t* msc_base = smem + L::OFF_MSC;
  const float* fsc = reinterpret_cast<const float*>(smem + L::OFF_FSC);

  XPrefetch pf;
  x_prefetch<KC>(pf, p, p.x_rows, row0, nrows, 0, min(KC, p.k), tid);

  uint32_t spin = kSpinLimit;
  for (int chunk = 0; chunk < nchunk; ++chunk) {
    const int kc_len = min(KC, p.k - chunk * KC);
    const int buf = chunk & 1;
    __half* xs = xs_base + buf * 8 * L::XP;
    float* xsum = xsum_base + buf * (KC / 32) * 8;
    x_commit<F::kPermX, F::kNeedXsum, KC>(pf, p, nrows, kc_len, tid, xs, xsum);
    if (FMT == HQ_FMT_MXFP4) {
      // e8m0 scale bytes of this chunk, [bank][row][block]; plain byte loads (scale rows are not 16B aligned)
      const int nb = kc_len / 32, kb_row = p.k / 32;
      uint8_t* msc = msc_base + buf * 2 * RT * (KC / 32);
      for (int i = tid; i < p.n_banks * rows_valid * nb; i += kConsumerThreads) {
        const int bank = i / (rows_valid * nb);
        const int j = i - bank * rows_valid * nb;
        const int r = j / nb, b = j - r * nb;
        const uint8_t* sc = reinterpret_cast<const uint8_t*>(bank == 0 ? p.scales : p.scales_up);
        msc[(bank * RT + r) * (KC / 32) + b] =
            sc[(int64_t)expert * p.scale_expert_stride + (int64_t)(n0 + r) * kb_row + chunk * (KC / 32) + b];
      }
    }
    if (chunk + 1 < nchunk)
      x_prefetch<KC>(pf, p, p.x_rows, row0, nrows, (chunk + 1) * KC, min(KC, p.k - (chunk + 1) * KC), tid);
    named_bar_sync(1, kConsumerThreads);

    const uint32_t xs_g = smem_u32(xs) + (uint32_t)g * L::XP * 2u;
    const uint32_t xsum_t = smem_u32(xsum) + 8u * t;
#pragma unroll
    for (int bank = 0; bank < 2; ++bank) {
      if (bank >= p.n_banks) break;
      const int it = chunk * p.n_banks + bank;
      const int s = it % NSTAGE;
      if (!mbar_wait(&full[s], (it / NSTAGE) & 1, spin)) {
        // bounded wait ran out: flag it and carry on (every warp still reaches every barrier)
        if (lane == 0) report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 200 + s);
        spin = 1;
      }
      const uint32_t rowA = smem_u32(smem + s * L::STAGE_BYTES) + (uint32_t)(16 * wr + g) * L::PITCH;
      const uint32_t rowB = rowA + 8u * L::PITCH;
      float(&a)[4] = acc[bank];
      if (FMT == HQ_FMT_Q8_0) {
        const int nunits = kc_len / 32;
#pragma unroll 2
        for (int u = wk; u < nunits; u += WK) unit_q8_0(a, rowA, rowB, xs_g, xsum_t, u, t);
      } else if (FMT == HQ_FMT_Q4_K) {
        const int nunits = kc_len / 64;
#pragma unroll 2
        for (int u = wk; u < nunits; u += WK) unit_q4_k(a, rowA, rowB, xs_g, xsum_t, u, t);
      } else if (FMT == HQ_FMT_FP8_BLOCK) {
        const int nunits = kc_len / 32;
#pragma unroll 2
        for (int u = wk; u < nunits; u += WK)
          unit_fp8(a, rowA, rowB, xs_g, u, t, fsc[bank * 256 + (chunk * KC + 32 * u) / 128]);
      } else {
        const int nunits = kc_len / 32;
        const uint8_t* msc = msc_base + (buf * 2 + bank) * RT * (KC / 32);
#pragma unroll 2
        for (int u = wk; u < nunits; u += WK) {
          // 2^(e-127) with the reference's bit trick (e = 0 decodes to 0), times 2^14 for the nibble encoding
          const float sA = __uint_as_float((uint32_t)msc[(16 * wr + g) * (KC / 32) + u] << 23) * 16384.f;
          const float sB = __uint_as_float((uint32_t)msc[(16 * wr + g + 8) * (KC / 32) + u] << 23) * 16384.f;
          unit_mxfp4(a, rowA, rowB, xs_g, u, t, sA, sB);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }
  }
  // ---- reduce the K-split partials across warps (fixed order), epilogue ----------
  float* red = reinterpret_cast<float*>(smem + L::OFF_RED);
  if (WK > 1) {
#pragma unroll
    for (int b = 0; b < 2; ++b)
#pragma unroll
      for (int i = 0; i < 4; ++i) red[((b * kConsumerWarps + warp) * 4 + i) * 32 + lane] = acc[b][i];
    named_bar_sync(1, kConsumerThreads);
    if (wk != 0) return;
#pragma unroll
    for (int b = 0; b < 2; ++b)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float s = 0.f;
        for (int j = 0; j < WK; ++j) s += red[((b * kConsumerWarps + wr * WK + j) * 4 + i) * 32 + lane];
        acc[b][i] = s;
      }
  }
  // rows of this lane: n0 + 16*wr + g (+8); columns 2t, 2t+1
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int n = n0 + 16 * wr + g + 8 * half;
    const bool n_ok = n < p.n;
    float v0 = acc[0][2 * half], v1 = acc[0][2 * half + 1];
    float u0 = acc[1][2 * half], u1 = acc[1][2 * half + 1];
    if (n_ok && p.bias != nullptr) {
      const float bv = load_as_float(p.bias, p.bias_dtype, (int64_t)expert * p.n + n);
      v0 += bv; v1 += bv;
    }
    if (n_ok && p.n_banks == 2 && p.bias_up != nullptr) {
      const float bv = load_as_float(p.bias_up, p.bias_dtype, (int64_t)expert * p.n + n);
      u0 += bv; u1 += bv;
    }
    int64_t out_n = n;
    bool write = n_ok;
    if (p.act.act != HQ_ACT_NONE) {
      if (p.n_banks == 2) {
        v0 = gated(v0, u0, p.act);
        v1 = gated(v1, u1, p.act);
      } else {
        // interleaved bank: even row = gate, odd row = up (the neighbour lane group g+1)
        const float p0 = __shfl_down_sync(0xffffffffu, v0, 4);
        const float p1 = __shfl_down_sync(0xffffffffu, v1, 4);
        v0 = gated(v0, p0, p.act);
        v1 = gated(v1, p1, p.act);
        write = n_ok && (n & 1) == 0;
        out_n = n >> 1;
      }
    }
    if (write) {
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int col = 2 * t + cc;
        if (col < nrows) {
          const int64_t yr = p.y_rows ? (int64_t)p.y_rows[row0 + col] : (int64_t)(row0 + col);
          store_from_float(p.y, p.y_dtype, yr * p.y_stride + out_n, cc ? v1 : v0);
        }
      }
    }
  }
}

// ---- host launcher ------------------------------------------------------------
template <int FMT, int WR, int KC, int NSTAGE>
static int32_t launch_cfg(const GemvParams& p, int grid_y, cudaStream_t stream) {
  using L = GemvSmem<FMT, WR, KC, NSTAGE>;
  static_assert(L::TOTAL <= 227 * 1024, "shared memory budget");
  static_assert((L::PITCH / 4) % 8 == 4, "row pitch must spread banks");
  auto kern = gemv_kernel<FMT, WR, KC, NSTAGE>;
  static bool attr_done[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return HQ_ERR_CUDA;
  if (dev < 64 && !attr_done[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess)
      return HQ_ERR_CUDA;
    attr_done[dev] = true;
  }
  dim3 grid((unsigned)((p.n + L::RT - 1) / L::RT), (unsigned)grid_y, 1);
  kern<<<grid, kGemvThreads, L::TOTAL, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

template <int FMT>
static int32_t launch_fmt(const GemvParams& p, int grid_y, cudaStream_t stream) {
  // pick the row-tile height so that every SM holds at least two CTAs
  const int64_t groups = ((int64_t)p.n + 15) / 16 * grid_y;
  if (groups < 2 * 296) return launch_cfg<FMT, 1, 1024, 4>(p, grid_y, stream);
  if (groups < 4 * 296) return launch_cfg<FMT, 2, 1024, 3>(p, grid_y, stream);
  if (groups < 16 * 296) return launch_cfg<FMT, 4, 512, 3>(p, grid_y, stream);
  return launch_cfg<FMT, 8, 256, 3>(p, grid_y, stream);
}

int32_t launch_gemv(const GemvParams& p, int grid_y, cudaStream_t stream) {
  switch (p.format) {
    case HQ_FMT_Q8_0: return launch_fmt<HQ_FMT_Q8_0>(p, grid_y, stream);
    case HQ_FMT_Q4_K: return launch_fmt<HQ_FMT_Q4_K>(p, grid_y, stream);
    case HQ_FMT_FP8_BLOCK: return launch_fmt<HQ_FMT_FP8_BLOCK>(p, grid_y, stream);
    case HQ_FMT_MXFP4: return launch_fmt<HQ_FMT_MXFP4>(p, grid_y, stream);
    default: return HQ_ERR_FORMAT;
  }
}

}  // namespace hq
