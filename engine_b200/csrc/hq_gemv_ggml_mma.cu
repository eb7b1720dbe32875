// Decode mat-vec (1..8 activation rows per work item, dense and expert-indexed) for the GGML types Q6_K, Q5_K,
// Q4_0, Q5_0, Q4_1, Q5_1, Q2_K and Q3_K of the reference's decode list (hanzo-quant/src/gguf/fast_mmvq.rs:36-50; the
// reference multiplies them with dp4a against Q8_1 activations, kernels/mmvq_gguf/mmvq_gguf.cu).
//
// The codes of these types are small integers (2 to 6 bits), exact in f16 and bf16, so the products run on the
// warp MMA m16n8k16 with f32 accumulation: one MMA covers 16 output rows x 16 consecutive weights x 8 activation
// rows, and the per-block factor (d * scale, or d) multiplies the f32 result of one (16-weight groups of Q6_K, Q3_K,
// Q2_K) or two (32-weight blocks) MMAs.  The additive term of Q5_K, Q2_K ("- dmin * m") and Q4_1 / Q5_1 ("+ m") uses
// the sum of the activations over the block, which a second MMA against a fragment of ones delivers in the same
// layout.  bf16 activations are multiplied as bf16 (nothing is converted or rounded), f16 as f16, f32 activations
// are rounded to f16 (clamped to +-65504 and flagged beyond).
//
// One CTA of eight warps per work item of 16 output rows (persistent, three CTAs per SM); the warps take the
// 256-weight spans of K in turn and their partial sums are added in warp order by one warp (the warps take turns;
// two buffers, one CTA barrier per item), so results are bit-reproducible.  Each warp brings its spans in through a
// two-deep ring of cp.async stages (16 rows x one span; aligned 16-byte pieces from the 32-byte boundary below the
// span on, since Q6_K and Q3_K rows start on 2-byte boundaries and Q2_K rows on 4-byte ones) that runs across work
// items, and picks the fields out of shared memory: lane (g, t) decodes the four consecutive weights 4 t .. 4 t + 3
// of a 16-weight group for the rows g and g + 8 (the MMA's k index is permuted accordingly on both operands), i.e.
// one 32-bit word of code bits plus one of high bits.  Codes become f16 / bf16 by a byte permute into the mantissa of
// 1024 / 128 and one packed subtraction.  Activations are read straight from global memory (8 bytes per lane and
// group; they stay in L1).
// Roofline: HBM; algorithmic bytes per launch = N*K*bits/8 + M*K*sizeof(x) + M*N*sizeof(y)
// (bits: 6.5625, 5.5, 4.5, 5.5, 5, 6, 2.625, 3.4375).
#include "hq_gemv_shared.cuh"

namespace hq {

constexpr int kGmWarps = 8;
constexpr int kGmThreads = kGmWarps * 32;
constexpr int kGmStages = 2;
constexpr int kGmRows = 16;

// SPAN: bytes per 256 weights; PITCH: distance of the rows in a stage (a multiple of 16 whose word count spreads the
// eight row groups over the banks, with room for the up to 30 bytes between the 32-byte boundary a copy starts at
// and the first byte of the span); ZERO: the code's zero point.
template <int FMT>
struct GmFmt;
template <>
struct GmFmt<HQ_FMT_Q6_K> {
  static constexpr int SPAN = 210, PITCH = 240, ZERO = 32;
};
template <>
struct GmFmt<HQ_FMT_Q5_K> {
  static constexpr int SPAN = 176, PITCH = 208, ZERO = 0;
};
template <>
struct GmFmt<HQ_FMT_Q4_0> {
  static constexpr int SPAN = 144, PITCH = 176, ZERO = 8;
};
template <>
struct GmFmt<HQ_FMT_Q5_0> {
  static constexpr int SPAN = 176, PITCH = 208, ZERO = 16;
};
template <>
struct GmFmt<HQ_FMT_Q4_1> {
  static constexpr int SPAN = 160, PITCH = 208, ZERO = 0;
};
template <>
struct GmFmt<HQ_FMT_Q5_1> {
  static constexpr int SPAN = 192, PITCH = 240, ZERO = 0;
};
template <>
struct GmFmt<HQ_FMT_Q2_K> {
  static constexpr int SPAN = 84, PITCH = 144, ZERO = 0;
};
template <>
struct GmFmt<HQ_FMT_Q3_K> {
  static constexpr int SPAN = 110, PITCH = 144, ZERO = 4;
};

template <bool BF>
__device__ __forceinline__ void gm_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  if (BF) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    mma_f16_16816(d, a0, a1, a2, a3, b0, b1);
  }
}

// the first MMA of a block: D = A.B (the zero C operands cost no register moves)
template <bool BF>
__device__ __forceinline__ void gm_mma0(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
  if (BF) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
  } else {
    mma_f16_16816_c(d, a0, a1, a2, a3, b0, b1, 0.f, 0.f, 0.f, 0.f);
  }
}

// The codes in bytes 2 pair and 2 pair + 1 of qq as f16x2 / bf16x2 of (code - ZERO): 0x64qq is 1024 + qq in f16,
// 0x43qq is 128 + qq in bf16 (qq < 64), and the subtraction is exact.
template <bool BF, int ZERO>
__device__ __forceinline__ uint32_t gm_pair(uint32_t qq, int pair) {
  const uint32_t v = __byte_perm(qq, BF ? 0x43434343u : 0x64646464u, pair == 0 ? 0x4140u : 0x4342u);
  constexpr uint32_t c = (BF ? 0x4300u : 0x6400u) + (uint32_t)ZERO;
  uint32_t r;
  if (BF) asm("sub.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(v), "r"(c | (c << 16)));
  else asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(v), "r"(c | (c << 16)));
  return r;
}

// 4 bytes at a 2-byte aligned shared-memory address
__device__ __forceinline__ uint32_t gm_ld32h(const uint8_t* p) {
  const uint16_t* h = reinterpret_cast<const uint16_t*>(p);
  return (uint32_t)h[0] | ((uint32_t)h[1] << 16);
}

// B fragment of one 16-weight group: four consecutive activations of this lane's activation row (none: zeros).
// xq points at the lane's first activation of the span, `col` (a multiple of 4, known at compile time) counts on
// from there, so the load takes an immediate offset.
template <int XDT>
__device__ __forceinline__ void gm_load_b(const char* xq, int col, uint32_t& b0, uint32_t& b1, bool& clamped) {
  b0 = b1 = 0u;
  if (xq == nullptr) return;
  if (XDT == HQ_DT_F32) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(xq) + (col >> 2));
    float f[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float a = fabsf(f[i]);
      if (a > 65504.f && a <= 3.402823466e38f) {   // finite and beyond f16: clamp; NaN and infinity pass through
        f[i] = copysignf(65504.f, f[i]);
        clamped = true;
      }
    }
    b0 = pack_half2(f[0], f[1]);
    b1 = pack_half2(f[2], f[3]);
  } else {
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(xq) + (col >> 2));
    b0 = v.x;
    b1 = v.y;
  }
}

// One 256-weight span of the rows g (block bytes at bA) and g + 8 (bB) against the activations of the span; xq
// points at activation 4 t of the span in this lane's activation row (nullptr: the lane feeds zeros).
template <int FMT, bool BF, int XDT>
__device__ __forceinline__ void gm_decode_span(float (&acc)[4], const uint8_t* bA, const uint8_t* bB, const char* xq,
                                               int t, bool& clamped) {
  constexpr int Z = GmFmt<FMT>::ZERO;
  if (FMT == HQ_FMT_Q6_K) {
    // {ql[128], qh[64], int8 scales[16], f16 d}: the 16-weight group 8 h + 2 j + u holds the weights
    // 128 h + 32 j + 16 u + i: nibble j / 2 of ql[64 h + 32 (j % 2) + 16 u + i], bits 2 j of qh[32 h + 16 u + i]
    // per group: span sum += scale * (codes . x), scale an int8; d multiplies the span sum once
    float sp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const uint32_t qhA = gm_ld32h(bA + 128 + 32 * h + 16 * u + 4 * t);
        const uint32_t qhB = gm_ld32h(bB + 128 + 32 * h + 16 * u + 4 * t);
#pragma unroll
        for (int jlo = 0; jlo < 2; ++jlo) {
          const uint32_t qlA = gm_ld32h(bA + 64 * h + 32 * jlo + 16 * u + 4 * t);
          const uint32_t qlB = gm_ld32h(bB + 64 * h + 32 * jlo + 16 * u + 4 * t);
#pragma unroll
          for (int jhi = 0; jhi < 2; ++jhi) {
            const int j = jlo + 2 * jhi, s16 = 8 * h + 2 * j + u;
            const uint32_t qa = ((qlA >> (4 * jhi)) & 0x0F0F0F0Fu) | (((qhA >> (2 * j)) & 0x03030303u) << 4);
            const uint32_t qb = ((qlB >> (4 * jhi)) & 0x0F0F0F0Fu) | (((qhB >> (2 * j)) & 0x03030303u) << 4);
            uint32_t b0, b1;
            gm_load_b<XDT>(xq, 16 * s16, b0, b1, clamped);
            float blk[4];
            gm_mma0<BF>(blk, gm_pair<BF, Z>(qa, 0), gm_pair<BF, Z>(qb, 0), gm_pair<BF, Z>(qa, 1),
                        gm_pair<BF, Z>(qb, 1), b0, b1);
            const float sA = (float)(int)(int8_t)bA[192 + s16];
            const float sB = (float)(int)(int8_t)bB[192 + s16];
            sp[0] = fmaf(sA, blk[0], sp[0]);
            sp[1] = fmaf(sA, blk[1], sp[1]);
            sp[2] = fmaf(sB, blk[2], sp[2]);
            sp[3] = fmaf(sB, blk[3], sp[3]);
          }
        }
      }
    }
    const float dA = __half2float(*reinterpret_cast<const __half*>(bA + 208));
    const float dB = __half2float(*reinterpret_cast<const __half*>(bB + 208));
    acc[0] = fmaf(dA, sp[0], acc[0]);
    acc[1] = fmaf(dA, sp[1], acc[1]);
    acc[2] = fmaf(dB, sp[2], acc[2]);
    acc[3] = fmaf(dB, sp[3], acc[3]);
  } else if (FMT == HQ_FMT_Q5_K) {
    // {f16 d, f16 dmin, scales[12], qh[32], qs[128]}: the 32-weight block j = 2 c + hi holds nibble hi of
    // qs[32 c + l] and bit j of qh[l], l = 0..31; value = d sc_j q - dmin m_j
    const uint4 hA = *reinterpret_cast<const uint4*>(bA), hB = *reinterpret_cast<const uint4*>(bB);
    const float dA = half_bits_to_float(hA.x), nA = half_bits_to_float(hA.x >> 16);
    const float dB = half_bits_to_float(hB.x), nB = half_bits_to_float(hB.x >> 16);
    uint32_t qhA[2], qhB[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      qhA[u] = *reinterpret_cast<const uint32_t*>(bA + 16 + 16 * u + 4 * t);
      qhB[u] = *reinterpret_cast<const uint32_t*>(bB + 16 + 16 * u + 4 * t);
    }
    constexpr uint32_t ONE = BF ? 0x3F803F80u : 0x3C003C00u;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t wA[2], wB[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        wA[u] = *reinterpret_cast<const uint32_t*>(bA + 48 + 32 * c + 16 * u + 4 * t);
        wB[u] = *reinterpret_cast<const uint32_t*>(bB + 48 + 32 * c + 16 * u + 4 * t);
      }
#pragma unroll
      for (int hi = 0; hi < 2; ++hi) {
        const int j = 2 * c + hi;
        uint32_t scA, mnA, scB, mnB;
        if (j < 4) {
          scA = (hA.y >> (8 * j)) & 63u;
          mnA = (hA.z >> (8 * j)) & 63u;
          scB = (hB.y >> (8 * j)) & 63u;
          mnB = (hB.z >> (8 * j)) & 63u;
        } else {
          const int jj = j - 4;
          scA = ((hA.w >> (8 * jj)) & 0xFu) | (((hA.y >> (8 * jj + 6)) & 3u) << 4);
          mnA = ((hA.w >> (8 * jj + 4)) & 0xFu) | (((hA.z >> (8 * jj + 6)) & 3u) << 4);
          scB = ((hB.w >> (8 * jj)) & 0xFu) | (((hB.y >> (8 * jj + 6)) & 3u) << 4);
          mnB = ((hB.w >> (8 * jj + 4)) & 0xFu) | (((hB.z >> (8 * jj + 6)) & 3u) << 4);
        }
        float bq[4], b1s[4];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const uint32_t qa = ((wA[u] >> (4 * hi)) & 0x0F0F0F0Fu) | (((qhA[u] >> j) & 0x01010101u) << 4);
          const uint32_t qb = ((wB[u] >> (4 * hi)) & 0x0F0F0F0Fu) | (((qhB[u] >> j) & 0x01010101u) << 4);
          uint32_t b0, b1;
          gm_load_b<XDT>(xq, 32 * j + 16 * u, b0, b1, clamped);
          if (u == 0) {
            gm_mma0<BF>(bq, gm_pair<BF, Z>(qa, 0), gm_pair<BF, Z>(qb, 0), gm_pair<BF, Z>(qa, 1), gm_pair<BF, Z>(qb, 1),
                        b0, b1);
            gm_mma0<BF>(b1s, ONE, ONE, ONE, ONE, b0, b1);            // sums of the activations, per column
          } else {
            gm_mma<BF>(bq, gm_pair<BF, Z>(qa, 0), gm_pair<BF, Z>(qb, 0), gm_pair<BF, Z>(qa, 1), gm_pair<BF, Z>(qb, 1),
                       b0, b1);
            gm_mma<BF>(b1s, ONE, ONE, ONE, ONE, b0, b1);
          }
        }
        const float sA = dA * (float)scA, sB = dB * (float)scB;       // exact
        const float oA = nA * (float)mnA, oB = nB * (float)mnB;
        acc[0] = fmaf(sA, bq[0], fmaf(-oA, b1s[0], acc[0]));
        acc[1] = fmaf(sA, bq[1], fmaf(-oA, b1s[1], acc[1]));
        acc[2] = fmaf(sB, bq[2], fmaf(-oB, b1s[2], acc[2]));
        acc[3] = fmaf(sB, bq[3], fmaf(-oB, b1s[3], acc[3]));
      }
    }
  } else if (FMT == HQ_FMT_Q2_K) {
    // {scales[16], qs[64], f16 d, f16 dmin}, 4-byte aligned: the 16-weight group 8 h + 2 j + u holds bits 2 j,
    // 2 j + 1 of qs[32 h + 16 u + i]; value = d (s & 15) q - dmin (s >> 4) with s = scales[group]
    const uint32_t hA = *reinterpret_cast<const uint32_t*>(bA + 80), hB = *reinterpret_cast<const uint32_t*>(bB + 80);
    const float dA = half_bits_to_float(hA), nA = half_bits_to_float(hA >> 16);
    const float dB = half_bits_to_float(hB), nB = half_bits_to_float(hB >> 16);
    uint32_t scA[4], scB[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      scA[i] = *reinterpret_cast<const uint32_t*>(bA + 4 * i);
      scB[i] = *reinterpret_cast<const uint32_t*>(bB + 4 * i);
    }
    constexpr uint32_t ONE = BF ? 0x3F803F80u : 0x3C003C00u;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const uint32_t wA = *reinterpret_cast<const uint32_t*>(bA + 16 + 32 * h + 16 * u + 4 * t);
        const uint32_t wB = *reinterpret_cast<const uint32_t*>(bB + 16 + 32 * h + 16 * u + 4 * t);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int s16 = 8 * h + 2 * j + u;
          const uint32_t qa = (wA >> (2 * j)) & 0x03030303u, qb = (wB >> (2 * j)) & 0x03030303u;
          uint32_t b0, b1;
          gm_load_b<XDT>(xq, 16 * s16, b0, b1, clamped);
          float bq[4], b1s[4];
          gm_mma0<BF>(bq, gm_pair<BF, Z>(qa, 0), gm_pair<BF, Z>(qb, 0), gm_pair<BF, Z>(qa, 1), gm_pair<BF, Z>(qb, 1),
                      b0, b1);
          gm_mma0<BF>(b1s, ONE, ONE, ONE, ONE, b0, b1);              // sums of the activations, per column
          const uint32_t sa = (scA[s16 >> 2] >> (8 * (s16 & 3))) & 0xFFu, sb = (scB[s16 >> 2] >> (8 * (s16 & 3))) & 0xFFu;
          const float sA = dA * (float)(sa & 15u), oA = nA * (float)(sa >> 4);      // exact
          const float sB = dB * (float)(sb & 15u), oB = nB * (float)(sb >> 4);
          acc[0] = fmaf(sA, bq[0], fmaf(-oA, b1s[0], acc[0]));
          acc[1] = fmaf(sA, bq[1], fmaf(-oA, b1s[1], acc[1]));
          acc[2] = fmaf(sB, bq[2], fmaf(-oB, b1s[2], acc[2]));
          acc[3] = fmaf(sB, bq[3], fmaf(-oB, b1s[3], acc[3]));
        }
      }
    }
  } else if (FMT == HQ_FMT_Q3_K) {
    // {hmask[32], qs[64], scales[12], f16 d}, 2-byte aligned: the 16-weight group 8 h + 2 j + u holds bits 2 j,
    // 2 j + 1 of qs[32 h + 16 u + i] and, as third bit, bit 4 h + j of hmask[16 u + i]; value = d (scale - 32)
    // (code - 4).  The sixteen 6-bit scales are unpacked four to a word as ggml does it.
    uint32_t auxA[4], auxB[4];
    {
      const uint32_t a0 = gm_ld32h(bA + 96), a1 = gm_ld32h(bA + 100), tm = gm_ld32h(bA + 104);
      auxA[0] = (a0 & 0x0F0F0F0Fu) | ((tm & 0x03030303u) << 4);
      auxA[1] = (a1 & 0x0F0F0F0Fu) | (((tm >> 2) & 0x03030303u) << 4);
      auxA[2] = ((a0 >> 4) & 0x0F0F0F0Fu) | (((tm >> 4) & 0x03030303u) << 4);
      auxA[3] = ((a1 >> 4) & 0x0F0F0F0Fu) | (((tm >> 6) & 0x03030303u) << 4);
      const uint32_t c0 = gm_ld32h(bB + 96), c1 = gm_ld32h(bB + 100), tn = gm_ld32h(bB + 104);
      auxB[0] = (c0 & 0x0F0F0F0Fu) | ((tn & 0x03030303u) << 4);
      auxB[1] = (c1 & 0x0F0F0F0Fu) | (((tn >> 2) & 0x03030303u) << 4);
      auxB[2] = ((c0 >> 4) & 0x0F0F0F0Fu) | (((tn >> 4) & 0x03030303u) << 4);
      auxB[3] = ((c1 >> 4) & 0x0F0F0F0Fu) | (((tn >> 6) & 0x03030303u) << 4);
    }
    float sp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const uint32_t hmA = gm_ld32h(bA + 16 * u + 4 * t), hmB = gm_ld32h(bB + 16 * u + 4 * t);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t wA = gm_ld32h(bA + 32 + 32 * h + 16 * u + 4 * t), wB = gm_ld32h(bB + 32 + 32 * h + 16 * u + 4 * t);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int s16 = 8 * h + 2 * j + u;
          const uint32_t qa = ((wA >> (2 * j)) & 0x03030303u) | (((hmA >> (4 * h + j)) & 0x01010101u) << 2);
          const uint32_t qb = ((wB >> (2 * j)) & 0x03030303u) | (((hmB >> (4 * h + j)) & 0x01010101u) << 2);
          uint32_t b0, b1;
          gm_load_b<XDT>(xq, 16 * s16, b0, b1, clamped);
          float blk[4];
          gm_mma0<BF>(blk, gm_pair<BF, Z>(qa, 0), gm_pair<BF, Z>(qb, 0), gm_pair<BF, Z>(qa, 1), gm_pair<BF, Z>(qb, 1),
                      b0, b1);
          const float sA = (float)((int)((auxA[s16 >> 2] >> (8 * (s16 & 3))) & 0xFFu) - 32);
          const float sB = (float)((int)((auxB[s16 >> 2] >> (8 * (s16 & 3))) & 0xFFu) - 32);
          sp[0] = fmaf(sA, blk[0], sp[0]);
          sp[1] = fmaf(sA, blk[1], sp[1]);
          sp[2] = fmaf(sB, blk[2], sp[2]);
          sp[3] = fmaf(sB, blk[3], sp[3]);
        }
      }
    }
    const float dA = __half2float(*reinterpret_cast<const __half*>(bA + 108));
    const float dB = __half2float(*reinterpret_cast<const __half*>(bB + 108));
    acc[0] = fmaf(dA, sp[0], acc[0]);
    acc[1] = fmaf(dA, sp[1], acc[1]);
    acc[2] = fmaf(dB, sp[2], acc[2]);
    acc[3] = fmaf(dB, sp[3], acc[3]);
  } else {
    // blocks of 32: Q4_0 {f16 d, qs[16]}, Q5_0 {f16 d, u32 qh, qs[16]}, Q4_1 {f16 d, f16 m, qs[16]}, Q5_1 {f16 d,
    // f16 m, u32 qh, qs[16]}: weight i < 16 is the low nibble of qs[i], weight i >= 16 the high nibble of
    // qs[i - 16]; the fifth bit of weight i is bit i of qh; value = d (q - zero) resp. d q + m
    constexpr bool FIVE = FMT == HQ_FMT_Q5_0 || FMT == HQ_FMT_Q5_1;
    constexpr bool MIN = FMT == HQ_FMT_Q4_1 || FMT == HQ_FMT_Q5_1;
    constexpr int BB = 18 + (FIVE ? 4 : 0) + (MIN ? 2 : 0);
    constexpr int QS = BB - 16;
    constexpr int QH = MIN ? 4 : 2;
    constexpr uint32_t ONE = BF ? 0x3F803F80u : 0x3C003C00u;
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const uint8_t* kA = bA + BB * b;
      const uint8_t* kB = bB + BB * b;
      const float dA = __half2float(*reinterpret_cast<const __half*>(kA));
      const float dB = __half2float(*reinterpret_cast<const __half*>(kB));
      // rows are 16-byte aligned, so the words of the blocks whose offset BB b + QS is a multiple of 4 are aligned
      const bool AL = (BB * b + QS) % 4 == 0;                     // folded once the loop is unrolled
      const uint32_t wA = AL ? *reinterpret_cast<const uint32_t*>(kA + QS + 4 * t) : gm_ld32h(kA + QS + 4 * t);
      const uint32_t wB = AL ? *reinterpret_cast<const uint32_t*>(kB + QS + 4 * t) : gm_ld32h(kB + QS + 4 * t);
      uint32_t qhA = 0u, qhB = 0u;
      if (FIVE) {
        qhA = (AL ? *reinterpret_cast<const uint32_t*>(kA + QH) : gm_ld32h(kA + QH)) >> (4 * t);
        qhB = (AL ? *reinterpret_cast<const uint32_t*>(kB + QH) : gm_ld32h(kB + QH)) >> (4 * t);
      }
      float blk[4], b1s[4];
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t qa = (wA >> (4 * hf)) & 0x0F0F0F0Fu, qb = (wB >> (4 * hf)) & 0x0F0F0F0Fu;
        if (FIVE) {
          // four bits -> bit 4 of four bytes: x * 0x00204081 puts bit c of x at bit 8 c
          qa |= ((((qhA >> (16 * hf)) & 0xFu) * 0x00204081u) & 0x01010101u) << 4;
          qb |= ((((qhB >> (16 * hf)) & 0xFu) * 0x00204081u) & 0x01010101u) << 4;
        }
        uint32_t b0, b1;
        gm_load_b<XDT>(xq, 32 * b + 16 * hf, b0, b1, clamped);
        if (hf == 0) {
          gm_mma0<BF>(blk, gm_pair<BF, Z>(qa, 0), gm_pair<BF, Z>(qb, 0), gm_pair<BF, Z>(qa, 1), gm_pair<BF, Z>(qb, 1),
                      b0, b1);
          if (MIN) gm_mma0<BF>(b1s, ONE, ONE, ONE, ONE, b0, b1);     // sums of the activations, per column
        } else {
          gm_mma<BF>(blk, gm_pair<BF, Z>(qa, 0), gm_pair<BF, Z>(qb, 0), gm_pair<BF, Z>(qa, 1), gm_pair<BF, Z>(qb, 1),
                     b0, b1);
          if (MIN) gm_mma<BF>(b1s, ONE, ONE, ONE, ONE, b0, b1);
        }
      }
      acc[0] = fmaf(dA, blk[0], acc[0]);
      acc[1] = fmaf(dA, blk[1], acc[1]);
      acc[2] = fmaf(dB, blk[2], acc[2]);
      acc[3] = fmaf(dB, blk[3], acc[3]);
      if (MIN) {
        const float mA = __half2float(*reinterpret_cast<const __half*>(kA + 2));
        const float mB = __half2float(*reinterpret_cast<const __half*>(kB + 2));
        acc[0] = fmaf(mA, b1s[0], acc[0]);
        acc[1] = fmaf(mA, b1s[1], acc[1]);
        acc[2] = fmaf(mB, b1s[2], acc[2]);
        acc[3] = fmaf(mB, b1s[3], acc[3]);
      }
    }
  }
}

template <int FMT, int BANKS>
constexpr int gm_smem_bytes() {
  return kGmWarps * kGmStages * kGmRows * GmFmt<FMT>::PITCH + 2 * kGmWarps * BANKS * 4 * 32 * 4;
}

template <int FMT, int BANKS, int XDT>
__global__ void __launch_bounds__(kGmThreads, 3) gemv_ggml_mma_kernel(const GemvParams p) {
  using F = GmFmt<FMT>;
  constexpr bool BF = XDT == HQ_DT_BF16;
  constexpr int STAGE = kGmRows * F::PITCH;
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  uint8_t* ring = smem + warp * (kGmStages * STAGE);
  float* red = reinterpret_cast<float*>(smem + kGmWarps * kGmStages * STAGE);   // [2][warps][BANKS][4][32]

  const int n_rt = (p.n + kGmRows - 1) / kGmRows;
  const int n_y = p.tiles != nullptr ? p.tile_count[0] : (p.m + 7) / 8;
  const int total = n_y * n_rt;
  const int spans = p.k / 256;
  const int64_t row_bytes = (int64_t)spans * F::SPAN;
  const int xsz = dtype_size(XDT);
  const uint8_t* wbank[2] = {reinterpret_cast<const uint8_t*>(p.w), reinterpret_cast<const uint8_t*>(p.w_up)};

  // ---- the copy side: the same walk over (item, span, bank) as the multiplying side, kGmStages - 1 steps ahead.
  // One commit group per step, empty once the walk is over (or for a warp without spans), so that the group count
  // stays in step with the waits.
  auto next_item = [&](int w) {
    while (w < total && get_item<kGmRows>(p, w, n_rt).nrows <= 0) w += (int)gridDim.x;
    return w;
  };
  int iw = warp < spans ? next_item((int)blockIdx.x) : total;
  int ispan = warp, ibank = 0, islot = 0;
  WorkItem iwi = iw < total ? get_item<kGmRows>(p, iw, n_rt) : WorkItem{};
  auto issue = [&]() {
    if (iw < total) {
      const int r = lane >> 1;
      const int n = min(iwi.n0 + r, p.n - 1);                    // rows past N repeat the last one; never stored
      const uint8_t* src =
          wbank[ibank] + (int64_t)iwi.expert * p.w_expert_stride + (int64_t)n * row_bytes + (int64_t)ispan * F::SPAN;
      // start at the 32-byte boundary: the two lanes of a row then ask for the two halves of one sector in the
      // same instruction, and no sector crosses to the SM twice
      const int off = (int)(reinterpret_cast<uintptr_t>(src) & 31u);
      src -= off;
      const int n16 = (off + F::SPAN + 15) >> 4;
      static_assert(((30 + F::SPAN + 15) >> 4) * 16 <= F::PITCH, "a row's pieces must fit its pitch");
      const uint32_t dst = smem_u32(ring + islot * STAGE + r * F::PITCH);
      for (int i = lane & 1; i < n16; i += 2) cp_async16(dst + 16u * i, src + 16 * i);
      if (++ibank == BANKS) {
        ibank = 0;
        ispan += kGmWarps;
        if (ispan >= spans) {
          ispan = warp;
          iw = next_item(iw + (int)gridDim.x);
          if (iw < total) iwi = get_item<kGmRows>(p, iw, n_rt);
        }
      }
    }
    cp_async_commit();
    islot = islot + 1 == kGmStages ? 0 : islot + 1;
  };
#pragma unroll
  for (int i = 0; i < kGmStages - 1; ++i) issue();

  int cslot = 0, item = 0;
  bool clamped = false;
  for (int w = blockIdx.x; w < total; w += gridDim.x) {
    const WorkItem wi = get_item<kGmRows>(p, w, n_rt);
    if (wi.nrows <= 0) continue;                                 // the same for every thread of the CTA
    float acc[BANKS][4];
#pragma unroll
    for (int b = 0; b < BANKS; ++b)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[b][i] = 0.f;
    // the activation row this lane feeds into the MMA (column g of the B operand)
    const char* xrow = nullptr;
    if (g < wi.nrows) {
      const int sr = wi.row0 + g;
      const int64_t xr = p.x_rows != nullptr ? (int64_t)p.x_rows[sr] : (int64_t)sr;
      xrow = reinterpret_cast<const char*>(p.x) + xr * p.x_stride * xsz;
    }
    const int64_t rowA = (int64_t)wi.expert * p.w_expert_stride + (int64_t)min(wi.n0 + g, p.n - 1) * row_bytes;
    const int64_t rowB = (int64_t)wi.expert * p.w_expert_stride + (int64_t)min(wi.n0 + g + 8, p.n - 1) * row_bytes;
    for (int span = warp; span < spans; span += kGmWarps) {
#pragma unroll
      for (int bank = 0; bank < BANKS; ++bank) {
        issue();
        cp_async_wait<kGmStages - 1>();
        __syncwarp();
        const uint8_t* st = ring + cslot * STAGE;
        const int offA = (int)(reinterpret_cast<uintptr_t>(wbank[bank] + rowA + (int64_t)span * F::SPAN) & 31u);
        const int offB = (int)(reinterpret_cast<uintptr_t>(wbank[bank] + rowB + (int64_t)span * F::SPAN) & 31u);
        gm_decode_span<FMT, BF, XDT>(acc[bank], st + g * F::PITCH + offA, st + (g + 8) * F::PITCH + offB,
                                     xrow != nullptr ? xrow + (int64_t)(256 * span + 4 * t) * xsz : nullptr, t, clamped);
        __syncwarp();                                            // the stage is refilled two steps on
        cslot = cslot + 1 == kGmStages ? 0 : cslot + 1;
      }
    }
    // ---- partial sums of the eight warps -> warp 0, which adds them in warp order and writes -----------------
    float* rb = red + (item & 1) * (kGmWarps * BANKS * 4 * 32);
#pragma unroll
    for (int b = 0; b < BANKS; ++b)
#pragma unroll
      for (int i = 0; i < 4; ++i) rb[((warp * BANKS + b) * 4 + i) * 32 + lane] = acc[b][i];
    __syncthreads();
    if (warp == (item & (kGmWarps - 1))) {                       // the adding warp rotates, so none falls behind
      float v[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int b = 0; b < BANKS; ++b)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float sum = 0.f;
#pragma unroll
          for (int j = 0; j < kGmWarps; ++j) sum += rb[((j * BANKS + b) * 4 + i) * 32 + lane];
          v[b][i] = sum;
        }
      // rows of this lane: n0 + g (+ 8); activation rows 2 t, 2 t + 1
      gemv_store_item(p, wi, g, 2 * t, true, v);
    }
    ++item;
  }
  if (clamped) report_status(p.status, HQ_DEV_F16_RANGE, 910);
}

template <int FMT, int BANKS, int XDT>
static int32_t launch_gm(const GemvParams& p, int64_t items, cudaStream_t stream) {
  auto kern = gemv_ggml_mma_kernel<FMT, BANKS, XDT>;
  constexpr int smem = gm_smem_bytes<FMT, BANKS>();
  static int ctas_per_sm[64] = {};                               // resident CTAs per SM, asked once per device
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= 64) return HQ_ERR_CUDA;
  if (ctas_per_sm[dev] == 0) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return HQ_ERR_CUDA;
    // several CTAs per SM need the largest shared-memory carve-out; the activations only need a few KB of L1
    if (cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) !=
        cudaSuccess)
      return HQ_ERR_CUDA;
    int occ = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, kGmThreads, smem) != cudaSuccess || occ <= 0)
      return HQ_ERR_CUDA;
    ctas_per_sm[dev] = occ;
  }
  // persistent: as many CTAs as stay resident, each walking the items with that stride
  const int64_t cap = (int64_t)sm_count() * ctas_per_sm[dev];
  const unsigned grid = (unsigned)(items < cap ? items : cap);
  kern<<<grid, kGmThreads, smem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

template <int FMT, int BANKS>
static int32_t launch_gm_x(const GemvParams& p, int64_t items, cudaStream_t stream) {
  switch (p.x_dtype) {
    case HQ_DT_F32: return launch_gm<FMT, BANKS, HQ_DT_F32>(p, items, stream);
    case HQ_DT_F16: return launch_gm<FMT, BANKS, HQ_DT_F16>(p, items, stream);
    case HQ_DT_BF16: return launch_gm<FMT, BANKS, HQ_DT_BF16>(p, items, stream);
    default: return HQ_ERR_FORMAT;
  }
}

template <int FMT>
static int32_t launch_gm_fmt(const GemvParams& p, int64_t items, cudaStream_t stream) {
  return p.n_banks == 2 ? launch_gm_x<FMT, 2>(p, items, stream) : launch_gm_x<FMT, 1>(p, items, stream);
}

// Plain projection, or a gate and an up bank with a gated activation; an interleaved gate/up bank is not taken.
// Activation rows must be 16-byte aligned (the entry points of the library check it), and so must the rows of the
// types whose blocks allow it.
int32_t launch_gemv_ggml_mma(const GemvParams& p, int n_y_max, cudaStream_t stream) {
  if (p.k % 256 != 0) return HQ_ERR_SHAPE;
  if (p.n_banks == 1 && p.act.act != HQ_ACT_NONE) return HQ_ERR_FORMAT;
  if (p.n_banks == 2 && p.act.act == HQ_ACT_NONE) return HQ_ERR_FORMAT;
  const int esz = dtype_size(p.x_dtype);
  if ((reinterpret_cast<uintptr_t>(p.x) & 15u) != 0 || (p.x_stride * esz) % 16 != 0) return HQ_ERR_ALIGN;
  // Q6_K and Q3_K blocks are picked apart with 16-bit loads; Q2_K blocks need 4-byte alignment (any K does, from an
  // aligned tensor); the other types rely on 16-byte aligned rows
  if (p.format == HQ_FMT_Q2_K) {
    if ((reinterpret_cast<uintptr_t>(p.w) & 3u) != 0 || p.w_expert_stride % 4 != 0) return HQ_ERR_ALIGN;
    if (p.n_banks == 2 && (reinterpret_cast<uintptr_t>(p.w_up) & 3u) != 0) return HQ_ERR_ALIGN;
  } else if (p.format != HQ_FMT_Q6_K && p.format != HQ_FMT_Q3_K) {
    if ((reinterpret_cast<uintptr_t>(p.w) & 15u) != 0 || p.w_expert_stride % 16 != 0) return HQ_ERR_ALIGN;
    if (p.n_banks == 2 && (reinterpret_cast<uintptr_t>(p.w_up) & 15u) != 0) return HQ_ERR_ALIGN;
  }
  const int64_t items = (int64_t)n_y_max * ((p.n + kGmRows - 1) / kGmRows);
  if (items <= 0) return HQ_OK;
  switch (p.format) {
    case HQ_FMT_Q6_K: return launch_gm_fmt<HQ_FMT_Q6_K>(p, items, stream);
    case HQ_FMT_Q5_K: return launch_gm_fmt<HQ_FMT_Q5_K>(p, items, stream);
    case HQ_FMT_Q4_0: return launch_gm_fmt<HQ_FMT_Q4_0>(p, items, stream);
    case HQ_FMT_Q5_0: return launch_gm_fmt<HQ_FMT_Q5_0>(p, items, stream);
    case HQ_FMT_Q4_1: return launch_gm_fmt<HQ_FMT_Q4_1>(p, items, stream);
    case HQ_FMT_Q5_1: return launch_gm_fmt<HQ_FMT_Q5_1>(p, items, stream);
    case HQ_FMT_Q2_K: return launch_gm_fmt<HQ_FMT_Q2_K>(p, items, stream);
    case HQ_FMT_Q3_K: return launch_gm_fmt<HQ_FMT_Q3_K>(p, items, stream);
    default: return HQ_ERR_FORMAT;
  }
}

}  // namespace hq
