// Grouped expert GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), for
// prefill-sized token counts: out[rows of expert e] = act( x_rows . dequant(W[e])^T ).
//
// One persistent CTA per SM walks (token tile, feature tile) work items of the
// expert-sorted assignment list.  UMMA roles are swapped so the 128 TMEM lanes hold
// output FEATURES and the columns hold TOKENS: D[feature, token] = W_tile[128, K] .
// X_tile[128 tokens, K]^T.  Warp roles:
//   warp 0        MMA issuer (one elected lane): tcgen05.mma kind::f16, 128x128x16 per
//                 instruction, operands through shared-memory descriptors (K-major,
//                 128-byte swizzle), f32 accumulators in tensor memory, double buffered
//   warps 1-4     epilogue: tcgen05.ld the accumulators, bias, gated activation
//                 (gate/up from two banks, or interleaved rows), store
//   warps 5-20    producers: read the quantized weight tile straight from the
//                 reference's byte layout, expand it to f16 in registers and write the
//                 swizzled operand tile; gather the tile's f16 activation rows (token order
//                 -> expert order) straight into the second operand tile with cp.async
// Stage hand-off is by mbarrier: producers arrive on full[s] after a proxy fence, the
// MMA warp releases a stage with tcgen05.commit, accumulator buffers alternate
// between MMA and epilogue through acc_full / acc_empty.  Every wait is bounded.
//
// Tensor-core bound for large token counts; algorithmic flops per launch =
// 2 * rows * N * K (* 2 with a gate and an up bank).
//
// A second kernel further down (grouped_gemm_ts_kernel) does the same product with the expanded weights written
// to tensor memory instead of shared memory; GroupedParams::weights_in_tmem selects it for 128-token tiles.
#include "hq_common.cuh"
#include "hq_kernels.h"

namespace hq {

constexpr int kGgProducerWarps = 16;
constexpr int kGgThreads = (5 + kGgProducerWarps) * 32;
constexpr int kTileM = 128;   // features per tile (TMEM lanes)
constexpr int kTileK = 64;    // k per stage: 64 f16 = one 128-byte swizzle row
constexpr int kOperandBytes = 128 * kTileK * 2;  // 16 KiB per operand tile
constexpr uint32_t kGgSpin = 1u << 22;

// ---- tcgen05 wrappers -----------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
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
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory operand descriptor: K-major tile of 128-byte rows, 128-byte swizzle,
// 8-row groups 1024 bytes apart, descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFFu);         // start address, 16-byte units
  d |= (uint64_t)1 << 16;                              // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                    // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                              // descriptor version
  d |= (uint64_t)2 << 61;                              // SWIZZLE_128B
  return d;
}
// kind::f16 instruction descriptor: f32 accumulate, f16 x f16, both K-major, M = 128, N = 128
// (both operands must have the same 16-bit format: f16 weights beside bf16 activations in one instruction
// raise an illegal-instruction error on B200, so bf16 activations are converted while their tile is written)
__device__ __forceinline__ uint32_t make_idesc_f16(int tile_n) {
  return (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(tile_n >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
}

// byte offset of 16-byte chunk `c` (0..7) of row `r` inside a swizzled 128 x 64 f16 operand tile
__device__ __forceinline__ uint32_t swz(int r, int c) {
  return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4));
}

// TN = tokens per tile (TMEM columns per accumulator): 128, or 256 when experts hold enough rows to fill it
template <int NB, int TN>
struct GgSmem {
  static constexpr int B_BYTES = TN * kTileK * 2;
  static constexpr int STAGE_BYTES = NB * kOperandBytes + B_BYTES;   // A bank(s) then B
  static constexpr int NSTAGE = (220 * 1024) / STAGE_BYTES > 6 ? 6 : (220 * 1024) / STAGE_BYTES;
  static constexpr int NBUF = (2 * NB * TN <= 512) ? 2 : 1;          // accumulator buffers in tensor memory
  static constexpr int OFF_BAR = NSTAGE * STAGE_BYTES;
  static constexpr int TOTAL = OFF_BAR + (2 * NSTAGE + 4) * 8 + 16 + 1024;  // + alignment slack
};

// ---- operand production, split in two halves so the global loads of the next stage are in flight while
// this stage is converted: fetch_a issues the loads into registers, emit_* converts to f16.  A thread owns 16
// consecutive k (quarter `q` of the stage's 64) of one weight row: two 16-byte chunks, natural k order.
struct RawA {
  uint4 hdr;          // Q4_K: super-block header {d, dmin, 12 scale bytes}; Q8_0: .x = fifth payload word
  uint4 q;            // Q4_K: 16 nibble bytes; FP8: 16 codes; MXFP4: .x/.y = 8 nibble bytes; Q8_0: payload words
  uint32_t aux;       // FP8: relative block scale (f32 bits); MXFP4: e8m0 byte; Q8_0: d (f16 bits) | shift << 16
  uint4 ext;          // Q6_K: .x / .y = fifth word of the low-nibble / high-bit bytes, .z = d (f16 bits) |
                      // scale byte << 16, .w = shifts (low-nibble bytes | high-bit bytes << 8); Q5_K: the 16 bytes
                      // of fifth bits; Q5_0 / Q5_1: .x = the 16 fifth bits of this half block; Q3_K: as Q6_K with
                      // the code words in q and the hmask words in hdr, .z = d | 6-bit scale << 16
};

template <int FMT>
__device__ __forceinline__ void fetch_a(RawA& r, const uint8_t* row_base, const uint8_t* scale_row, const float* rel,
                                        int k0, int q) {
  if (FMT == HQ_FMT_Q4_K) {
    // sub-blocks 2c and 2c+1 share 32 nibble bytes; quarters 0,1 are the low nibbles, 2,3 the high nibbles
    const int sb = k0 >> 8, c = (k0 & 255) >> 6;
    const uint8_t* blk = row_base + 144 * sb;
    r.hdr = __ldg(reinterpret_cast<const uint4*>(blk));
    r.q = __ldg(reinterpret_cast<const uint4*>(blk + 16 + 32 * c + 16 * (q & 1)));
  } else if (FMT == HQ_FMT_FP8_BLOCK) {
    r.q = __ldg(reinterpret_cast<const uint4*>(row_base + k0 + 16 * q));
    r.aux = __float_as_uint(__ldg(rel + k0 / 128));
  } else if (FMT == HQ_FMT_Q6_K) {
    // 16 consecutive k inside a 210-byte super-block: position 128 h + 32 j + 16 s + t (t = 0..15) takes the low
    // (j < 2) or high nibbles of ql[64 h + 32 (j & 1) + 16 s + t] and bits 2j, 2j + 1 of qh[32 h + 16 s + t], with
    // scale 8 h + 2 j + s.  Blocks start on 2-byte boundaries: aligned words, five when the run starts in the
    // middle of a word (the extra bytes are inside the block or, in front of it, inside the tensor)
    const int pos = (k0 & 255) + 16 * q;
    const int h = pos >> 7, j = (pos >> 5) & 3, sx = (pos >> 4) & 1;
    const uint8_t* blk = row_base + 210 * (k0 >> 8);
    const uint8_t* pl = blk + 64 * h + 32 * (j & 1) + 16 * sx;
    const uint8_t* ph = blk + 128 + 32 * h + 16 * sx;
    const uint32_t ml = (uint32_t)(reinterpret_cast<uintptr_t>(pl) & 2u), mh = (uint32_t)(reinterpret_cast<uintptr_t>(ph) & 2u);
    const uint32_t* wl = reinterpret_cast<const uint32_t*>(pl - ml);
    const uint32_t* wh = reinterpret_cast<const uint32_t*>(ph - mh);
    r.q = make_uint4(__ldg(wl), __ldg(wl + 1), __ldg(wl + 2), __ldg(wl + 3));
    r.hdr = make_uint4(__ldg(wh), __ldg(wh + 1), __ldg(wh + 2), __ldg(wh + 3));
    r.ext.x = ml ? __ldg(wl + 4) : 0u;
    r.ext.y = mh ? __ldg(wh + 4) : 0u;
    r.ext.z = (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(blk + 208)) |
              ((uint32_t)__ldg(blk + 192 + 8 * h + 2 * j + sx) << 16);
    r.ext.w = (ml << 3) | (mh << 11);
    r.aux = (uint32_t)j;
  } else if (FMT == HQ_FMT_Q5_K) {
    // as Q4_K with 176-byte super-blocks {d, dmin, scales[12], qh[32], qs[128]}: quarter q of the 64 weights 64 c ..
    // takes nibble q / 2 of qs[32 c + 16 (q % 2) + t] and bit 2 c + q / 2 of qh[16 (q % 2) + t]
    const int sb = k0 >> 8, c = (k0 & 255) >> 6;
    const uint8_t* blk = row_base + 176 * sb;
    r.hdr = __ldg(reinterpret_cast<const uint4*>(blk));
    r.q = __ldg(reinterpret_cast<const uint4*>(blk + 48 + 32 * c + 16 * (q & 1)));
    r.ext = __ldg(reinterpret_cast<const uint4*>(blk + 16 + 16 * (q & 1)));
  } else if (FMT == HQ_FMT_Q4_0 || FMT == HQ_FMT_Q5_0 || FMT == HQ_FMT_Q4_1 || FMT == HQ_FMT_Q5_1) {
    // half a block of 32 {f16 d, [f16 m,] [u32 qh,] qs[16]}: weight i < 16 is the low nibble of qs[i], weight i + 16
    // its high nibble, so both halves read the same 16 bytes.  Blocks start on 2-byte boundaries: aligned words, five
    // when the bytes start in the middle of a word (the fifth then shares its word with the block's last bytes)
    constexpr bool FIVE = FMT == HQ_FMT_Q5_0 || FMT == HQ_FMT_Q5_1;
    constexpr bool MIN = FMT == HQ_FMT_Q4_1 || FMT == HQ_FMT_Q5_1;
    constexpr int BB = 18 + (FIVE ? 4 : 0) + (MIN ? 2 : 0);
    const uint8_t* blk = row_base + BB * ((k0 >> 5) + (q >> 1));
    const uint8_t* pay = blk + (BB - 16);
    const uint32_t mis = (uint32_t)(reinterpret_cast<uintptr_t>(pay) & 2u);
    const uint32_t* wp = reinterpret_cast<const uint32_t*>(pay - mis);
    r.q = make_uint4(__ldg(wp), __ldg(wp + 1), __ldg(wp + 2), __ldg(wp + 3));
    r.hdr.x = mis ? __ldg(wp + 4) : 0u;
    r.aux = (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(blk)) | (mis << 19) | ((uint32_t)(q & 1) << 24);
    if (MIN) r.hdr.y = (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(blk + 2));
    if (FIVE) r.ext.x = (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(blk + (MIN ? 4 : 2) + 2 * (q & 1)));
  } else if (FMT == HQ_FMT_Q2_K) {
    // 16 consecutive k of an 84-byte super-block {scales[16], qs[64], d, dmin} (4-byte aligned): position
    // 128 h + 32 j + 16 u + t takes bits 2 j, 2 j + 1 of qs[32 h + 16 u + t], group 8 h + 2 j + u
    const int pos = (k0 & 255) + 16 * q;
    const int h = pos >> 7, j = (pos >> 5) & 3, u = (pos >> 4) & 1;
    const uint8_t* blk = row_base + 84 * (k0 >> 8);
    const uint32_t* wq = reinterpret_cast<const uint32_t*>(blk + 16 + 32 * h + 16 * u);
    r.q = make_uint4(__ldg(wq), __ldg(wq + 1), __ldg(wq + 2), __ldg(wq + 3));
    r.hdr.x = __ldg(reinterpret_cast<const uint32_t*>(blk + 80));
    r.aux = (uint32_t)__ldg(blk + 8 * h + 2 * j + u) | ((uint32_t)j << 8);
  } else if (FMT == HQ_FMT_Q3_K) {
    // 16 consecutive k of a 110-byte super-block {hmask[32], qs[64], scales[12], d} (2-byte aligned, words fetched
    // as for Q6_K): position 128 h + 32 j + 16 u + t takes bits 2 j, 2 j + 1 of qs[32 h + 16 u + t] and bit 4 h + j
    // of hmask[16 u + t]; the 6-bit scale of group 4 a + b = 8 h + 2 j + u is a nibble of byte 4 (a % 2) + b (low for
    // a < 2) with bits 2 a, 2 a + 1 of byte 8 + b on top
    const int pos = (k0 & 255) + 16 * q;
    const int h = pos >> 7, j = (pos >> 5) & 3, u = (pos >> 4) & 1;
    const uint8_t* blk = row_base + 110 * (k0 >> 8);
    const uint8_t* pl = blk + 32 + 32 * h + 16 * u;
    const uint8_t* ph = blk + 16 * u;
    const uint32_t ml = (uint32_t)(reinterpret_cast<uintptr_t>(pl) & 2u), mh = (uint32_t)(reinterpret_cast<uintptr_t>(ph) & 2u);
    const uint32_t* wl = reinterpret_cast<const uint32_t*>(pl - ml);
    const uint32_t* wh = reinterpret_cast<const uint32_t*>(ph - mh);
    r.q = make_uint4(__ldg(wl), __ldg(wl + 1), __ldg(wl + 2), __ldg(wl + 3));
    r.hdr = make_uint4(__ldg(wh), __ldg(wh + 1), __ldg(wh + 2), __ldg(wh + 3));
    r.ext.x = ml ? __ldg(wl + 4) : 0u;
    r.ext.y = mh ? __ldg(wh + 4) : 0u;
    const int s16 = 8 * h + 2 * j + u, a = s16 >> 2, b = s16 & 3;
    const uint32_t nib = __ldg(blk + 96 + 4 * (a & 1) + b), top = __ldg(blk + 104 + b);
    const uint32_t sc6 = (a < 2 ? (nib & 15u) : (nib >> 4)) | (((top >> (2 * a)) & 3u) << 4);
    r.ext.z = (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(blk + 108)) | (sc6 << 16);
    r.ext.w = (ml << 3) | (mh << 11);
    r.aux = (uint32_t)j | ((uint32_t)(4 * h + j) << 8);
  } else if (FMT == HQ_FMT_Q8_0) {
    // half a 34-byte block: 16 int8 behind the block's f16 d.  Blocks start on 2-byte boundaries (rows on 4-byte
    // ones), so the payload is fetched as aligned words -- five when it starts in the middle of a word, in which
    // case the fifth still lies inside the block -- and shifted into place by emit_q8_0
    const uint8_t* blk = row_base + 34 * ((k0 >> 5) + (q >> 1));
    const uint8_t* pay = blk + 2 + 16 * (q & 1);
    const uint32_t mis = (uint32_t)(reinterpret_cast<uintptr_t>(pay) & 2u);
    const uint32_t* wp = reinterpret_cast<const uint32_t*>(pay - mis);
    r.q = make_uint4(__ldg(wp), __ldg(wp + 1), __ldg(wp + 2), __ldg(wp + 3));
    r.hdr.x = mis ? __ldg(wp + 4) : 0u;
    r.aux = (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(blk)) | (mis << 19);
  } else {
    const int blk = (k0 >> 5) + (q >> 1);
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(row_base + 16 * blk + 8 * (q & 1)));
    r.q.x = v.x;
    r.q.y = v.y;
    r.aux = __ldg(scale_row + blk);
  }
}

// Q4_K: w = code * d1 - m1 with d1 = d * sc, m1 = dmin * m.  Codes are extracted as the f16 pair
// (1024 + e0, 1024 + e1) with one permute (bytes {code, 0x64}); the offset and the min go into one constant
// C = -(m1 + 1024 * d1).  d1 and C are each split into a leading f16 and its remainder, so
// w = fma(p, dh, Ch) + fma(p, dl, Cl) carries only the final roundings of weight-sized quantities.
__device__ __forceinline__ void emit_q4_k(const RawA& r, int k0, int q, uint32_t (&out)[8]) {
  const int c = (k0 & 255) >> 6;
  const int hi = q >> 1;
  const int j = 2 * c + hi;
  uint32_t s, m;
  if (j < 4) {
    s = (r.hdr.y >> (8 * j)) & 63u;
    m = (r.hdr.z >> (8 * j)) & 63u;
  } else {
    const int jj = j - 4;
    s = ((r.hdr.w >> (8 * jj)) & 0xFu) | (((r.hdr.y >> (8 * jj + 6)) & 3u) << 4);
    m = ((r.hdr.w >> (8 * jj + 4)) & 0xFu) | (((r.hdr.z >> (8 * jj + 6)) & 3u) << 4);
  }
  const float d1 = half_bits_to_float(r.hdr.x) * (float)s;
  const float cc = -fmaf(1024.f, d1, half_bits_to_float(r.hdr.x >> 16) * (float)m);
  const __half dh = __float2half_rn(d1), ch = __float2half_rn(cc);
  const __half2 dh2 = __half2half2(dh), ch2 = __half2half2(ch);
  const __half2 dl2 = __float2half2_rn(d1 - __half2float(dh));
  const __half2 cl2 = __float2half2_rn(cc - __half2float(ch));
  const uint32_t qw[4] = {r.q.x, r.q.y, r.q.z, r.q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t vm = (hi ? (qw[i] >> 4) : qw[i]) & 0x0F0F0F0Fu;
    uint32_t p01 = __byte_perm(vm, 0x64646464u, 0x4140);   // f16 pair (1024 + e0, 1024 + e1)
    uint32_t p23 = __byte_perm(vm, 0x64646464u, 0x4342);
    const __half2 h01 = *reinterpret_cast<__half2*>(&p01), h23 = *reinterpret_cast<__half2*>(&p23);
    __half2 w01 = __hadd2(__hfma2(h01, dh2, ch2), __hfma2(h01, dl2, cl2));
    __half2 w23 = __hadd2(__hfma2(h23, dh2, ch2), __hfma2(h23, dl2, cl2));
    out[2 * i] = *reinterpret_cast<uint32_t*>(&w01);
    out[2 * i + 1] = *reinterpret_cast<uint32_t*>(&w23);
  }
}

// Q8_0: w = d * q.  Bytes q + 128 become the f16 pair (1024 + u0, 1024 + u1) with one permute, 1152 is subtracted
// exactly, and the product with the block's f16 d is rounded once to f16 (relative error <= 2^-11 per weight).
__device__ __forceinline__ void emit_q8_0(const RawA& r, uint32_t (&out)[8]) {
  const uint32_t sh = (r.aux >> 16) & 31u;          // 0 or 16
  const uint32_t raw[5] = {r.q.x, r.q.y, r.q.z, r.q.w, r.hdr.x};
  const uint32_t d16 = r.aux & 0xFFFFu;
  const uint32_t dd = d16 | (d16 << 16);
  const __half2 d2 = *reinterpret_cast<const __half2*>(&dd);
  const uint32_t off = 0x64806480u;                  // f16 1152 twice
  const __half2 o2 = *reinterpret_cast<const __half2*>(&off);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t w = __funnelshift_r(raw[i], raw[i + 1], sh) ^ 0x80808080u;
    uint32_t p01 = __byte_perm(w, 0x64646464u, 0x4140);
    uint32_t p23 = __byte_perm(w, 0x64646464u, 0x4342);
    __half2 w01 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&p01), o2), d2);
    __half2 w23 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&p23), o2), d2);
    out[2 * i] = *reinterpret_cast<uint32_t*>(&w01);
    out[2 * i + 1] = *reinterpret_cast<uint32_t*>(&w23);
  }
}

// Q6_K: w = d * scale * (q - 32).  The 6-bit codes are assembled bytewise (nibble | two high bits << 4), become the
// f16 pair (1024 + q0, 1024 + q1) with one permute, 1056 is subtracted exactly, and the product with d * scale
// (computed in f32, rounded to f16) is rounded once more: two roundings of 2^-11 per weight.
__device__ __forceinline__ void emit_q6_k(const RawA& r, uint32_t (&out)[8]) {
  const uint32_t shl = r.ext.w & 31u, shh = (r.ext.w >> 8) & 31u;   // 0 or 16
  const uint32_t j = r.aux;
  const uint32_t lo[5] = {r.q.x, r.q.y, r.q.z, r.q.w, r.ext.x};
  const uint32_t hi[5] = {r.hdr.x, r.hdr.y, r.hdr.z, r.hdr.w, r.ext.y};
  const float ds = half_bits_to_float(r.ext.z & 0xFFFFu) * (float)(int)(int8_t)((r.ext.z >> 16) & 0xFFu);
  const __half2 ds2 = __float2half2_rn(ds);
  const uint32_t off = 0x64206420u;                  // f16 1056 twice
  const __half2 o2 = *reinterpret_cast<const __half2*>(&off);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t lw = __funnelshift_r(lo[i], lo[i + 1], shl);
    const uint32_t hw = __funnelshift_r(hi[i], hi[i + 1], shh);
    const uint32_t nib = (j < 2 ? lw : (lw >> 4)) & 0x0F0F0F0Fu;
    const uint32_t w6 = nib | (((hw >> (2 * j)) & 0x03030303u) << 4);
    uint32_t p01 = __byte_perm(w6, 0x64646464u, 0x4140);
    uint32_t p23 = __byte_perm(w6, 0x64646464u, 0x4342);
    __half2 w01 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&p01), o2), ds2);
    __half2 w23 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&p23), o2), ds2);
    out[2 * i] = *reinterpret_cast<uint32_t*>(&w01);
    out[2 * i + 1] = *reinterpret_cast<uint32_t*>(&w23);
  }
}

// Q5_K: w = code * d1 - m1 as for Q4_K, the 5-bit code = nibble | fifth bit << 4.
__device__ __forceinline__ void emit_q5_k(const RawA& r, int k0, int q, uint32_t (&out)[8]) {
  const int c = (k0 & 255) >> 6;
  const int hi = q >> 1;
  const int j = 2 * c + hi;
  uint32_t s, m;
  if (j < 4) {
    s = (r.hdr.y >> (8 * j)) & 63u;
    m = (r.hdr.z >> (8 * j)) & 63u;
  } else {
    const int jj = j - 4;
    s = ((r.hdr.w >> (8 * jj)) & 0xFu) | (((r.hdr.y >> (8 * jj + 6)) & 3u) << 4);
    m = ((r.hdr.w >> (8 * jj + 4)) & 0xFu) | (((r.hdr.z >> (8 * jj + 6)) & 3u) << 4);
  }
  const float d1 = half_bits_to_float(r.hdr.x) * (float)s;
  const float cc = -fmaf(1024.f, d1, half_bits_to_float(r.hdr.x >> 16) * (float)m);
  const __half dh = __float2half_rn(d1), ch = __float2half_rn(cc);
  const __half2 dh2 = __half2half2(dh), ch2 = __half2half2(ch);
  const __half2 dl2 = __float2half2_rn(d1 - __half2float(dh));
  const __half2 cl2 = __float2half2_rn(cc - __half2float(ch));
  const uint32_t qw[4] = {r.q.x, r.q.y, r.q.z, r.q.w};
  const uint32_t hw[4] = {r.ext.x, r.ext.y, r.ext.z, r.ext.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t vm = ((hi ? (qw[i] >> 4) : qw[i]) & 0x0F0F0F0Fu) | (((hw[i] >> j) & 0x01010101u) << 4);
    uint32_t p01 = __byte_perm(vm, 0x64646464u, 0x4140);   // f16 pair (1024 + e0, 1024 + e1)
    uint32_t p23 = __byte_perm(vm, 0x64646464u, 0x4342);
    const __half2 h01 = *reinterpret_cast<__half2*>(&p01), h23 = *reinterpret_cast<__half2*>(&p23);
    __half2 w01 = __hadd2(__hfma2(h01, dh2, ch2), __hfma2(h01, dl2, cl2));
    __half2 w23 = __hadd2(__hfma2(h23, dh2, ch2), __hfma2(h23, dl2, cl2));
    out[2 * i] = *reinterpret_cast<uint32_t*>(&w01);
    out[2 * i + 1] = *reinterpret_cast<uint32_t*>(&w23);
  }
}

// Q4_0: w = d * (q - 8); Q5_0: w = d * (q - 16); Q4_1 / Q5_1: w = d * q + m; q = nibble [| fifth bit << 4].  The
// codes become the f16 pair (1024 + q0, 1024 + q1) with one permute, 1024 + zero point is subtracted exactly, and the
// product with the block's f16 d (plus m, in one fused multiply-add) is rounded once to f16.
template <int FMT>
__device__ __forceinline__ void emit_q4_0_q5_0(const RawA& r, uint32_t (&out)[8]) {
  constexpr bool FIVE = FMT == HQ_FMT_Q5_0 || FMT == HQ_FMT_Q5_1;
  constexpr bool MIN = FMT == HQ_FMT_Q4_1 || FMT == HQ_FMT_Q5_1;
  const uint32_t sh = (r.aux >> 16) & 31u;           // 0 or 16
  const uint32_t half = (r.aux >> 24) & 1u;
  const uint32_t raw[5] = {r.q.x, r.q.y, r.q.z, r.q.w, r.hdr.x};
  const uint32_t d16 = r.aux & 0xFFFFu;
  const uint32_t dd = d16 | (d16 << 16);
  const __half2 d2 = *reinterpret_cast<const __half2*>(&dd);
  const uint32_t m16 = MIN ? (r.hdr.y & 0xFFFFu) : 0u;
  const uint32_t mm = m16 | (m16 << 16);
  const __half2 m2 = *reinterpret_cast<const __half2*>(&mm);
  const uint32_t off = MIN ? 0x64006400u : (FMT == HQ_FMT_Q4_0 ? 0x64086408u : 0x64106410u);   // f16 1024 + zero, twice
  const __half2 o2 = *reinterpret_cast<const __half2*>(&off);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t w = __funnelshift_r(raw[i], raw[i + 1], sh);
    uint32_t vm = (half ? (w >> 4) : w) & 0x0F0F0F0Fu;
    if (FIVE)   // four bits -> bit 4 of four bytes: x * 0x00204081 puts bit c of x at bit 8 c
      vm |= ((((r.ext.x >> (4 * i)) & 0xFu) * 0x00204081u) & 0x01010101u) << 4;
    uint32_t p01 = __byte_perm(vm, 0x64646464u, 0x4140);
    uint32_t p23 = __byte_perm(vm, 0x64646464u, 0x4342);
    const __half2 q01 = __hsub2(*reinterpret_cast<__half2*>(&p01), o2), q23 = __hsub2(*reinterpret_cast<__half2*>(&p23), o2);
    __half2 w01 = MIN ? __hfma2(q01, d2, m2) : __hmul2(q01, d2);
    __half2 w23 = MIN ? __hfma2(q23, d2, m2) : __hmul2(q23, d2);
    out[2 * i] = *reinterpret_cast<uint32_t*>(&w01);
    out[2 * i + 1] = *reinterpret_cast<uint32_t*>(&w23);
  }
}

// Q2_K: w = code * d1 - m1 with d1 = d * (s & 15), m1 = dmin * (s >> 4), in the split f16 arithmetic of emit_q4_k.
__device__ __forceinline__ void emit_q2_k(const RawA& r, uint32_t (&out)[8]) {
  const uint32_t j = (r.aux >> 8) & 3u, sc = r.aux & 0xFFu;
  const float d1 = half_bits_to_float(r.hdr.x) * (float)(sc & 15u);
  const float cc = -fmaf(1024.f, d1, half_bits_to_float(r.hdr.x >> 16) * (float)(sc >> 4));
  const __half dh = __float2half_rn(d1), ch = __float2half_rn(cc);
  const __half2 dh2 = __half2half2(dh), ch2 = __half2half2(ch);
  const __half2 dl2 = __float2half2_rn(d1 - __half2float(dh));
  const __half2 cl2 = __float2half2_rn(cc - __half2float(ch));
  const uint32_t qw[4] = {r.q.x, r.q.y, r.q.z, r.q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t vm = (qw[i] >> (2 * j)) & 0x03030303u;
    uint32_t p01 = __byte_perm(vm, 0x64646464u, 0x4140);   // f16 pair (1024 + e0, 1024 + e1)
    uint32_t p23 = __byte_perm(vm, 0x64646464u, 0x4342);
    const __half2 h01 = *reinterpret_cast<__half2*>(&p01), h23 = *reinterpret_cast<__half2*>(&p23);
    __half2 w01 = __hadd2(__hfma2(h01, dh2, ch2), __hfma2(h01, dl2, cl2));
    __half2 w23 = __hadd2(__hfma2(h23, dh2, ch2), __hfma2(h23, dl2, cl2));
    out[2 * i] = *reinterpret_cast<uint32_t*>(&w01);
    out[2 * i + 1] = *reinterpret_cast<uint32_t*>(&w23);
  }
}

// Q3_K: w = d * (scale - 32) * (q - 4), q = two code bits | hmask bit << 2: as emit_q6_k with 1028 subtracted.
__device__ __forceinline__ void emit_q3_k(const RawA& r, uint32_t (&out)[8]) {
  const uint32_t shl = r.ext.w & 31u, shh = (r.ext.w >> 8) & 31u;   // 0 or 16
  const uint32_t j = r.aux & 3u, hbit = (r.aux >> 8) & 7u;
  const uint32_t lo[5] = {r.q.x, r.q.y, r.q.z, r.q.w, r.ext.x};
  const uint32_t hi[5] = {r.hdr.x, r.hdr.y, r.hdr.z, r.hdr.w, r.ext.y};
  const float ds = half_bits_to_float(r.ext.z & 0xFFFFu) * (float)((int)((r.ext.z >> 16) & 0xFFu) - 32);
  const __half2 ds2 = __float2half2_rn(ds);
  const uint32_t off = 0x64046404u;                  // f16 1028 twice
  const __half2 o2 = *reinterpret_cast<const __half2*>(&off);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t lw = __funnelshift_r(lo[i], lo[i + 1], shl);
    const uint32_t hw = __funnelshift_r(hi[i], hi[i + 1], shh);
    const uint32_t w3 = ((lw >> (2 * j)) & 0x03030303u) | (((hw >> hbit) & 0x01010101u) << 2);
    uint32_t p01 = __byte_perm(w3, 0x64646464u, 0x4140);
    uint32_t p23 = __byte_perm(w3, 0x64646464u, 0x4342);
    __half2 w01 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&p01), o2), ds2);
    __half2 w23 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&p23), o2), ds2);
    out[2 * i] = *reinterpret_cast<uint32_t*>(&w01);
    out[2 * i + 1] = *reinterpret_cast<uint32_t*>(&w23);
  }
}

// e4m3 -> f16 is exact; the block's scale relative to the largest scale of its 128-row block (<= 1) is folded
// in here, the largest scale itself multiplies the accumulator in the epilogue.
__device__ __forceinline__ void emit_fp8(const RawA& r, uint32_t (&out)[8]) {
  const uint32_t w[4] = {r.q.x, r.q.y, r.q.z, r.q.w};
  const __half2 r2 = __float2half2_rn(__uint_as_float(r.aux));
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t lo, hi;
    asm("{\n"
        ".reg .b16 l, h;\n"
        "mov.b32 {l, h}, %2;\n"
        "cvt.rn.f16x2.e4m3x2 %0, l;\n"
        "cvt.rn.f16x2.e4m3x2 %1, h;\n"
        "}\n"
        : "=r"(lo), "=r"(hi)
        : "r"(w[i]));
    __half2 l2 = __hmul2(*reinterpret_cast<__half2*>(&lo), r2);
    __half2 h2 = __hmul2(*reinterpret_cast<__half2*>(&hi), r2);
    out[2 * i] = *reinterpret_cast<uint32_t*>(&l2);
    out[2 * i + 1] = *reinterpret_cast<uint32_t*>(&h2);
  }
}

// MXFP4: e2m1 pairs -> f16x2 (hardware conversion, low nibble = even element = low half), times 2^(e-127) as
// an exact f16 power of two.  e = 0 decodes to a zero scale (the reference's table builds the scale from the
// bits e << 23).  The f16 operand covers block scales 2^-14 .. 2^13 (e = 113 .. 140); a block outside that
// range is expanded as zero and the caller raises HQ_DEV_SCALE_RANGE, so a bank with such blocks has to stay on
// the decode kernel, which applies the scale in f32.
__device__ __forceinline__ bool emit_mxfp4(const RawA& r, uint32_t (&out)[8]) {
  const uint32_t e = r.aux;
  const bool in_range = (e == 0) || (e >= 113 && e <= 140);   // 2^-14 .. 2^13: products stay finite in f16
  const uint32_t ef = (e >= 113 && e <= 140) ? (e - 112) : 0u;  // f16 exponent field of 2^(e-127)
  const uint32_t sc16 = ef << 10;
  const uint32_t sc2 = sc16 | (sc16 << 16);
  const __half2 s2 = *reinterpret_cast<const __half2*>(&sc2);
  const uint32_t w[2] = {r.q.x, r.q.y};
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint32_t h[4];
    asm("{\n"
        ".reg .b8 b0, b1, b2, b3;\n"
        "mov.b32 {b0, b1, b2, b3}, %4;\n"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n"
        "cvt.rn.f16x2.e2m1x2 %3, b3;\n"
        "}\n"
        : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
        : "r"(w[i]));
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      __half2 v = __hmul2(*reinterpret_cast<__half2*>(&h[b]), s2);
      out[4 * i + b] = *reinterpret_cast<uint32_t*>(&v);
    }
  }
  return in_range;
}

__device__ __forceinline__ void store_chunks(uint8_t* tile, int r, int c0, const uint32_t (&v)[8]) {
#pragma unroll
  for (int c = 0; c < 2; ++c)
    *reinterpret_cast<uint4*>(tile + swz(r, c0 + c)) = make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
}

__device__ __forceinline__ float gg_gated(float g, float u, const hq_act_args& a) {
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

struct GgTile {
  int expert, row_start, count, n0;
};

template <int TN>
__device__ __forceinline__ GgTile gg_tile(const GroupedParams& p, int w, int n_nt) {
  constexpr int kTileN = TN;
  GgTile t;
  const int tt = w / n_nt;
  t.n0 = (w - tt * n_nt) * kTileM;
  if (p.tiles != nullptr) {
    t.expert = p.tiles[2 * tt];
    t.row_start = p.tiles[2 * tt + 1];
    t.count = min(kTileN, p.expert_bounds[t.expert + 1] - t.row_start);
  } else {
    t.expert = 0;
    t.row_start = kTileN * tt;
    t.count = min(kTileN, p.m - t.row_start);
  }
  return t;
}

template <int FMT, int NB, int TN>
__global__ void __launch_bounds__(kGgThreads, 1) grouped_gemm_kernel(const GroupedParams p) {
  using L = GgSmem<NB, TN>;
  constexpr int NSTAGE = L::NSTAGE;
  constexpr int NBUF = L::NBUF;
  constexpr int kTileN = TN;
  extern __shared__ uint8_t smem_raw[];
  // operand tiles need 1024-byte alignment for the 128-byte swizzle
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* empty = full + NSTAGE;
  uint64_t* acc_full = empty + NSTAGE;     // [2]
  uint64_t* acc_empty = acc_full + 2;      // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_nt = (p.n + kTileM - 1) / kTileM;
  const int n_tt = p.tiles != nullptr ? p.tile_count[0] : (p.m + kTileN - 1) / kTileN;
  const int total = n_tt * n_nt;
  const int n_ks = p.k / kTileK;

  if (tid == 0) {
    for (int s = 0; s < NSTAGE; ++s) {
      mbar_init(&full[s], kGgProducerWarps);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // =========================== MMA issuer ======================================
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(TN);
      uint32_t spin = kGgSpin;
      int it = 0, tcount = 0;
      for (int w = blockIdx.x; w < total; w += gridDim.x, ++tcount) {
        const int buf = tcount % NBUF;
        if (tcount >= NBUF) {
          if (!mbar_wait_backoff(&acc_empty[buf], ((tcount / NBUF) - 1) & 1, spin)) {
            report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 300 + buf);
            spin = 1;
          }
        }
        tc_fence_after();
        const uint32_t d0 = tmem_base + (uint32_t)(buf * NB * kTileN);
        for (int ks = 0; ks < n_ks; ++ks, ++it) {
          const int s = it % NSTAGE;
          if (!mbar_wait_backoff(&full[s], (it / NSTAGE) & 1, spin)) {
            report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 310 + s);
            spin = 1;
          }
          tc_fence_after();
          const uint32_t stage = smem_u32(smem + s * L::STAGE_BYTES);
          const uint64_t bdesc = make_smem_desc(stage + NB * kOperandBytes);
#pragma unroll
          for (int bank = 0; bank < NB; ++bank) {
            const uint64_t adesc = make_smem_desc(stage + bank * kOperandBytes);
#pragma unroll
            for (int kk = 0; kk < kTileK / 16; ++kk) {
              // 16 k per instruction = 32 bytes along the swizzled row: advance the start address by 2 units
              tc_mma_f16(d0 + bank * kTileN, adesc + 2 * kk, bdesc + 2 * kk, idesc, (ks > 0 || kk > 0) ? 1u : 0u);
            }
          }
          tc_commit(&empty[s]);     // stage is free once these MMAs have read it
        }
        tc_commit(&acc_full[buf]);  // accumulators complete
      }
    }
    __syncwarp();
  } else if (warp <= 4) {
    // =========================== epilogue ========================================
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    uint32_t spin = kGgSpin;
    bool failed = false;
    int tcount = 0;
    for (int w = blockIdx.x; w < total; w += gridDim.x, ++tcount) {
      const GgTile t = gg_tile<TN>(p, w, n_nt);
      const int buf = tcount % NBUF;
      if (!mbar_wait_backoff(&acc_full[buf], (tcount / NBUF) & 1, spin)) {
        if (lane == 0) report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 400 + buf);
        spin = 1;
        failed = true;                 // nothing is stored once a wait has run out
      }
      tc_fence_after();
      const int n = t.n0 + 32 * q + lane;       // feature owned by this thread
      const bool n_ok = n < p.n;
      float bias0 = 0.f, bias1 = 0.f;
      if (n_ok && p.bias != nullptr) bias0 = load_as_float(p.bias, p.bias_dtype, (int64_t)t.expert * p.n + n);
      if (NB == 2 && n_ok && p.bias_up != nullptr)
        bias1 = load_as_float(p.bias_up, p.bias_dtype, (int64_t)t.expert * p.n + n);
      float sc0 = 1.f, sc1 = 1.f;
      if (FMT == HQ_FMT_FP8_BLOCK) {
        sc0 = __ldg(p.fp8_tile_scale + (int64_t)t.expert * p.fp8_nb + t.n0 / 128);
        if (NB == 2) sc1 = __ldg(p.fp8_tile_scale_up + (int64_t)t.expert * p.fp8_nb + t.n0 / 128);
      }
      const bool interleaved = NB == 1 && p.act.act != HQ_ACT_NONE;
      const int64_t out_n = interleaved ? (n >> 1) : n;
      const bool writer = n_ok && !failed && (!interleaved || (n & 1) == 0);
      const uint32_t taddr = tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(buf * NB * kTileN);
      // Output row of the token in column 32*cc + lane (-1 past the tile's tokens).  One coalesced load per
      // column group, issued a group ahead, then broadcast by shuffle: a load per stored element would
      // serialise the stores behind the load latency, since the compiler must assume y aliases y_rows.
      const int* __restrict__ yrows = p.y_rows;
      auto row_of = [&](int cc) -> int {
        const int col = 32 * cc + lane;
        if (cc >= kTileN / 32 || col >= t.count) return -1;
        const int sp = t.row_start + col;
        return yrows != nullptr ? __ldg(yrows + sp) : sp;
      };
      const int esz = dtype_size(p.y_dtype);
      char* const ybase = reinterpret_cast<char*>(p.y) + out_n * esz;
      const int64_t ystride_b = (int64_t)p.y_stride * esz;
      int myrow = row_of(0);
#pragma unroll 1
      for (int cc = 0; cc < kTileN / 32; ++cc) {
        if (32 * cc >= t.count) break;          // warp-uniform: no tokens in this column group
        uint32_t v0[32], v1[32];
        tmem_ld32(taddr + 32 * cc, v0);
        if (NB == 2) tmem_ld32(taddr + kTileN + 32 * cc, v1);
        const int nextrow = row_of(cc + 1);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float r = fmaf(__uint_as_float(v0[j]), sc0, bias0);
          if (NB == 2) {
            r = gg_gated(r, fmaf(__uint_as_float(v1[j]), sc1, bias1), p.act);
          } else if (interleaved) {
            const float partner = __shfl_xor_sync(0xffffffffu, r, 1);
            r = gg_gated(r, partner, p.act);
          }
          v0[j] = __float_as_uint(r);
        }
        auto store_group = [&](auto cvt) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int orow = __shfl_sync(0xffffffffu, myrow, j);
            if (writer && orow >= 0) {
              using T = decltype(cvt(0.f));
              *reinterpret_cast<T*>(ybase + orow * ystride_b) = cvt(__uint_as_float(v0[j]));
            }
          }
        };
        if (p.y_dtype == HQ_DT_BF16) store_group([](float f) { return __float2bfloat16_rn(f); });
        else if (p.y_dtype == HQ_DT_F16) store_group([](float f) { return __float2half_rn(f); });
        else store_group([](float f) { return f; });
        myrow = nextrow;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  } else {
    // =========================== producers ========================================
    const int ptid = tid - 5 * 32;            // 0..511
    const int r = ptid >> 2, q = ptid & 3;    // weight row and which 16-k quarter of the stage
    constexpr int BROWS = TN / 64;            // activation rows per thread (one 16-byte chunk of each)
    uint32_t spin = kGgSpin;

    // cursor over the flattened (tile, k stage) sequence of this CTA
    struct Cursor {
      int w, ks;
      const uint8_t *w0, *w1, *s0, *s1;
      const float *rel0, *rel1;
      bool n_ok;
      int64_t boff[BROWS];    // element offset of this thread's chunk in each of its activation rows, -1 = no row
    };
    auto open_tile = [&](Cursor& c) {
      const GgTile t = gg_tile<TN>(p, c.w, n_nt);
      const int n = t.n0 + r;
      c.n_ok = n < p.n;
      const int64_t wrow = (int64_t)t.expert * p.n + (c.n_ok ? n : 0);
      c.w0 = reinterpret_cast<const uint8_t*>(p.w) + wrow * p.w_row_bytes;
      c.w1 = NB == 2 ? reinterpret_cast<const uint8_t*>(p.w_up) + wrow * p.w_row_bytes : nullptr;
      c.s0 = c.s1 = nullptr;
      c.rel0 = c.rel1 = nullptr;
      if (FMT == HQ_FMT_MXFP4) {
        c.s0 = reinterpret_cast<const uint8_t*>(p.scales) + wrow * (p.k / 32);
        if (NB == 2) c.s1 = reinterpret_cast<const uint8_t*>(p.scales_up) + wrow * (p.k / 32);
      }
      if (FMT == HQ_FMT_FP8_BLOCK) {
        const int64_t g = ((int64_t)t.expert * p.fp8_nb + t.n0 / 128) * p.fp8_kb;
        c.rel0 = p.fp8_rel_scale + g;
        if (NB == 2) c.rel1 = p.fp8_rel_scale_up + g;
      }
#pragma unroll
      for (int j = 0; j < BROWS; ++j) {
        const int row = (ptid >> 3) + 64 * j;
        c.boff[j] = -1;
        if (row < t.count) {
          const int sp = t.row_start + row;
          c.boff[j] = (p.x_rows ? (int64_t)p.x_rows[sp] : (int64_t)sp) * p.x_stride + 8 * (ptid & 7);
        }
      }
    };
    auto fetch = [&](const Cursor& c, RawA (&ra)[NB]) {
      const int k0 = c.ks * kTileK;
      if (c.n_ok) {
        fetch_a<FMT>(ra[0], c.w0, c.s0, c.rel0, k0, q);
        if (NB == 2) fetch_a<FMT>(ra[NB - 1], c.w1, c.s1, c.rel1, k0, q);
      }
    };
    int waited = NSTAGE - 1;                  // stages up to this index are known to be free
    auto ensure_empty = [&](int j) {
      if (j > waited) {
        if (!mbar_wait(&empty[j % NSTAGE], ((j / NSTAGE) - 1) & 1, spin)) {
          if (lane == 0) report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 500 + j % NSTAGE);
          spin = 1;
        }
        waited = j;
      }
    };
    // activation rows (f16, gathered token order -> expert order): 16 bytes global -> shared per chunk without
    // passing through registers; a missing row is zero-filled
    auto copy_b = [&](const Cursor& c, int stage_index) {
      uint8_t* btile = smem + (stage_index % NSTAGE) * L::STAGE_BYTES + NB * kOperandBytes;
      const int k0 = c.ks * kTileK;
#pragma unroll
      for (int j = 0; j < BROWS; ++j) {
        const int row = (ptid >> 3) + 64 * j;
        const uint32_t dst = smem_u32(btile + swz(row, ptid & 7));
        const bool ok = c.boff[j] >= 0;
        const void* src = ok ? reinterpret_cast<const void*>(reinterpret_cast<const uint16_t*>(p.x) + c.boff[j] + k0)
                             : p.x;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(ok ? 16 : 0) : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };

    Cursor cur;
    cur.w = blockIdx.x;
    cur.ks = 0;
    // two register sets used alternately: the set being loaded for the next stage is never copied, so nothing
    // waits on those loads until the stage after is converted
    RawA ra0[NB], ra1[NB];
    bool live = cur.w < total;
    if (live) {
      open_tile(cur);
      fetch(cur, ra0);
      copy_b(cur, 0);
    }
    int it = 0;
    // one stage: start the next stage's loads into `ld`, convert this stage from `use`
    auto step = [&](RawA (&use)[NB], RawA (&ld)[NB]) {
      Cursor nxt = cur;
      bool next_live = true;
      if (cur.ks + 1 < n_ks) {
        nxt.ks = cur.ks + 1;
      } else {
        nxt.w = cur.w + gridDim.x;
        nxt.ks = 0;
        next_live = nxt.w < total;
        if (next_live) open_tile(nxt);
      }
      if (next_live) {
        fetch(nxt, ld);
        ensure_empty(it + 1);
        copy_b(nxt, it + 1);
      }
      ensure_empty(it);
      const int s = it % NSTAGE;
      uint8_t* stage = smem + s * L::STAGE_BYTES;
      const int k0 = cur.ks * kTileK;
      uint32_t v[8];
#pragma unroll
      for (int bank = 0; bank < NB; ++bank) {
        if (cur.n_ok) {
          if (FMT == HQ_FMT_Q4_K) {
            emit_q4_k(use[bank], k0, q, v);
          } else if (FMT == HQ_FMT_FP8_BLOCK) {
            emit_fp8(use[bank], v);
          } else if (FMT == HQ_FMT_Q8_0) {
            emit_q8_0(use[bank], v);
          } else if (FMT == HQ_FMT_Q6_K) {
            emit_q6_k(use[bank], v);
          } else if (FMT == HQ_FMT_Q5_K) {
            emit_q5_k(use[bank], k0, q, v);
          } else if (FMT == HQ_FMT_Q4_0 || FMT == HQ_FMT_Q5_0 || FMT == HQ_FMT_Q4_1 || FMT == HQ_FMT_Q5_1) {
            emit_q4_0_q5_0<FMT>(use[bank], v);
          } else if (FMT == HQ_FMT_Q2_K) {
            emit_q2_k(use[bank], v);
          } else if (FMT == HQ_FMT_Q3_K) {
            emit_q3_k(use[bank], v);
          } else {
            if (!emit_mxfp4(use[bank], v)) report_status(p.status, HQ_DEV_SCALE_RANGE, 600);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = 0u;
        }
        store_chunks(stage + bank * kOperandBytes, r, 2 * q, v);
      }
      // this stage's activation copies were issued one iteration ago; the next stage's may stay in flight
      if (next_live) asm volatile("cp.async.wait_group 1;" ::: "memory");
      else asm volatile("cp.async.wait_group 0;" ::: "memory");
      fence_proxy_async_smem();     // generic-proxy writes -> visible to the tensor core (async proxy)
      __syncwarp();
      if (lane == 0) mbar_arrive(&full[s]);
      ++it;
      cur = nxt;
      live = next_live;
    };
    while (live) {
      step(ra0, ra1);
      if (!live) break;
      step(ra1, ra0);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ================= weights through tensor memory ======================================================
// Second kernel for 128-token tiles.  The kernel above is bounded by shared-memory bandwidth: per 64-k stage
// the producers write both operand tiles and the tensor core reads both back.  Here the expanded weights never
// touch shared memory: a producer thread owns one weight row (one TMEM lane) for a whole stage, expands its 64
// weights in registers and writes them with tcgen05.st into a ring of A-operand stages in tensor memory; the MMA
// takes A from tensor memory and only the activation tile B from shared memory.  With a gate and an up bank a
// tile holds 64 features: lanes 16q..16q+15 of every 32-lane quarter q carry the gate rows, the next 16 lanes
// the up rows of the same features, so one MMA serves both banks, one accumulator set is enough (two buffers
// of 128 columns), and the gated activation pairs lanes 16 apart of one epilogue warp.
//   tensor memory: columns 0..255 two accumulator buffers, 256..511 eight A stages of 32 columns (64 f16)
//   warps 5..20: four groups of four warps (one per lane quarter); group j takes the stages it = j mod 4 of the
//   CTA's flattened (tile, k) sequence: expands A, copies the stage's activation rows, arrives on full[s]
constexpr int kTsACol0 = 256;                 // first tensor-memory column of the A ring
constexpr int kTsAStageCols = kTileK / 2;
// 128 tokens per tile.  (256-token tiles -- one accumulator buffer, six stages, an expanded stage serving twice
// the tokens -- were built and measured slower on every layer tried: 1.17 against 0.99 ms on the Q4_K layer.)
constexpr int kTsTokens = 128;
struct TsSmem {
  static constexpr int NSTAGE = 8;
  static constexpr int NBUF = 2;
  static constexpr int B_BYTES = kTsTokens * kTileK * 2;
  static constexpr int OFF_BAR = NSTAGE * B_BYTES;
  static constexpr int TOTAL = OFF_BAR + (2 * NSTAGE + 4) * 8 + 16 + 1024;
};

__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
      "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// raw bytes of one weight row for one 64-k stage
struct TsRaw {
  uint4 hdr;        // Q4_K: super-block header
  uint4 v[4];       // Q4_K: 32 nibble bytes in v[0..1]; MXFP4: two 16-byte blocks in v[0..1]; FP8: 64 codes
  uint32_t aux0;    // FP8: relative block scale (f32 bits); MXFP4: e8m0 byte of the first block
  uint32_t aux1;    // MXFP4: e8m0 byte of the second block
};
template <int FMT>
__device__ __forceinline__ void ts_fetch(TsRaw& r, const uint8_t* row_base, const uint8_t* scale_row, const float* rel,
                                         int k0) {
  if (FMT == HQ_FMT_Q4_K) {
    const uint8_t* blk = row_base + 144 * (k0 >> 8);
    const int c = (k0 & 255) >> 6;
    r.hdr = __ldg(reinterpret_cast<const uint4*>(blk));
    r.v[0] = __ldg(reinterpret_cast<const uint4*>(blk + 16 + 32 * c));
    r.v[1] = __ldg(reinterpret_cast<const uint4*>(blk + 32 + 32 * c));
  } else if (FMT == HQ_FMT_FP8_BLOCK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) r.v[i] = __ldg(reinterpret_cast<const uint4*>(row_base + k0 + 16 * i));
    r.aux0 = __float_as_uint(__ldg(rel + k0 / 128));
  } else {
    const int blk = k0 >> 5;
    r.v[0] = __ldg(reinterpret_cast<const uint4*>(row_base + 16 * blk));
    r.v[1] = __ldg(reinterpret_cast<const uint4*>(row_base + 16 * blk + 16));
    r.aux0 = __ldg(scale_row + blk);
    r.aux1 = __ldg(scale_row + blk + 1);
  }
}
// the 32 weights k0 + 32*half .. of the stage as 16 f16 pairs, natural k order
template <int FMT>
__device__ __forceinline__ bool ts_expand(const TsRaw& r, int k0, int half, uint32_t (&out)[16]) {
  bool ok = true;
  RawA a;
  uint32_t lo[8], hi[8];
  if (FMT == HQ_FMT_Q4_K) {
    a.hdr = r.hdr;
    a.q = r.v[0];
    emit_q4_k(a, k0, 2 * half, lo);
    a.q = r.v[1];
    emit_q4_k(a, k0, 2 * half + 1, hi);
  } else if (FMT == HQ_FMT_FP8_BLOCK) {
    a.aux = r.aux0;
    a.q = r.v[2 * half];
    emit_fp8(a, lo);
    a.q = r.v[2 * half + 1];
    emit_fp8(a, hi);
  } else {
    const uint4 blk = r.v[half];
    a.aux = half == 0 ? r.aux0 : r.aux1;
    a.q.x = blk.x; a.q.y = blk.y;
    ok = emit_mxfp4(a, lo);
    a.q.x = blk.z; a.q.y = blk.w;
    ok = emit_mxfp4(a, hi) && ok;
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    out[i] = lo[i];
    out[8 + i] = hi[i];
  }
  return ok;
}

template <int NB>
__device__ __forceinline__ GgTile ts_tile(const GroupedParams& p, int w, int n_nt) {
  constexpr int FW = NB == 2 ? 64 : 128;     // features per tile
  constexpr int TN = kTsTokens;
  GgTile t;
  const int tt = w / n_nt;
  t.n0 = (w - tt * n_nt) * FW;
  if (p.tiles != nullptr) {
    t.expert = p.tiles[2 * tt];
    t.row_start = p.tiles[2 * tt + 1];
    t.count = min(TN, p.expert_bounds[t.expert + 1] - t.row_start);
  } else {
    t.expert = 0;
    t.row_start = TN * tt;
    t.count = min(TN, p.m - t.row_start);
  }
  return t;
}

template <int FMT, int NB>
__global__ void __launch_bounds__(kGgThreads, 1) grouped_gemm_ts_kernel(const GroupedParams p) {
  using L = TsSmem;
  constexpr int TN = kTsTokens;
  constexpr int NSTAGE = L::NSTAGE;
  constexpr int NBUF = L::NBUF;
  constexpr int FW = NB == 2 ? 64 : 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* empty = full + NSTAGE;
  uint64_t* acc_full = empty + NSTAGE;     // [2]
  uint64_t* acc_empty = acc_full + 2;      // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_nt = (p.n + FW - 1) / FW;
  const int n_tt = p.tiles != nullptr ? p.tile_count[0] : (p.m + TN - 1) / TN;
  const int total = n_tt * n_nt;
  const int n_ks = p.k / kTileK;

  if (tid == 0) {
    for (int s = 0; s < NSTAGE; ++s) {
      mbar_init(&full[s], 4);       // the four warps of the group that owns the stage
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // =========================== MMA issuer ======================================
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(TN);
      uint32_t spin = kGgSpin;
      int it = 0, tcount = 0;
      for (int w = blockIdx.x; w < total; w += gridDim.x, ++tcount) {
        const int buf = tcount % NBUF;
        if (tcount >= NBUF) {
          if (!mbar_wait_backoff(&acc_empty[buf], ((tcount / NBUF) - 1) & 1, spin)) {
            report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 700 + buf);
            spin = 1;
          }
        }
        tc_fence_after();
        const uint32_t d0 = tmem_base + (uint32_t)(buf * TN);
        for (int ks = 0; ks < n_ks; ++ks, ++it) {
          const int s = it % NSTAGE;
          if (!mbar_wait_backoff(&full[s], (it / NSTAGE) & 1, spin)) {
            report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 710 + s);
            spin = 1;
          }
          tc_fence_after();
          const uint64_t bdesc = make_smem_desc(smem_u32(smem + s * L::B_BYTES));
          const uint32_t a0 = tmem_base + (uint32_t)(kTsACol0 + kTsAStageCols * s);
#pragma unroll
          for (int kk = 0; kk < kTileK / 16; ++kk) {
            // 16 k per instruction: 8 columns of A in tensor memory, 32 bytes along the swizzled row of B
            tc_mma_f16_ts(d0, a0 + 8 * kk, bdesc + 2 * kk, idesc, (ks > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(&empty[s]);     // A stage and B stage are free once these MMAs have read them
        }
        tc_commit(&acc_full[buf]);
      }
    }
    __syncwarp();
  } else if (warp <= 4) {
    // =========================== epilogue ========================================
    const int q = warp & 3;
    uint32_t spin = kGgSpin;
    bool failed = false;
    int tcount = 0;
    const bool interleaved = NB == 1 && p.act.act != HQ_ACT_NONE;
    const int bank = NB == 2 ? (lane >> 4) : 0;
    const int frow = NB == 2 ? 16 * q + (lane & 15) : 32 * q + lane;
    for (int w = blockIdx.x; w < total; w += gridDim.x, ++tcount) {
      const GgTile t = ts_tile<NB>(p, w, n_nt);
      const int buf = tcount % NBUF;
      if (!mbar_wait_backoff(&acc_full[buf], (tcount / NBUF) & 1, spin)) {
        if (lane == 0) report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 800 + buf);
        spin = 1;
        failed = true;                 // nothing is stored once a wait has run out
      }
      tc_fence_after();
      const int n = t.n0 + frow;
      const bool n_ok = n < p.n;
      float bias = 0.f;
      const void* bptr = bank == 0 ? p.bias : p.bias_up;
      if (n_ok && bptr != nullptr) bias = load_as_float(bptr, p.bias_dtype, (int64_t)t.expert * p.n + n);
      float sc = 1.f;
      if (FMT == HQ_FMT_FP8_BLOCK) {
        const float* ts = bank == 0 ? p.fp8_tile_scale : p.fp8_tile_scale_up;
        sc = n_ok ? __ldg(ts + (int64_t)t.expert * p.fp8_nb + n / 128) : 0.f;
      }
      const int64_t out_n = interleaved ? (n >> 1) : n;
      const bool writer = n_ok && !failed && (NB == 2 ? lane < 16 : (!interleaved || (n & 1) == 0));
      const uint32_t taddr = tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(buf * TN);
      const int* __restrict__ yrows = p.y_rows;
      auto row_of = [&](int cc) -> int {
        const int col = 32 * cc + lane;
        if (cc >= TN / 32 || col >= t.count) return -1;
        const int sp = t.row_start + col;
        return yrows != nullptr ? __ldg(yrows + sp) : sp;
      };
      const int esz = dtype_size(p.y_dtype);
      char* const ybase = reinterpret_cast<char*>(p.y) + out_n * esz;
      const int64_t ystride_b = (int64_t)p.y_stride * esz;
      int myrow = row_of(0);
#pragma unroll 1
      for (int cc = 0; cc < TN / 32; ++cc) {
        if (32 * cc >= t.count) break;
        uint32_t v0[32];
        tmem_ld32(taddr + 32 * cc, v0);
        const int nextrow = row_of(cc + 1);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float r = fmaf(__uint_as_float(v0[j]), sc, bias);
          if (NB == 2) {
            const float partner = __shfl_xor_sync(0xffffffffu, r, 16);   // the up row of this gate row
            r = gg_gated(r, partner, p.act);
          } else if (interleaved) {
            const float partner = __shfl_xor_sync(0xffffffffu, r, 1);
            r = gg_gated(r, partner, p.act);
          }
          v0[j] = __float_as_uint(r);
        }
        auto store_group = [&](auto cvt) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int orow = __shfl_sync(0xffffffffu, myrow, j);
            if (writer && orow >= 0) {
              using T = decltype(cvt(0.f));
              *reinterpret_cast<T*>(ybase + orow * ystride_b) = cvt(__uint_as_float(v0[j]));
            }
          }
        };
        if (p.y_dtype == HQ_DT_BF16) store_group([](float f) { return __float2bfloat16_rn(f); });
        else if (p.y_dtype == HQ_DT_F16) store_group([](float f) { return __float2half_rn(f); });
        else store_group([](float f) { return f; });
        myrow = nextrow;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  } else {
    // =========================== producers ========================================
    const int grp = (warp - 5) >> 2;              // this group's stages: it = grp (mod 4)
    const int q = warp & 3;                       // tensor-memory lane quarter this warp may write
    const int gt = ((warp - 5) & 3) * 32 + lane;  // thread within the group, for the activation copy
    const int bank = NB == 2 ? (lane >> 4) : 0;
    const int frow = NB == 2 ? 16 * q + (lane & 15) : 32 * q + lane;   // feature within the tile
    const int bchunk = gt & 7, brow0 = gt >> 3;   // activation rows brow0 + 16 j, 16-byte chunk bchunk of each
    constexpr int BR = TN / 16;                   // activation chunks a thread copies per stage
    // byte offset of this thread's first chunk inside a B tile; the others lie 2048 bytes (16 rows) apart
    const uint32_t bswz0 = swz(brow0, bchunk);
    const uint32_t x_stride16 = (uint32_t)(p.x_stride >> 3);   // activation row pitch in 16-byte units
    uint32_t spin = kGgSpin;

    struct Cursor {
      int w, ks, it;
      bool n_ok;
      const uint8_t* wrow;
      const uint8_t* srow;
      const float* rel;
      uint32_t boff[BR];    // 16-byte index of each copied chunk (at k = 0) in the activations, ~0 = no row
    };
    auto open_tile = [&](Cursor& c) {
      const GgTile t = ts_tile<NB>(p, c.w, n_nt);
      const int n = t.n0 + frow;
      c.n_ok = n < p.n;
      const int64_t wrow = (int64_t)t.expert * p.n + (c.n_ok ? n : 0);
      c.wrow = reinterpret_cast<const uint8_t*>(bank == 0 ? p.w : p.w_up) + wrow * p.w_row_bytes;
      c.srow = nullptr;
      c.rel = nullptr;
      if (FMT == HQ_FMT_MXFP4)
        c.srow = reinterpret_cast<const uint8_t*>(bank == 0 ? p.scales : p.scales_up) + wrow * (p.k / 32);
      if (FMT == HQ_FMT_FP8_BLOCK)
        c.rel = (bank == 0 ? p.fp8_rel_scale : p.fp8_rel_scale_up) +
                ((int64_t)t.expert * p.fp8_nb + (c.n_ok ? n : 0) / 128) * p.fp8_kb;
#pragma unroll
      for (int j = 0; j < BR; ++j) {
        const int row = brow0 + 16 * j;
        c.boff[j] = 0xFFFFFFFFu;
        if (row < t.count) {
          const int sp = t.row_start + row;
          c.boff[j] = (uint32_t)(p.x_rows ? p.x_rows[sp] : sp) * x_stride16 + (uint32_t)bchunk;
        }
      }
    };
    // four stages on: returns false past the CTA's last tile
    auto advance = [&](Cursor& c) -> bool {
      c.it += 4;
      c.ks += 4;
      bool moved = false;
      while (c.ks >= n_ks && c.w < total) {
        c.ks -= n_ks;
        c.w += gridDim.x;
        moved = true;
      }
      if (c.w >= total) return false;
      if (moved) open_tile(c);
      return true;
    };
    int waited = NSTAGE - 1;                  // stages up to this index are known to be free
    auto ensure_empty = [&](int j) {
      if (j > waited) {
        if (!mbar_wait(&empty[j % NSTAGE], ((j / NSTAGE) - 1) & 1, spin)) {
          if (lane == 0) report_status(p.status, HQ_DEV_WAIT_TIMEOUT, 900 + j % NSTAGE);
          spin = 1;
        }
        waited = j;
      }
    };
    auto copy_b = [&](const Cursor& c) {
      const uint32_t dst0 = smem_u32(smem + (c.it % NSTAGE) * L::B_BYTES) + bswz0;
      const uint32_t kofs = (uint32_t)c.ks * (kTileK / 8);
      const uint4* x16 = reinterpret_cast<const uint4*>(p.x);
#pragma unroll
      for (int j = 0; j < BR; ++j) {
        const bool ok = c.boff[j] != 0xFFFFFFFFu;
        const uint4* src = x16 + (ok ? c.boff[j] + kofs : 0u);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst0 + 2048u * j), "l"(src), "r"(ok ? 16 : 0)
                     : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    auto fetch = [&](const Cursor& c, TsRaw& r) {
      if (c.n_ok) ts_fetch<FMT>(r, c.wrow, c.srow, c.rel, c.ks * kTileK);
    };

    Cursor cur;
    cur.w = blockIdx.x;
    cur.ks = grp - 4;
    cur.it = grp - 4;
    bool live = false;
    if (cur.w < total) {
      // the first stage of this group: ks = grp may already lie in a later tile when K is very short
      cur.ks = grp;
      cur.it = grp;
      while (cur.ks >= n_ks && cur.w < total) {
        cur.ks -= n_ks;
        cur.w += gridDim.x;
      }
      live = cur.w < total;
      if (live) open_tile(cur);
    }
    TsRaw ra0, ra1;
    if (live) {
      fetch(cur, ra0);
      copy_b(cur);
    }
    // One stage: the next own stage's weight loads go out first; this stage is expanded into its tensor-memory
    // slot (known to be free since its activation copies were issued) and handed over; only then does the group
    // wait for the slot of its next stage and start that stage's activation copies -- by then the MMA has had a
    // whole step to drain the slot, and the copies have the next expansion to land.
    auto step = [&](TsRaw& use, TsRaw& ld) {
      Cursor nxt = cur;
      const bool next_live = advance(nxt);
      if (next_live) fetch(nxt, ld);
      const int s = cur.it % NSTAGE;
      const uint32_t taddr = tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(kTsACol0 + kTsAStageCols * s);
      const int k0 = cur.ks * kTileK;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t v[16];
        if (cur.n_ok) {
          if (!ts_expand<FMT>(use, k0, half, v)) report_status(p.status, HQ_DEV_SCALE_RANGE, 600);
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = 0u;
        }
        tmem_st16(taddr + 16 * half, v);
      }
      tmem_st_wait();
      asm volatile("cp.async.wait_group 0;" ::: "memory");   // this stage's activation copies, issued a step ago
      fence_proxy_async_smem();     // cp.async writes -> visible to the tensor core (async proxy)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&full[s]);
      if (next_live) {
        ensure_empty(nxt.it);
        copy_b(nxt);
      }
      cur = nxt;
      live = next_live;
    };
    while (live) {
      step(ra0, ra1);
      if (!live) break;
      step(ra1, ra0);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---- block-FP8 scale preparation (once per layer) -------------------------------------
// scales [groups = E*NB][KB] -> tile_scale[group] = max_kb scale, rel_scale[group][kb] = scale / tile_scale.
__global__ void __launch_bounds__(128) fp8_scale_prepare_kernel(const float* __restrict__ scales, int64_t n_groups,
                                                                int kb, float* __restrict__ tile_scale,
                                                                float* __restrict__ rel_scale) {
  const int64_t grp = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (grp >= n_groups) return;
  const int lane = threadIdx.x & 31;
  float m = 0.f;
  for (int i = lane; i < kb; i += 32) m = fmaxf(m, scales[grp * kb + i]);
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
  if (lane == 0) tile_scale[grp] = m;
  for (int i = lane; i < kb; i += 32) rel_scale[grp * kb + i] = m > 0.f ? scales[grp * kb + i] / m : 0.f;
}

int32_t launch_fp8_scale_prepare(const float* scales, int64_t n_groups, int kb, float* tile_scale, float* rel_scale,
                                 cudaStream_t stream) {
  if (n_groups == 0) return HQ_OK;
  fp8_scale_prepare_kernel<<<(unsigned)((n_groups + 3) / 4), 128, 0, stream>>>(scales, n_groups, kb, tile_scale,
                                                                             rel_scale);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

// ---- host launcher -----------------------------------------------------------------
template <int FMT, int NB, int TN>
static int32_t launch_gg(const GroupedParams& p, int max_tiles, cudaStream_t stream) {
  using L = GgSmem<NB, TN>;
  static_assert(L::TOTAL <= 227 * 1024, "shared memory budget");
  static_assert(L::NSTAGE >= 3, "pipeline depth");
  auto kern = grouped_gemm_kernel<FMT, NB, TN>;
  static bool attr_done[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return HQ_ERR_CUDA;
  if (dev < 64 && !attr_done[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess)
      return HQ_ERR_CUDA;
    attr_done[dev] = true;
  }
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  const int64_t items = (int64_t)max_tiles * ((p.n + kTileM - 1) / kTileM);
  const int64_t grid = items < sms ? items : sms;
  if (grid <= 0) return HQ_OK;
  kern<<<(unsigned)grid, kGgThreads, L::TOTAL, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

template <int FMT, int NB>
static int32_t launch_gg_ts(const GroupedParams& p, int max_tiles, cudaStream_t stream) {
  using L = TsSmem;
  constexpr int TN = kTsTokens;
  static_assert(L::TOTAL <= 227 * 1024, "shared memory budget");
  static_assert(kTsACol0 + kTsAStageCols * L::NSTAGE <= 512 && L::NBUF * TN <= kTsACol0, "tensor memory budget");
  auto kern = grouped_gemm_ts_kernel<FMT, NB>;
  static bool attr_done[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return HQ_ERR_CUDA;
  if (dev < 64 && !attr_done[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess)
      return HQ_ERR_CUDA;
    attr_done[dev] = true;
  }
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  constexpr int FW = NB == 2 ? 64 : 128;
  const int64_t items = (int64_t)max_tiles * ((p.n + FW - 1) / FW);
  const int64_t grid = items < sms ? items : sms;
  if (grid <= 0) return HQ_OK;
  kern<<<(unsigned)grid, kGgThreads, L::TOTAL, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? HQ_OK : HQ_ERR_CUDA;
}

template <int FMT>
static int32_t launch_gg_fmt(const GroupedParams& p, int max_tiles, cudaStream_t stream) {
  const bool two = p.w_up != nullptr;
  // only Q4_K, block-FP8 and MXFP4 have the variant that keeps the expanded weights in tensor memory
  if constexpr (FMT == HQ_FMT_Q4_K || FMT == HQ_FMT_FP8_BLOCK || FMT == HQ_FMT_MXFP4) {
    if (p.tile_rows == 128 && p.weights_in_tmem)
      return two ? launch_gg_ts<FMT, 2>(p, max_tiles, stream) : launch_gg_ts<FMT, 1>(p, max_tiles, stream);
  }
  if (p.tile_rows == 256) {
    return two ? launch_gg<FMT, 2, 256>(p, max_tiles, stream) : launch_gg<FMT, 1, 256>(p, max_tiles, stream);
  }
  return two ? launch_gg<FMT, 2, 128>(p, max_tiles, stream) : launch_gg<FMT, 1, 128>(p, max_tiles, stream);
}

bool grouped_gemm_supported(int format, int64_t n, int64_t k) {
  if (format != HQ_FMT_Q4_K && format != HQ_FMT_FP8_BLOCK && format != HQ_FMT_MXFP4 && format != HQ_FMT_Q8_0 &&
      format != HQ_FMT_Q6_K && format != HQ_FMT_Q5_K && format != HQ_FMT_Q4_0 && format != HQ_FMT_Q5_0 &&
      format != HQ_FMT_Q4_1 && format != HQ_FMT_Q5_1 && format != HQ_FMT_Q2_K && format != HQ_FMT_Q3_K)
    return false;
  if (k % kTileK != 0) return false;
  if (format == HQ_FMT_FP8_BLOCK && (n % 128 != 0 || k % 128 != 0)) return false;
  return true;
}

int32_t launch_grouped_gemm(const GroupedParams& p, int max_tiles, cudaStream_t stream) {
  if (p.tile_rows != 128 && p.tile_rows != 256) return HQ_ERR_SHAPE;
  if (p.x_dtype != HQ_DT_F16) return HQ_ERR_FORMAT;   // activations are copied into the operand tiles as f16
  switch (p.format) {
    case HQ_FMT_Q4_K: return launch_gg_fmt<HQ_FMT_Q4_K>(p, max_tiles, stream);
    case HQ_FMT_FP8_BLOCK: return launch_gg_fmt<HQ_FMT_FP8_BLOCK>(p, max_tiles, stream);
    case HQ_FMT_MXFP4: return launch_gg_fmt<HQ_FMT_MXFP4>(p, max_tiles, stream);
    case HQ_FMT_Q8_0:
      if ((reinterpret_cast<uintptr_t>(p.w) & 3u) != 0 || (p.w_up != nullptr && (reinterpret_cast<uintptr_t>(p.w_up) & 3u) != 0))
        return HQ_ERR_ALIGN;
      return launch_gg_fmt<HQ_FMT_Q8_0>(p, max_tiles, stream);
    case HQ_FMT_Q6_K:
    case HQ_FMT_Q2_K:
    case HQ_FMT_Q3_K:
      if ((reinterpret_cast<uintptr_t>(p.w) & 3u) != 0 || (p.w_up != nullptr && (reinterpret_cast<uintptr_t>(p.w_up) & 3u) != 0))
        return HQ_ERR_ALIGN;
      if (p.format == HQ_FMT_Q2_K) return launch_gg_fmt<HQ_FMT_Q2_K>(p, max_tiles, stream);
      if (p.format == HQ_FMT_Q3_K) return launch_gg_fmt<HQ_FMT_Q3_K>(p, max_tiles, stream);
      return launch_gg_fmt<HQ_FMT_Q6_K>(p, max_tiles, stream);
    case HQ_FMT_Q5_K:
    case HQ_FMT_Q4_0:
    case HQ_FMT_Q5_0:
    case HQ_FMT_Q4_1:
    case HQ_FMT_Q5_1:
      // rows are multiples of 16 bytes; the producers read 16-byte pieces (Q5_K) or aligned words (Q4_0 / Q5_0)
      if ((reinterpret_cast<uintptr_t>(p.w) & 15u) != 0 || (p.w_up != nullptr && (reinterpret_cast<uintptr_t>(p.w_up) & 15u) != 0))
        return HQ_ERR_ALIGN;
      if (p.format == HQ_FMT_Q5_K) return launch_gg_fmt<HQ_FMT_Q5_K>(p, max_tiles, stream);
      if (p.format == HQ_FMT_Q4_0) return launch_gg_fmt<HQ_FMT_Q4_0>(p, max_tiles, stream);
      if (p.format == HQ_FMT_Q4_1) return launch_gg_fmt<HQ_FMT_Q4_1>(p, max_tiles, stream);
      if (p.format == HQ_FMT_Q5_1) return launch_gg_fmt<HQ_FMT_Q5_1>(p, max_tiles, stream);
      return launch_gg_fmt<HQ_FMT_Q5_0>(p, max_tiles, stream);
    default: return HQ_ERR_FORMAT;
  }
}

}  // namespace hq
