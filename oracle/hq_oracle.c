/*
 * CPU oracle in C: TEST INFRASTRUCTURE ONLY.  A plain restatement of the
 * reference's CPU arithmetic for the quantized-linear / MoE path (per-block
 * dequantize to f32, f32 dot products), used as the checker at sizes numpy is
 * too slow for and as the timed CPU baseline ("port") of the benchmark.  The
 * library never links or loads this file.
 *
 * Follows: Q8_0 / Q4_K block structs and value formulas
 * (hanzo-quant/kernels/mmvq_gguf/mmvq_gguf.cu:134-137, :166-170, :385-404,
 * :595-606); the other GGML types of the reference's decode list
 * (hanzo-quant/src/gguf/fast_mmvq.rs:36-50) as ggml's dequantize_row_*
 * functions define them; block-FP8 dequant (hanzo-quant/src/blockwise_fp8/ops.rs:11-59);
 * MXFP4 LUT dequant and the blocked dot of forward_dequantize /
 * gather_forward_dequantize (hanzo-quant/src/mxfp4/mod.rs:473-489, :550-726);
 * per-expert grouping of the slow experts backend
 * (hanzo-engine/src/moe/experts/backends.rs:900-959).
 * Parity of this file is pinned by tests/test_oracle_c.py against the numpy
 * oracle (itself pinned against gguf-py and the reference's golden vectors).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum { FMT_Q8_0 = 0, FMT_Q4_K = 1, FMT_FP8 = 2, FMT_MXFP4 = 3, FMT_Q6_K = 4, FMT_Q5_K = 5, FMT_Q4_0 = 6, FMT_Q5_0 = 7,
       FMT_Q4_1 = 8, FMT_Q5_1 = 9, FMT_Q2_K = 10, FMT_Q3_K = 11 };

static float half_to_float(uint16_t h) {
  uint32_t s = (uint32_t)(h >> 15) << 31, e = (h >> 10) & 31, m = h & 1023, b;
  if (e == 0) {
    if (m == 0) { b = s; }
    else { int sh = 0; while (!(m & 1024)) { m <<= 1; ++sh; } b = s | ((uint32_t)(113 - sh) << 23) | ((m & 1023) << 13); }
  } else if (e == 31) b = s | 0x7F800000u | (m << 13);
  else b = s | ((e + 112) << 23) | (m << 13);
  float f; memcpy(&f, &b, 4); return f;
}

static float e4m3_decode(uint8_t c) {
  int e = (c >> 3) & 15, m = c & 7;
  float v;
  if (e == 15 && m == 7) v = NAN;
  else if (e == 0) v = ldexpf((float)m / 8.0f, -6);
  else v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
  return (c & 0x80) ? -v : v;
}
/* the 256 values of the format, decoded once (every entry point fills it before its parallel region) */
static float E4M3[256];
static int e4m3_ready = 0;
static void e4m3_init(void) {
  if (!e4m3_ready) {
    for (int c = 0; c < 256; ++c) E4M3[c] = e4m3_decode((uint8_t)c);
    e4m3_ready = 1;
  }
}
static inline float e4m3_to_float(uint8_t c) { return E4M3[c]; }

static const float FP4[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                              -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

int64_t oracle_row_bytes(int fmt, int64_t k) {
  switch (fmt) {
    case FMT_Q8_0: return k / 32 * 34;
    case FMT_Q4_K: return k / 256 * 144;
    case FMT_FP8: return k;
    case FMT_Q6_K: return k / 256 * 210;
    case FMT_Q5_K: return k / 256 * 176;
    case FMT_Q4_0: return k / 32 * 18;
    case FMT_Q5_0: return k / 32 * 22;
    case FMT_Q4_1: return k / 32 * 20;
    case FMT_Q5_1: return k / 32 * 24;
    case FMT_Q2_K: return k / 256 * 84;
    case FMT_Q3_K: return k / 256 * 110;
    default: return k / 2;
  }
}

static float half_at(const uint8_t* p) {
  uint16_t h; memcpy(&h, p, 2);
  return half_to_float(h);
}

/* scale and min j (0..7) of the 12 packed bytes of a Q4_K / Q5_K super-block */
static void k4_scale_min(const uint8_t* sc, int j, int* s, int* m) {
  if (j < 4) { *s = sc[j] & 63; *m = sc[j + 4] & 63; }
  else { *s = (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4); *m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
}

/* The further GGML types: one row, element order and arithmetic of ggml's dequantize_row_*. */
static void dequant_row_ggml(int fmt, const uint8_t* row, int64_t k, float* out) {
  if (fmt == FMT_Q4_0 || fmt == FMT_Q5_0 || fmt == FMT_Q4_1 || fmt == FMT_Q5_1) {
    const int five = fmt == FMT_Q5_0 || fmt == FMT_Q5_1, has_min = fmt == FMT_Q4_1 || fmt == FMT_Q5_1;
    const int bb = 18 + 4 * five + 2 * has_min;
    for (int64_t b = 0; b < k / 32; ++b) {
      const uint8_t* p = row + bb * b;
      const float d = half_at(p), m = has_min ? half_at(p + 2) : 0.0f;
      uint32_t qh = 0;
      if (five) memcpy(&qh, p + (has_min ? 4 : 2), 4);
      const uint8_t* qs = p + bb - 16;
      const int zero = has_min ? 0 : (five ? 16 : 8);
      for (int j = 0; j < 16; ++j) {
        const int x0 = (qs[j] & 0xF) | (int)(((qh >> j) & 1u) << 4);
        const int x1 = (qs[j] >> 4) | (int)(((qh >> (j + 16)) & 1u) << 4);
        if (has_min) {
          out[32 * b + j] = d * (float)x0 + m;
          out[32 * b + j + 16] = d * (float)x1 + m;
        } else {
          out[32 * b + j] = d * (float)(x0 - zero);
          out[32 * b + j + 16] = d * (float)(x1 - zero);
        }
      }
    }
  } else if (fmt == FMT_Q5_K) {
    for (int64_t sb = 0; sb < k / 256; ++sb) {
      const uint8_t* p = row + 176 * sb;
      const float d = half_at(p), dmin = half_at(p + 2);
      const uint8_t* qh = p + 16;
      for (int j = 0; j < 8; ++j) {
        int s, m;
        k4_scale_min(p + 4, j, &s, &m);
        const float d1 = d * (float)s, m1 = dmin * (float)m;
        const uint8_t* q = p + 48 + 32 * (j / 2);
        float* o = out + 256 * sb + 32 * j;
        for (int l = 0; l < 32; ++l) {
          const int nib = (j & 1) ? (q[l] >> 4) : (q[l] & 0xF);
          o[l] = d1 * (float)(nib | (((qh[l] >> j) & 1) << 4)) - m1;
        }
      }
    }
  } else if (fmt == FMT_Q6_K) {
    for (int64_t sb = 0; sb < k / 256; ++sb) {
      const uint8_t* p = row + 210 * sb;
      const int8_t* sc = (const int8_t*)(p + 192);
      const float d = half_at(p + 208);
      for (int h = 0; h < 2; ++h) {
        const uint8_t* ql = p + 64 * h;
        const uint8_t* qh = p + 128 + 32 * h;
        float* o = out + 256 * sb + 128 * h;
        for (int l = 0; l < 32; ++l) {
          const int is = 8 * h + l / 16;
          const int q1 = (int)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
          const int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
          const int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
          const int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
          o[l] = d * (float)sc[is] * (float)q1;
          o[l + 32] = d * (float)sc[is + 2] * (float)q2;
          o[l + 64] = d * (float)sc[is + 4] * (float)q3;
          o[l + 96] = d * (float)sc[is + 6] * (float)q4;
        }
      }
    }
  } else if (fmt == FMT_Q2_K) {
    for (int64_t sb = 0; sb < k / 256; ++sb) {
      const uint8_t* p = row + 84 * sb;
      const float d = half_at(p + 80), dmin = half_at(p + 82);
      for (int h = 0; h < 2; ++h)
        for (int j = 0; j < 4; ++j)
          for (int l = 0; l < 32; ++l) {
            const uint8_t s = p[8 * h + 2 * j + l / 16];
            const float dl = d * (float)(s & 0xF), ml = dmin * (float)(s >> 4);
            out[256 * sb + 128 * h + 32 * j + l] = dl * (float)((p[16 + 32 * h + l] >> (2 * j)) & 3) - ml;
          }
    }
  } else {   /* FMT_Q3_K */
    for (int64_t sb = 0; sb < k / 256; ++sb) {
      const uint8_t* p = row + 110 * sb;
      const uint8_t* raw = p + 96;
      const float d = half_at(p + 108);
      int scale[16];
      for (int is = 0; is < 16; ++is) {
        const int a = is / 4, b = is % 4;
        const int lo = a < 2 ? (raw[4 * a + b] & 0xF) : (raw[4 * (a - 2) + b] >> 4);
        scale[is] = (lo | (((raw[8 + b] >> (2 * a)) & 3) << 4)) - 32;
      }
      for (int h = 0; h < 2; ++h)
        for (int j = 0; j < 4; ++j)
          for (int l = 0; l < 32; ++l) {
            const float dl = d * (float)scale[8 * h + 2 * j + l / 16];
            const int q = (int)((p[32 + 32 * h + l] >> (2 * j)) & 3) - (((p[l] >> (4 * h + j)) & 1) ? 0 : 4);
            out[256 * sb + 128 * h + 32 * j + l] = dl * (float)q;
          }
    }
  }
}

/* Dequantize one weight row to f32.  scales: FP8 -> f32 row of the scale grid for this row's 128-block,
 * MXFP4 -> the row's e8m0 bytes. */
static void dequant_row(int fmt, const uint8_t* row, const void* scales, int64_t k, float* out) {
  if (fmt == FMT_Q8_0) {
    for (int64_t b = 0; b < k / 32; ++b) {
      const uint8_t* p = row + 34 * b;
      uint16_t dh; memcpy(&dh, p, 2);
      const float d = half_to_float(dh);
      const int8_t* q = (const int8_t*)(p + 2);
      for (int i = 0; i < 32; ++i) out[32 * b + i] = d * (float)q[i];
    }
  } else if (fmt == FMT_Q4_K) {
    for (int64_t sb = 0; sb < k / 256; ++sb) {
      const uint8_t* p = row + 144 * sb;
      uint16_t dh, mh; memcpy(&dh, p, 2); memcpy(&mh, p + 2, 2);
      const float d = half_to_float(dh), dmin = half_to_float(mh);
      const uint8_t* sc = p + 4;
      const uint8_t* qs = p + 16;
      for (int j = 0; j < 8; ++j) {
        int s, m;
        if (j < 4) { s = sc[j] & 63; m = sc[j + 4] & 63; }
        else { s = (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4); m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
        const float d1 = d * (float)s, m1 = dmin * (float)m;
        const uint8_t* q = qs + 32 * (j / 2);
        float* o = out + 256 * sb + 32 * j;
        if (j & 1) for (int i = 0; i < 32; ++i) o[i] = d1 * (float)(q[i] >> 4) - m1;
        else for (int i = 0; i < 32; ++i) o[i] = d1 * (float)(q[i] & 0xF) - m1;
      }
    }
  } else if (fmt == FMT_FP8) {
    const float* s = (const float*)scales;
    for (int64_t i = 0; i < k; ++i) out[i] = e4m3_to_float(row[i]) * s[i / 128];
  } else if (fmt >= FMT_Q6_K) {
    dequant_row_ggml(fmt, row, k, out);
  } else {
    const uint8_t* s = (const uint8_t*)scales;
    for (int64_t b = 0; b < k / 32; ++b) {
      uint32_t bits = (uint32_t)s[b] << 23;
      float sf; memcpy(&sf, &bits, 4);
      for (int i = 0; i < 16; ++i) {
        const uint8_t byte = row[16 * b + i];
        out[32 * b + 2 * i] = FP4[byte & 0xF] * sf;
        out[32 * b + 2 * i + 1] = FP4[byte >> 4] * sf;
      }
    }
  }
}

static const void* row_scales(int fmt, const void* scales, int64_t n_row, int64_t k) {
  if (fmt == FMT_FP8) return (const float*)scales + (n_row / 128) * ((k + 127) / 128);
  if (fmt == FMT_MXFP4) return (const uint8_t*)scales + n_row * (k / 32);
  return NULL;
}

/* y[m, n] = sum_k x[m, k] * dequant(W)[n, k] (+ bias[n]); f32 accumulation per row. */
void oracle_linear(int fmt, const uint8_t* w, const void* scales, const float* bias, const float* x, float* y,
                   int64_t n, int64_t k, int64_t m, int threads) {
  const int64_t rb = oracle_row_bytes(fmt, k);
  e4m3_init();
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#endif
#pragma omp parallel
  {
    float* wrow = (float*)malloc(sizeof(float) * (size_t)k);
#pragma omp for schedule(static)
    for (int64_t r = 0; r < n; ++r) {
      dequant_row(fmt, w + r * rb, row_scales(fmt, scales, r, k), k, wrow);
      for (int64_t j = 0; j < m; ++j) {
        const float* xr = x + j * k;
        float acc = 0.f;
        for (int64_t i = 0; i < k; ++i) acc += xr[i] * wrow[i];
        y[j * n + r] = acc + (bias ? bias[r] : 0.f);
      }
    }
    free(wrow);
  }
}

/* Per-assignment projection out of an expert bank, grouped by expert in stable (token, slot) order:
 * out[rows[i], :] for every sorted position i of expert e uses x[xrows[i], :]. */
void oracle_gather(int fmt, const uint8_t* w, const void* scales, const float* bias, const float* x, float* out,
                   int64_t n, int64_t k, int n_experts, const int32_t* bounds, const int32_t* xrows,
                   const int32_t* orows, int threads) {
  const int64_t rb = oracle_row_bytes(fmt, k);
  e4m3_init();
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#endif
#pragma omp parallel
  {
    float* wrow = (float*)malloc(sizeof(float) * (size_t)k);
#pragma omp for schedule(dynamic, 16) collapse(2)
    for (int e = 0; e < n_experts; ++e) {
      for (int64_t r = 0; r < n; ++r) {
        const int lo = bounds[e], hi = bounds[e + 1];
        if (lo == hi) continue;
        const int64_t gr = (int64_t)e * n + r;
        const void* sc = NULL;
        if (fmt == FMT_FP8) sc = (const float*)scales + ((int64_t)e * ((n + 127) / 128) + r / 128) * ((k + 127) / 128);
        else if (fmt == FMT_MXFP4) sc = (const uint8_t*)scales + gr * (k / 32);
        dequant_row(fmt, w + gr * rb, sc, k, wrow);
        for (int i = lo; i < hi; ++i) {
          const float* xr = x + (int64_t)xrows[i] * k;
          float acc = 0.f;
          for (int64_t c = 0; c < k; ++c) acc += xr[c] * wrow[c];
          out[(int64_t)orows[i] * n + r] = acc + (bias ? bias[gr] : 0.f);
        }
      }
    }
    free(wrow);
  }
}

int oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
