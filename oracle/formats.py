"""CPU oracle: weight/activation formats of the quantized-linear hot path.

TEST INFRASTRUCTURE ONLY.  Nothing the library ships imports this module; it is
the checker for the CUDA kernels (tests, the smoke run, the CPU leg of the
benchmark).  Every function restates, in numpy, the arithmetic of one piece of
the reference (hanzo-quant) and cites the file:line it follows.

Pinned against (see tests/test_oracle_*.py and tests/golden/):
  * gguf-py `dequantize` for Q8_0 and Q4_K bytes (bit-exact),
  * the reference's own Python Q4_K quantizer (scripts/convert_fp8_to_gguf.py)
    through committed golden bytes,
  * the reference's known-answer tests for FP8 block / vector dequant and the
    MXFP4 value table.
Parity unpinned (no reference vector exists, third-party crate arithmetic):
  e4m3 rounding at exact ties (crate `float8` 0.7.0) -- round-to-nearest-even
  is assumed, as in `ml_dtypes.float8_e4m3fn`.
"""
from __future__ import annotations

import numpy as np

QK8_0 = 32          # elements per Q8_0 block
Q8_0_BYTES = 34     # half d + 32 int8
QK_K = 256          # elements per k-quant super-block
Q4_K_BYTES = 144    # half d, half dmin, 12 scale bytes, 128 nibble bytes
Q6_K_BYTES = 210    # 128 low-nibble bytes, 64 high-bit bytes, 16 int8 scales, half d
Q5_K_BYTES = 176    # half d, half dmin, 12 scale bytes, 32 high-bit bytes, 128 nibble bytes
Q4_0_BYTES = 18     # half d, 16 nibble bytes (32 weights)
Q5_0_BYTES = 22     # half d, 4 high-bit bytes, 16 nibble bytes (32 weights)
Q4_1_BYTES = 20     # half d, half m, 16 nibble bytes (32 weights)
Q5_1_BYTES = 24     # half d, half m, 4 high-bit bytes, 16 nibble bytes (32 weights)
Q2_K_BYTES = 84     # 16 scale|min bytes, 64 bytes of 2-bit codes, half d, half dmin
Q3_K_BYTES = 110    # 32 high-bit bytes, 64 bytes of 2-bit codes, 12 bytes of 6-bit scales, half d
MXFP4_BLOCK = 32
FP8_MAX = 448.0

# ----------------------------------------------------------------------------
# Q8_0  (block_q8_0 {half d; int8 qs[32]}: hanzo-quant/kernels/mmvq_gguf/mmvq_gguf.cu:134-137)
# ----------------------------------------------------------------------------


def q8_0_quantize(w: np.ndarray) -> np.ndarray:
    """f32 [rows, K] -> uint8 [rows, K/32*34].  d = absmax/127 (fp16), q = round(x/d).

    Any valid block bytes are acceptable test data: parity is defined against
    the dequantization of the same bytes.  Matches gguf-py's Q8_0 quantizer.
    """
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, k = w.shape
    assert k % QK8_0 == 0
    blk = w.reshape(rows, k // QK8_0, QK8_0)
    amax = np.abs(blk).max(axis=2, keepdims=True)
    d = amax / np.float32(127.0)
    with np.errstate(divide="ignore", invalid="ignore"):
        inv = np.where(d > 0, np.float32(1.0) / d, np.float32(0.0)).astype(np.float32)
    q = np.rint(blk * inv).astype(np.int8)
    out = np.empty((rows, k // QK8_0, Q8_0_BYTES), np.uint8)
    out[:, :, 0:2] = d.astype(np.float16).view(np.uint8).reshape(rows, -1, 2)
    out[:, :, 2:] = q.view(np.uint8)
    return out.reshape(rows, -1)


def q8_0_dequant(raw: np.ndarray, k: int) -> np.ndarray:
    """uint8 [rows, K/32*34] -> f32 [rows, K]; value = d * q (mmvq_gguf.cu:134-137)."""
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    rows = raw.shape[0]
    blk = raw.reshape(rows, k // QK8_0, Q8_0_BYTES)
    d = blk[:, :, 0:2].copy().view(np.float16).astype(np.float32)          # [rows, nb, 1]
    q = blk[:, :, 2:].copy().view(np.int8).astype(np.float32)
    return (d * q).reshape(rows, k)


# ----------------------------------------------------------------------------
# Q4_K  (block_q4_K {half2 dm; uint8 scales[12]; uint8 qs[128]}: mmvq_gguf.cu:166-170;
#        6-bit scale/min unpack :595-606; value = d*sc*q - dmin*m :385-404;
#        element order inside a super-block: scripts/convert_fp8_to_gguf.py:191-211)
# ----------------------------------------------------------------------------


def q4_k_unpack_scales(sc_bytes: np.ndarray):
    """uint8 [..., 12] -> (sc [..., 8], m [..., 8]) 6-bit integers (mmvq_gguf.cu:595-606)."""
    b = sc_bytes.astype(np.uint8)
    sc = np.empty(b.shape[:-1] + (8,), np.uint8)
    mn = np.empty_like(sc)
    for j in range(4):
        sc[..., j] = b[..., j] & 63
        mn[..., j] = b[..., j + 4] & 63
    for j in range(4, 8):
        sc[..., j] = (b[..., j + 4] & 0x0F) | ((b[..., j - 4] >> 6) << 4)
        mn[..., j] = (b[..., j + 4] >> 4) | ((b[..., j] >> 6) << 4)
    return sc, mn


def q4_k_dequant(raw: np.ndarray, k: int) -> np.ndarray:
    """uint8 [rows, K/256*144] -> f32 [rows, K].

    Sub-block j=2c takes the LOW nibbles of qs[32c..32c+31], sub-block 2c+1 the
    HIGH nibbles of the same bytes; value = (d*sc_j)*q - (dmin*m_j).
    """
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    rows = raw.shape[0]
    nsb = k // QK_K
    blk = raw.reshape(rows, nsb, Q4_K_BYTES)
    d = blk[:, :, 0:2].copy().view(np.float16).astype(np.float32)          # [rows, nsb, 1]
    dmin = blk[:, :, 2:4].copy().view(np.float16).astype(np.float32)
    sc, mn = q4_k_unpack_scales(blk[:, :, 4:16])
    qs = blk[:, :, 16:].reshape(rows, nsb, 4, 32)
    q = np.empty((rows, nsb, 8, 32), np.float32)
    q[:, :, 0::2, :] = (qs & 0x0F).astype(np.float32)
    q[:, :, 1::2, :] = (qs >> 4).astype(np.float32)
    d1 = (d * sc.astype(np.float32))[..., None]                            # [rows, nsb, 8, 1]
    m1 = (dmin * mn.astype(np.float32))[..., None]
    return (d1 * q - m1).reshape(rows, k)


# ----------------------------------------------------------------------------
# Q6_K  (block_q6_K {uint8 ql[128]; uint8 qh[64]; int8 scales[16]; half d}; 16 sub-blocks of 16 elements,
#        value = d * scale * (q - 32), q = 4 low bits from ql + 2 high bits from qh.  The type carries
#        attn_v / ffn_down in Q4_K_M files; it is in the reference's decode list,
#        hanzo-quant/src/gguf/fast_mmvq.rs:36-50.  Element order per 128-element half: for l in 0..31 the bytes
#        ql[l], ql[l+32], qh[l] give elements l, l+32, l+64, l+96 -- ggml's dequantize_row_q6_K.)
# ----------------------------------------------------------------------------

def q6_k_dequant(raw: np.ndarray, k: int) -> np.ndarray:
    """uint8 [rows, K/256*210] -> f32 [rows, K]."""
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    rows = raw.shape[0]
    nsb = k // QK_K
    blk = raw.reshape(rows, nsb, Q6_K_BYTES)
    ql = blk[:, :, 0:128].reshape(rows, nsb, 2, 2, 32)        # [half][first/second 32 bytes][l]
    qh = blk[:, :, 128:192].reshape(rows, nsb, 2, 32)         # [half][l]
    sc = blk[:, :, 192:208].copy().view(np.int8).astype(np.float32).reshape(rows, nsb, 2, 8)
    d = blk[:, :, 208:210].copy().view(np.float16).astype(np.float32)          # [rows, nsb, 1]
    q = np.empty((rows, nsb, 2, 4, 32), np.int32)             # [half][j][l] -> element 128 half + 32 j + l
    for j in range(4):
        nib = (ql[:, :, :, j & 1, :] & 0x0F) if j < 2 else (ql[:, :, :, j & 1, :] >> 4)
        q[:, :, :, j, :] = (nib.astype(np.int32) | (((qh >> (2 * j)) & 3).astype(np.int32) << 4)) - 32
    # scale index inside a half: 2 j + l // 16
    s = sc.reshape(rows, nsb, 2, 4, 2)
    s = np.repeat(s, 16, axis=-1)                              # [half][j][l]
    out = d[:, :, :, None, None] * s * q.astype(np.float32)
    return out.reshape(rows, k).astype(np.float32)


def q6_k_quantize(w: np.ndarray) -> np.ndarray:
    """f32 [rows, K] -> uint8 [rows, K/256*210].  A plain quantizer for building test and benchmark weights (ggml's
    own make_qx_quants search is not restated; any valid block exercises the kernels): per 16-element sub-block
    scale = absmax / 31 signed by the element of largest magnitude, d = max|scale| / 127, integer scales and
    6-bit codes by round-to-nearest."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, k = w.shape
    nsb = k // QK_K
    x = w.reshape(rows, nsb, 16, 16)
    amax = np.abs(x).max(-1)
    scale = amax / np.float32(31.0)
    dmax = scale.max(-1, keepdims=True)
    d = (dmax / np.float32(127.0)).astype(np.float16)
    df = d.astype(np.float32)
    isc = np.where(df > 0, np.rint(scale / np.where(df > 0, df, 1)), 0).clip(-128, 127).astype(np.int8)
    step = df * isc.astype(np.float32)
    q = np.where(step[..., None] != 0, np.rint(x / np.where(step[..., None] != 0, step[..., None], 1)), 0)
    q = (q.clip(-32, 31) + 32).astype(np.uint8).reshape(rows, nsb, 2, 4, 32)   # [half][j][l]
    blk = np.zeros((rows, nsb, Q6_K_BYTES), np.uint8)
    ql = np.zeros((rows, nsb, 2, 2, 32), np.uint8)
    qh = np.zeros((rows, nsb, 2, 32), np.uint8)
    for j in range(4):
        nib = q[:, :, :, j, :] & 0x0F
        ql[:, :, :, j & 1, :] |= nib if j < 2 else (nib << 4)
        qh |= ((q[:, :, :, j, :] >> 4) & 3) << (2 * j)
    blk[:, :, 0:128] = ql.reshape(rows, nsb, 128)
    blk[:, :, 128:192] = qh.reshape(rows, nsb, 64)
    blk[:, :, 192:208] = isc.reshape(rows, nsb, 16).view(np.uint8)
    blk[:, :, 208:210] = d.reshape(rows, nsb, 1).view(np.uint8)
    return blk.reshape(rows, nsb * Q6_K_BYTES)


# ----------------------------------------------------------------------------
# Q5_K, Q4_0, Q5_0 (the further types of the reference's decode list, hanzo-quant/src/gguf/fast_mmvq.rs:36-50).
# Layouts as in ggml: Q5_K = Q4_K plus one high bit per weight (qh[l] bit 2c / 2c+1 for the low- / high-nibble
# sub-block of chunk c); Q4_0 / Q5_0 blocks of 32: element j < 16 from the low nibble of qs[j], element j + 16 from
# the high nibble, value (q - 8) d resp. (q - 16) d with the fifth bit from qh bit j / j + 16.
# ----------------------------------------------------------------------------

def q5_k_dequant(raw: np.ndarray, k: int) -> np.ndarray:
    """uint8 [rows, K/256*176] -> f32 [rows, K]."""
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    rows = raw.shape[0]
    nsb = k // QK_K
    blk = raw.reshape(rows, nsb, Q5_K_BYTES)
    d = blk[:, :, 0:2].copy().view(np.float16).astype(np.float32)
    dmin = blk[:, :, 2:4].copy().view(np.float16).astype(np.float32)
    sc, mn = q4_k_unpack_scales(blk[:, :, 4:16])
    qh = blk[:, :, 16:48]                                         # [rows, nsb, 32]
    qs = blk[:, :, 48:].reshape(rows, nsb, 4, 32)
    q = np.empty((rows, nsb, 8, 32), np.float32)
    for c in range(4):
        q[:, :, 2 * c, :] = ((qs[:, :, c, :] & 0x0F) | (((qh >> (2 * c)) & 1) << 4)).astype(np.float32)
        q[:, :, 2 * c + 1, :] = ((qs[:, :, c, :] >> 4) | (((qh >> (2 * c + 1)) & 1) << 4)).astype(np.float32)
    d1 = (d * sc.astype(np.float32))[..., None]
    m1 = (dmin * mn.astype(np.float32))[..., None]
    return (d1 * q - m1).reshape(rows, k)


def q4_0_dequant(raw: np.ndarray, k: int) -> np.ndarray:
    """uint8 [rows, K/32*18] -> f32 [rows, K]."""
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    rows = raw.shape[0]
    blk = raw.reshape(rows, k // 32, Q4_0_BYTES)
    d = blk[:, :, 0:2].copy().view(np.float16).astype(np.float32)
    qs = blk[:, :, 2:]
    q = np.concatenate([(qs & 0x0F).astype(np.int32), (qs >> 4).astype(np.int32)], axis=2) - 8
    return (d * q.astype(np.float32)).reshape(rows, k)


def q5_0_dequant(raw: np.ndarray, k: int) -> np.ndarray:
    """uint8 [rows, K/32*22] -> f32 [rows, K]."""
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    rows = raw.shape[0]
    blk = raw.reshape(rows, k // 32, Q5_0_BYTES)
    d = blk[:, :, 0:2].copy().view(np.float16).astype(np.float32)
    qh = blk[:, :, 2:6].copy().view(np.uint32).astype(np.int64)    # [rows, nb, 1]
    qs = blk[:, :, 6:]
    j = np.arange(16)
    lo = (qs & 0x0F).astype(np.int64) | (((qh >> j) & 1) << 4)
    hi = (qs >> 4).astype(np.int64) | (((qh >> (j + 16)) & 1) << 4)
    q = np.concatenate([lo, hi], axis=2) - 16
    return (d * q.astype(np.float32)).reshape(rows, k)


# ----------------------------------------------------------------------------
# Q4_1, Q5_1, Q2_K, Q3_K (the rest of the reference's decode list, hanzo-quant/src/gguf/fast_mmvq.rs:36-50).
# Layouts as in ggml.  Q4_1 / Q5_1 = Q4_0 / Q5_0 with an f16 minimum behind d and value q d + m.  Q2_K / Q3_K hold
# 2-bit codes four to a byte: per 128-weight half, byte l (0..31) of its 32 code bytes gives the weights l, l + 32,
# l + 64, l + 96 (bits 0-1, 2-3, 4-5, 6-7), and the 16-weight group of weight 128 h + 32 j + l is 8 h + 2 j + l // 16.
# Q2_K: value = d (s & 15) q - dmin (s >> 4) with one byte s per group.  Q3_K: value = d (scale - 32) (q - 4 (1 - hb))
# with hb = bit 4 h + j of hmask[l] and 6-bit scales packed in 12 bytes (low nibbles of bytes 0..7 for groups 0..7,
# high nibbles for groups 8..15, bits 4-5 of group 4 a + b in bits 2 a, 2 a + 1 of byte 8 + b).
# ----------------------------------------------------------------------------

def q4_1_dequant(raw: np.ndarray, k: int) -> np.ndarray:
    """uint8 [rows, K/32*20] -> f32 [rows, K]."""
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    rows = raw.shape[0]
    blk = raw.reshape(rows, k // 32, Q4_1_BYTES)
    d = blk[:, :, 0:2].copy().view(np.float16).astype(np.float32)
    m = blk[:, :, 2:4].copy().view(np.float16).astype(np.float32)
    qs = blk[:, :, 4:]
    q = np.concatenate([(qs & 0x0F), (qs >> 4)], axis=2).astype(np.float32)
    return (d * q + m).reshape(rows, k)


def q5_1_dequant(raw: np.ndarray, k: int) -> np.ndarray:
    """uint8 [rows, K/32*24] -> f32 [rows, K]."""
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    rows = raw.shape[0]
    blk = raw.reshape(rows, k // 32, Q5_1_BYTES)
    d = blk[:, :, 0:2].copy().view(np.float16).astype(np.float32)
    m = blk[:, :, 2:4].copy().view(np.float16).astype(np.float32)
    qh = blk[:, :, 4:8].copy().view(np.uint32).astype(np.int64)    # [rows, nb, 1]
    qs = blk[:, :, 8:]
    j = np.arange(16)
    lo = (qs & 0x0F).astype(np.int64) | (((qh >> j) & 1) << 4)
    hi = (qs >> 4).astype(np.int64) | (((qh >> (j + 16)) & 1) << 4)
    q = np.concatenate([lo, hi], axis=2).astype(np.float32)
    return (d * q + m).reshape(rows, k)


def _two_bit_codes(qs: np.ndarray) -> np.ndarray:
    """uint8 [rows, nsb, 64] -> int32 [rows, nsb, 2, 4, 32]: [half][j][l] = weight 128 half + 32 j + l."""
    rows, nsb = qs.shape[:2]
    q = qs.reshape(rows, nsb, 2, 1, 32).astype(np.int32)
    shifts = (2 * np.arange(4)).reshape(1, 1, 1, 4, 1)
    return (q >> shifts) & 3


def q2_k_dequant(raw: np.ndarray, k: int) -> np.ndarray:
    """uint8 [rows, K/256*84] -> f32 [rows, K]."""
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    rows = raw.shape[0]
    nsb = k // QK_K
    blk = raw.reshape(rows, nsb, Q2_K_BYTES)
    sc = blk[:, :, 0:16]
    d = blk[:, :, 80:82].copy().view(np.float16).astype(np.float32)       # [rows, nsb, 1]
    dmin = blk[:, :, 82:84].copy().view(np.float16).astype(np.float32)
    dl = d * (sc & 0x0F).astype(np.float32)                               # [rows, nsb, 16], group 8 h + 2 j + u
    ml = dmin * (sc >> 4).astype(np.float32)
    dl = np.repeat(dl.reshape(rows, nsb, 2, 4, 2), 16, axis=-1)           # [half][j][l]
    ml = np.repeat(ml.reshape(rows, nsb, 2, 4, 2), 16, axis=-1)
    q = _two_bit_codes(blk[:, :, 16:80]).astype(np.float32)
    return (dl * q - ml).reshape(rows, k).astype(np.float32)


def q3_k_unpack_scales(sc12: np.ndarray) -> np.ndarray:
    """uint8 [..., 12] -> int32 [..., 16]: the 6-bit scales (before the -32)."""
    lo = np.concatenate([sc12[..., 0:8] & 0x0F, sc12[..., 0:8] >> 4], axis=-1).astype(np.int32)   # groups 0..15
    hb = sc12[..., 8:12].astype(np.int32)
    a = np.arange(16) // 4
    b = np.arange(16) % 4
    hi = (hb[..., b] >> (2 * a)) & 3
    return lo | (hi << 4)


def q3_k_dequant(raw: np.ndarray, k: int) -> np.ndarray:
    """uint8 [rows, K/256*110] -> f32 [rows, K]."""
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    rows = raw.shape[0]
    nsb = k // QK_K
    blk = raw.reshape(rows, nsb, Q3_K_BYTES)
    hm = blk[:, :, 0:32].astype(np.int32)                                 # [rows, nsb, 32]
    d = blk[:, :, 108:110].copy().view(np.float16).astype(np.float32)     # [rows, nsb, 1]
    scale = (q3_k_unpack_scales(blk[:, :, 96:108]) - 32).astype(np.float32)
    dl = np.repeat((d * scale).reshape(rows, nsb, 2, 4, 2), 16, axis=-1)  # [half][j][l]
    q = _two_bit_codes(blk[:, :, 32:96])
    bit = (4 * np.arange(2).reshape(2, 1) + np.arange(4).reshape(1, 4)).reshape(1, 1, 2, 4, 1)
    hb = (hm.reshape(rows, nsb, 1, 1, 32) >> bit) & 1
    q = (q - 4 * (1 - hb)).astype(np.float32)
    return (dl * q).reshape(rows, k).astype(np.float32)


_GGML_LAYOUT = {"Q6_K": (256, 210, [208]), "Q5_K": (256, 176, [0, 2]), "Q4_0": (32, 18, [0]), "Q5_0": (32, 22, [0]),
                "Q4_1": (32, 20, [0, 2]), "Q5_1": (32, 24, [0, 2]), "Q2_K": (256, 84, [80, 82]), "Q3_K": (256, 110, [108])}


def ggml_random_blocks(fmt: str, rng, rows: int, k: int, d_lo: float = 2e-4, d_hi: float = 3e-3) -> np.ndarray:
    """Random valid blocks of a GGML type whose every bit pattern is valid (Q6_K, Q5_K, Q4_0, Q5_0, Q4_1, Q5_1, Q2_K,
    Q3_K), with the f16 scale fields drawn from [d_lo, d_hi] so that the weights have the magnitude of N(0, 0.02^2)
    weights: test and benchmark input for types the oracle has no quantizer for."""
    per, nbytes, scale_off = _GGML_LAYOUT[fmt]
    nb = k // per
    blk = rng.integers(0, 256, (rows, nb, nbytes), dtype=np.uint8)
    for off in scale_off:
        blk[:, :, off:off + 2] = np.asarray(rng.uniform(d_lo, d_hi, (rows, nb, 1)), np.float16).view(np.uint8)
    return blk.reshape(rows, nb * nbytes)


GGML_DEQUANT = {"Q8_0": q8_0_dequant, "Q4_K": q4_k_dequant, "Q6_K": q6_k_dequant, "Q5_K": q5_k_dequant,
                "Q4_0": q4_0_dequant, "Q5_0": q5_0_dequant, "Q4_1": q4_1_dequant, "Q5_1": q5_1_dequant,
                "Q2_K": q2_k_dequant, "Q3_K": q3_k_dequant}


def _nearest_int(f: np.ndarray) -> np.ndarray:
    # round-half-even of a float32, as the magic-number trick in ggml does
    return np.rint(np.asarray(f, dtype=np.float32)).astype(np.int32)


def _fit_scale_min(x: np.ndarray, wts: np.ndarray, nmax: int, nstep: int = 20,
                   rmin: float = -1.0, rdelta: float = 0.1):
    """Weighted least-squares (scale, min) search over 32-vectors, the published
    ggml `make_qkx2_quants` procedure, vectorised over the leading axis.
    Returns (scale >= 0, minus_min >= 0)."""
    x = x.astype(np.float32)
    lo = np.minimum(x.min(1), 0.0).astype(np.float32)
    hi = x.max(1).astype(np.float32)
    span = hi - lo
    ok = span > 0
    sw = wts.sum(1)
    sx = (wts * x).sum(1)
    span_s = np.where(ok, span, 1.0)
    inv = np.where(ok, nmax / span_s, 0.0).astype(np.float32)
    scale = np.where(ok, span_s / nmax, 0.0).astype(np.float32)
    lv = np.clip(_nearest_int(inv[:, None] * (x - lo[:, None])), 0, nmax)
    err = scale[:, None] * lv + lo[:, None] - x
    best = (wts * err * err).sum(1)
    cur_lo = lo.copy()
    for step in range(nstep + 1):
        den = np.where(ok, hi - cur_lo, 1.0)
        inv = np.where(ok, (rmin + rdelta * step + nmax) / den, 0.0).astype(np.float32)
        la = np.clip(_nearest_int(inv[:, None] * (x - cur_lo[:, None])), 0, nmax).astype(np.float64)
        sl = (wts * la).sum(1)
        sl2 = (wts * la * la).sum(1)
        sxl = (wts * la * x).sum(1)
        det = sw * sl2 - sl * sl
        good = ok & (det > 0)
        det_s = np.where(good, det, 1.0)
        s_new = (sw * sxl - sx * sl) / det_s
        m_new = (sl2 * sx - sl * sxl) / det_s
        clip = m_new > 0.0
        s_new = np.where(clip, sxl / np.where(sl2 > 0, sl2, 1.0), s_new)
        m_new = np.where(clip, 0.0, m_new)
        e = s_new[:, None] * la + m_new[:, None] - x
        mad = (wts * e * e).sum(1)
        take = good & (mad < best)
        best = np.where(take, mad, best)
        scale = np.where(take, s_new, scale)
        cur_lo = np.where(take, m_new, cur_lo)
    return scale.astype(np.float32), (-cur_lo).astype(np.float32)


def q4_k_quantize(w: np.ndarray) -> np.ndarray:
    """f32 [rows, K] (K % 256 == 0) -> uint8 [rows, K/256*144], the published
    ggml `quantize_row_q4_K_ref` procedure (what the reference's Python
    converter, scripts/convert_fp8_to_gguf.py:155-216, also follows)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, k = w.shape
    assert k % QK_K == 0
    nsb = rows * (k // QK_K)
    sub = w.reshape(nsb * 8, 32)
    rms = np.sqrt((sub * sub).sum(1) / 32.0)
    sc_f, mn_f = _fit_scale_min(sub, rms[:, None] + np.abs(sub), 15)
    sc_f = sc_f.reshape(nsb, 8)
    mn_f = mn_f.reshape(nsb, 8)
    top_s = sc_f.max(1)
    top_m = mn_f.max(1)
    inv_s = np.where(top_s > 0, 63.0 / np.where(top_s > 0, top_s, 1.0), 0.0)
    inv_m = np.where(top_m > 0, 63.0 / np.where(top_m > 0, top_m, 1.0), 0.0)
    ls = np.minimum(_nearest_int(inv_s[:, None] * sc_f), 63).astype(np.uint8)
    lm = np.minimum(_nearest_int(inv_m[:, None] * mn_f), 63).astype(np.uint8)
    packed = np.zeros((nsb, 12), np.uint8)
    packed[:, 0:4] = ls[:, 0:4] | ((ls[:, 4:8] >> 4) << 6)
    packed[:, 4:8] = lm[:, 0:4] | ((lm[:, 4:8] >> 4) << 6)
    packed[:, 8:12] = (ls[:, 4:8] & 0x0F) | ((lm[:, 4:8] & 0x0F) << 4)
    d = (top_s / 63.0).astype(np.float16)
    dmin = (top_m / 63.0).astype(np.float16)
    sc_i, mn_i = q4_k_unpack_scales(packed)
    d1 = d.astype(np.float32)[:, None] * sc_i.astype(np.float32)
    m1 = dmin.astype(np.float32)[:, None] * mn_i.astype(np.float32)
    vals = w.reshape(nsb, 8, 32)
    d1s = np.where(d1 != 0, d1, 1.0)[:, :, None]
    lvl = np.where(d1[:, :, None] != 0,
                   np.clip(_nearest_int((vals + m1[:, :, None]) / d1s), 0, 15), 0).astype(np.uint8)
    qs = (lvl[:, 0::2, :] | (lvl[:, 1::2, :] << 4)).reshape(nsb, 128)
    out = np.concatenate([d.view(np.uint8).reshape(nsb, 2), dmin.view(np.uint8).reshape(nsb, 2),
                          packed, qs], axis=1)
    return out.reshape(rows, (k // QK_K) * Q4_K_BYTES)


# ----------------------------------------------------------------------------
# FP8 e4m3 (weights with 128x128 f32 block scales, activations with 1x128 scales)
# ----------------------------------------------------------------------------


def _build_e4m3_table() -> np.ndarray:
    """All 256 e4m3fn codes -> f32.  4 exponent bits (bias 7), 3 mantissa bits,
    no infinities, 0x7f/0xff are NaN, largest finite 448."""
    t = np.zeros(256, np.float32)
    for c in range(256):
        s = -1.0 if c & 0x80 else 1.0
        e = (c >> 3) & 0xF
        m = c & 7
        if e == 0xF and m == 7:
            v = np.nan
        elif e == 0:
            v = s * (m / 8.0) * 2.0 ** (-6)
        else:
            v = s * (1.0 + m / 8.0) * 2.0 ** (e - 7)
        t[c] = v
    return t


E4M3_TABLE = _build_e4m3_table()


def e4m3_decode(codes: np.ndarray) -> np.ndarray:
    return E4M3_TABLE[np.asarray(codes, dtype=np.uint8)]


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """f32 -> e4m3fn code, round-to-nearest-even, inputs already clamped to +-448
    (the reference clamps before converting: blockwise_fp8/ops.rs:399)."""
    x = np.asarray(x, dtype=np.float32)
    a = np.abs(x).astype(np.float64)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    # quantum of the target grid at |x|: 2^-9 below 2^-6 (subnormals), else 2^(floor(log2 a) - 3)
    with np.errstate(divide="ignore"):
        ex = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    ex = np.clip(ex, -6, 8)
    q = 2.0 ** (ex - 3)
    n = np.rint(a / q)                     # numpy rint = half-to-even
    v = np.minimum(n * q, FP8_MAX)
    # re-derive exponent after rounding (n may have carried to the next binade)
    with np.errstate(divide="ignore"):
        ex2 = np.floor(np.log2(np.where(v > 0, v, 1.0)))
    ex2 = np.clip(ex2, -6, 8)
    sub = v < 2.0 ** (-6)
    mant = np.where(sub, np.rint(v / 2.0 ** (-9)), np.rint((v / 2.0 ** ex2 - 1.0) * 8.0)).astype(np.int64)
    expo = np.where(sub, 0, ex2 + 7).astype(np.int64)
    code = (expo << 3 | mant).astype(np.uint8)
    return (code | sign).astype(np.uint8)


def fp8_block_dequant(codes: np.ndarray, scale: np.ndarray, by: int = 128, bx: int = 128) -> np.ndarray:
    """e4m3 [N, K] x scale [ceil(N/by), ceil(K/bx)] -> f32 [N, K]; edge blocks are
    clipped (hanzo-quant/src/blockwise_fp8/ops.rs:11-59)."""
    n, k = codes.shape
    s = np.repeat(np.repeat(scale.astype(np.float32), by, axis=0), bx, axis=1)[:n, :k]
    return e4m3_decode(codes) * s


def fp8_block_quant(w: np.ndarray, by: int = 128, bx: int = 128):
    """f32 [N, K] -> (codes uint8 [N, K], scale f32 [ceil(N/by), ceil(K/bx)]).
    scale = absmax/448 (1e-12 for an all-zero block), q = e4m3(clamp(v/scale, +-448))
    (blockwise_fp8/ops.rs:329-411)."""
    w = np.asarray(w, dtype=np.float32)
    n, k = w.shape
    gy, gx = -(-n // by), -(-k // bx)
    pad = np.zeros((gy * by, gx * bx), np.float32)
    pad[:n, :k] = w
    blk = pad.reshape(gy, by, gx, bx)
    amax = np.abs(blk).max(axis=(1, 3))
    scale = np.where(amax > 0, amax / np.float32(FP8_MAX), np.float32(1e-12)).astype(np.float32)
    scaled = np.clip(blk / scale[:, None, :, None], -FP8_MAX, FP8_MAX).astype(np.float32)
    codes = e4m3_encode(scaled).reshape(gy * by, gx * bx)[:n, :k]
    return np.ascontiguousarray(codes), scale


def fp8_vector_quant(x: np.ndarray, group: int = 128):
    """flat groups of `group` elements: scale = absmax/448 (or 1e-12), codes as
    above (hanzo-quant/src/vector_fp8/ops.rs:235-287).  x [..., K], K % group == 0
    -> (codes uint8 same shape, scale f32 [..., K/group])."""
    x = np.asarray(x, dtype=np.float32)
    shp = x.shape
    g = x.reshape(-1, group)
    amax = np.abs(g).max(1)
    scale = np.where(amax > 0, amax / np.float32(FP8_MAX), np.float32(1e-12)).astype(np.float32)
    scaled = np.clip(g / scale[:, None], -FP8_MAX, FP8_MAX).astype(np.float32)
    codes = e4m3_encode(scaled).reshape(shp)
    return codes, scale.reshape(shp[:-1] + (shp[-1] // group,))


def fp8_vector_dequant(codes: np.ndarray, scale: np.ndarray, group: int = 128) -> np.ndarray:
    """inverse of fp8_vector_quant (vector_fp8/ops.rs, KAT :459-480)."""
    v = e4m3_decode(codes)
    return v * np.repeat(scale.astype(np.float32), group, axis=-1)


# ----------------------------------------------------------------------------
# MXFP4 (e2m1 nibbles, 32-element blocks, e8m0 shared exponent)
# ----------------------------------------------------------------------------

FP4_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
                       -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], np.float32)


def e8m0_to_f32(s: np.ndarray) -> np.ndarray:
    """The reference builds the scale as f32::from_bits(s << 23)
    (hanzo-quant/src/mxfp4/mod.rs:480): s = 0 decodes to 0.0, s = 255 to +inf."""
    return (np.asarray(s, dtype=np.uint32) << np.uint32(23)).view(np.float32)


def mxfp4_quantize(w: np.ndarray):
    """f32 [N, K] -> (blocks uint8 [N, K/2], scales uint8 [N, K/32])
    (mxfp4/mod.rs:216-333).  e = clamp(floor(log2(absmax/6)) + 127, 0, 254), 127
    for an all-zero block; nibble chosen by midpoint thresholds; byte i holds
    element 2i in its low nibble and 2i+1 in its high nibble."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    n, k = w.shape
    assert k % MXFP4_BLOCK == 0
    blk = w.reshape(n, k // MXFP4_BLOCK, MXFP4_BLOCK)
    amax = np.abs(blk).max(2)
    with np.errstate(divide="ignore"):
        raw = np.floor(np.log2((amax / np.float32(6.0)).astype(np.float32))).astype(np.float64) + 127
    e = np.where(amax == 0, 127, np.clip(raw, 0, 254)).astype(np.uint8)
    sf = np.exp2(e.astype(np.float32) - 127).astype(np.float32)
    inv = np.where(sf == 0, np.float32(0), np.float32(1) / sf).astype(np.float32)
    v = blk * inv[:, :, None]
    a = np.abs(v)
    nib = np.select([a < 0.25, a < 0.75, a < 1.25, a < 1.75, a < 2.5, a < 3.5, a < 5.0],
                    [0, 1, 2, 3, 4, 5, 6], default=7).astype(np.uint8)
    nib = nib | ((v < 0).astype(np.uint8) << 3)
    nib = nib.reshape(n, k)
    packed = (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8)
    return packed, e


def mxfp4_dequant(blocks: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """(uint8 [N, K/2], uint8 [N, K/32]) -> f32 [N, K] via the reference's
    DEQUANT_LUT[scale][nibble] = fp4[nibble] * from_bits(scale << 23)
    (mxfp4/mod.rs:473-545)."""
    blocks = np.asarray(blocks, dtype=np.uint8)
    n, kh = blocks.shape
    k = kh * 2
    nib = np.empty((n, k), np.uint8)
    nib[:, 0::2] = blocks & 0x0F
    nib[:, 1::2] = blocks >> 4
    sf = np.repeat(e8m0_to_f32(scales), MXFP4_BLOCK, axis=1)
    with np.errstate(invalid="ignore"):
        return FP4_VALUES[nib] * sf


# ----------------------------------------------------------------------------
# MXFP8 activations (e4m3 elements, 32-element blocks, e8m0 shared exponent)
# ----------------------------------------------------------------------------

def mxfp8_quant(x: np.ndarray):
    """f32 [..., K] -> (codes uint8 [..., K], scales uint8 [..., K/32]).  The reference has no MXFP8 quantizer; this
    is the OCP microscaling rule for e4m3 elements with the structure of MXFP4Layer::quantize
    (hanzo-quant/src/mxfp4/mod.rs:216-300): e = clamp(floor(log2(absmax)) - 8 + 127, 0, 254) (8 = exponent of
    e4m3's largest binade), 127 for an all-zero block; elements times 2^-(e-127), clamped to +-448, rounded to
    nearest even."""
    x = np.asarray(x, dtype=np.float32)
    shp = x.shape
    g = x.reshape(-1, MXFP4_BLOCK)
    amax = np.abs(g).max(1)
    ex = ((amax.view(np.uint32) >> np.uint32(23)) & np.uint32(0xFF)).astype(np.int64) - 127   # floor(log2), normals
    e = np.where(amax > 0, np.clip(ex - 8 + 127, 0, 254), 127).astype(np.uint8)
    inv = ((np.uint32(254) - e.astype(np.uint32)) << np.uint32(23)).view(np.float32)
    with np.errstate(over="ignore", invalid="ignore"):
        scaled = np.clip(g * inv[:, None], -FP8_MAX, FP8_MAX).astype(np.float32)
    codes = e4m3_encode(scaled).reshape(shp)
    return codes, e.reshape(shp[:-1] + (shp[-1] // MXFP4_BLOCK,))


def mxfp8_dequant(codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """inverse of mxfp8_quant: e4m3 value times 2^(scale - 127) per 32-element block."""
    return e4m3_decode(codes) * np.repeat(e8m0_to_f32(scales), MXFP4_BLOCK, axis=-1)


# ----------------------------------------------------------------------------
# 16-bit rounding helpers
# ----------------------------------------------------------------------------


def round_bf16(x: np.ndarray) -> np.ndarray:
    """f32 -> nearest-even bf16, returned as f32."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    return (round_bf16(x).view(np.uint32) >> 16).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
