"""The index arithmetic of the two kernels that pick GGML blocks apart, restated in numpy and checked against the
oracle's dequantizers: which bytes, shifts and masks give which weight.

* `hq::gm_decode_span` (engine_b200/csrc/hq_gemv_ggml_mma.cu): lane t of a quad decodes the four weights 4t..4t+3 of
  every 16-weight group of a 256-weight span from one 32-bit word of code bits (+ one of high bits);
* `hq::fetch_a` / `emit_*` (engine_b200/csrc/hq_grouped_gemm.cu): a producer thread expands 16 consecutive weights
  (quarter q of a 64-weight stage) from four or five aligned words, funnel-shifted when the block starts in the
  middle of a word.

The restatement uses f32 products in the oracle's order, so a correct mapping reproduces the oracle bit for bit.  It
is how the mappings were settled before the kernels first ran; the kernels themselves are compared with the oracle by
the GPU tests."""
import numpy as np
import pytest

from oracle import formats as F

f32 = np.float32


def _f16(b, o):
    return float(np.frombuffer(bytes(b[o:o + 2]), dtype=np.float16)[0])


def _ld32(b, o):
    return int(b[o]) | int(b[o + 1]) << 8 | int(b[o + 2]) << 16 | int(b[o + 3]) << 24


def _bytes4(w):
    return [(w >> (8 * i)) & 0xFF for i in range(4)]


def _spread4(x):
    """four bits -> bit 0 of four bytes (the kernels' x * 0x00204081 & 0x01010101)"""
    return ((x & 0xF) * 0x00204081) & 0xFFFFFFFF & 0x01010101


def _q3k_aux(b, o):
    a0, a1, tm = _ld32(b, o), _ld32(b, o + 4), _ld32(b, o + 8)
    return [(a0 & 0x0F0F0F0F) | ((tm & 0x03030303) << 4), (a1 & 0x0F0F0F0F) | (((tm >> 2) & 0x03030303) << 4),
            ((a0 >> 4) & 0x0F0F0F0F) | (((tm >> 4) & 0x03030303) << 4),
            ((a1 >> 4) & 0x0F0F0F0F) | (((tm >> 6) & 0x03030303) << 4)]


def _k4_scale_min(hdr, j):
    if j < 4:
        return (hdr[1] >> (8 * j)) & 63, (hdr[2] >> (8 * j)) & 63
    jj = j - 4
    return (((hdr[3] >> (8 * jj)) & 0xF) | (((hdr[1] >> (8 * jj + 6)) & 3) << 4),
            ((hdr[3] >> (8 * jj + 4)) & 0xF) | (((hdr[2] >> (8 * jj + 6)) & 3) << 4))


# ---- the decode kernel: one 256-weight span -------------------------------------------------------------------------

def decode_span(fmt, b):
    out = np.zeros(256, f32)
    for t in range(4):
        if fmt == "Q6_K":
            d = _f16(b, 208)
            for h in range(2):
                for u in range(2):
                    qh = _ld32(b, 128 + 32 * h + 16 * u + 4 * t)
                    for jlo in range(2):
                        ql = _ld32(b, 64 * h + 32 * jlo + 16 * u + 4 * t)
                        for jhi in range(2):
                            j = jlo + 2 * jhi
                            s16 = 8 * h + 2 * j + u
                            qq = ((ql >> (4 * jhi)) & 0x0F0F0F0F) | (((qh >> (2 * j)) & 0x03030303) << 4)
                            sc = int(np.int8(b[192 + s16]))
                            for i, q in enumerate(_bytes4(qq)):
                                out[16 * s16 + 4 * t + i] = f32(d) * f32(sc) * f32(q - 32)
        elif fmt == "Q5_K":
            hdr = [_ld32(b, 4 * i) for i in range(4)]
            d, dmin = _f16(b, 0), _f16(b, 2)
            qh = [_ld32(b, 16 + 16 * u + 4 * t) for u in range(2)]
            for c in range(4):
                w = [_ld32(b, 48 + 32 * c + 16 * u + 4 * t) for u in range(2)]
                for hi in range(2):
                    j = 2 * c + hi
                    sc, mn = _k4_scale_min(hdr, j)
                    for u in range(2):
                        qq = ((w[u] >> (4 * hi)) & 0x0F0F0F0F) | (((qh[u] >> j) & 0x01010101) << 4)
                        for i, q in enumerate(_bytes4(qq)):
                            out[32 * j + 16 * u + 4 * t + i] = f32(d * sc) * f32(q) - f32(dmin * mn)
        elif fmt == "Q2_K":
            d, dmin = _f16(b, 80), _f16(b, 82)
            sc = [_ld32(b, 4 * i) for i in range(4)]
            for h in range(2):
                for u in range(2):
                    w = _ld32(b, 16 + 32 * h + 16 * u + 4 * t)
                    for j in range(4):
                        s16 = 8 * h + 2 * j + u
                        s = (sc[s16 >> 2] >> (8 * (s16 & 3))) & 0xFF
                        for i, q in enumerate(_bytes4((w >> (2 * j)) & 0x03030303)):
                            out[16 * s16 + 4 * t + i] = f32(f32(d) * f32(s & 15)) * f32(q) - f32(f32(dmin) * f32(s >> 4))
        elif fmt == "Q3_K":
            aux = _q3k_aux(b, 96)
            d = _f16(b, 108)
            for u in range(2):
                hm = _ld32(b, 16 * u + 4 * t)
                for h in range(2):
                    w = _ld32(b, 32 + 32 * h + 16 * u + 4 * t)
                    for j in range(4):
                        s16 = 8 * h + 2 * j + u
                        qq = ((w >> (2 * j)) & 0x03030303) | (((hm >> (4 * h + j)) & 0x01010101) << 2)
                        s = ((aux[s16 >> 2] >> (8 * (s16 & 3))) & 0xFF) - 32
                        for i, q in enumerate(_bytes4(qq)):
                            out[16 * s16 + 4 * t + i] = f32(f32(d) * f32(s)) * f32(q - 4)
        else:
            five, has_min = fmt in ("Q5_0", "Q5_1"), fmt in ("Q4_1", "Q5_1")
            bb = 18 + 4 * five + 2 * has_min
            zero = 0 if has_min else (16 if five else 8)
            for blk in range(8):
                k = b[bb * blk:bb * blk + bb]
                d, m = _f16(k, 0), (_f16(k, 2) if has_min else 0.0)
                w = _ld32(k, bb - 16 + 4 * t)
                qh = (_ld32(k, 4 if has_min else 2) >> (4 * t)) if five else 0
                for hf in range(2):
                    qq = (w >> (4 * hf)) & 0x0F0F0F0F
                    if five:
                        qq |= _spread4(qh >> (16 * hf)) << 4
                    for i, q in enumerate(_bytes4(qq)):
                        out[32 * blk + 16 * hf + 4 * t + i] = f32(d) * f32(q - zero) + f32(m)
    return out


@pytest.mark.parametrize("fmt", ["Q6_K", "Q5_K", "Q4_0", "Q5_0", "Q4_1", "Q5_1", "Q2_K", "Q3_K"])
def test_decode_kernel_lane_map(fmt):
    rng = np.random.Generator(np.random.PCG64(11))
    raw = F.ggml_random_blocks(fmt, rng, 3, 256)
    want = F.GGML_DEQUANT[fmt](raw, 256)
    for r in range(3):
        assert np.array_equal(decode_span(fmt, raw[r]), want[r]), fmt


# ---- the grouped GEMM's producers: 16 consecutive weights per thread ------------------------------------------------

def _words(buf, addr, n):
    return [int.from_bytes(bytes(buf[addr + 4 * i:addr + 4 * i + 4]).ljust(4, b"\0"), "little") for i in range(n)]


def _funnel(lo, hi, sh):
    return ((lo | (hi << 32)) >> sh) & 0xFFFFFFFF


def _five_words(buf, p):
    """the 16 bytes at the 2-byte aligned address p as four aligned words, a fifth when p is 2 bytes off"""
    mis = p & 2
    w = _words(buf, p - mis, 4) + [_words(buf, p - mis + 16, 1)[0] if mis else 0]
    return [_funnel(w[i], w[i + 1], 8 * mis) for i in range(4)]


def producer_row(fmt, buf, base, k):
    """`buf`: bytes of a 16-byte aligned tensor, `base`: offset of the row in it."""
    out = np.zeros(k, f32)
    for k0 in range(0, k, 64):
        for q in range(4):
            pos = (k0 & 255) + 16 * q
            h, j, u = pos >> 7, (pos >> 5) & 3, (pos >> 4) & 1
            o = k0 + 16 * q
            if fmt == "Q5_K":
                blk = base + 176 * (k0 >> 8)
                c, hi = (k0 & 255) >> 6, q >> 1
                hdr = _words(buf, blk, 4)
                qw = _words(buf, blk + 48 + 32 * c + 16 * (q & 1), 4)
                hw = _words(buf, blk + 16 + 16 * (q & 1), 4)
                jj = 2 * c + hi
                sc, mn = _k4_scale_min(hdr, jj)
                d, dmin = _f16(buf, blk), _f16(buf, blk + 2)
                for i in range(4):
                    vm = (((qw[i] >> 4) if hi else qw[i]) & 0x0F0F0F0F) | (((hw[i] >> jj) & 0x01010101) << 4)
                    for t, code in enumerate(_bytes4(vm)):
                        out[o + 4 * i + t] = f32(d * sc) * f32(code) - f32(dmin * mn)
            elif fmt == "Q2_K":
                blk = base + 84 * (k0 >> 8)
                qw = _words(buf, blk + 16 + 32 * h + 16 * u, 4)
                s = int(buf[blk + 8 * h + 2 * j + u])
                d, dmin = _f16(buf, blk + 80), _f16(buf, blk + 82)
                for i in range(4):
                    for t, code in enumerate(_bytes4((qw[i] >> (2 * j)) & 0x03030303)):
                        out[o + 4 * i + t] = f32(f32(d) * f32(s & 15)) * f32(code) - f32(f32(dmin) * f32(s >> 4))
            elif fmt in ("Q6_K", "Q3_K"):
                if fmt == "Q6_K":
                    blk = base + 210 * (k0 >> 8)
                    lw = _five_words(buf, blk + 64 * h + 32 * (j & 1) + 16 * u)
                    hw = _five_words(buf, blk + 128 + 32 * h + 16 * u)
                    d, sc = _f16(buf, blk + 208), int(np.int8(buf[blk + 192 + 8 * h + 2 * j + u]))
                    for i in range(4):
                        nib = (lw[i] if j < 2 else (lw[i] >> 4)) & 0x0F0F0F0F
                        w6 = nib | (((hw[i] >> (2 * j)) & 0x03030303) << 4)
                        for t, code in enumerate(_bytes4(w6)):
                            out[o + 4 * i + t] = f32(d) * f32(sc) * f32(code - 32)
                else:
                    blk = base + 110 * (k0 >> 8)
                    lw = _five_words(buf, blk + 32 + 32 * h + 16 * u)
                    hw = _five_words(buf, blk + 16 * u)
                    s16 = 8 * h + 2 * j + u
                    a, b = s16 >> 2, s16 & 3
                    nib, top = int(buf[blk + 96 + 4 * (a & 1) + b]), int(buf[blk + 104 + b])
                    sc6 = ((nib & 15) if a < 2 else (nib >> 4)) | (((top >> (2 * a)) & 3) << 4)
                    d = _f16(buf, blk + 108)
                    for i in range(4):
                        w3 = ((lw[i] >> (2 * j)) & 0x03030303) | (((hw[i] >> (4 * h + j)) & 0x01010101) << 2)
                        for t, code in enumerate(_bytes4(w3)):
                            out[o + 4 * i + t] = f32(f32(d) * f32(sc6 - 32)) * f32(code - 4)
            else:
                five, has_min = fmt in ("Q5_0", "Q5_1"), fmt in ("Q4_1", "Q5_1")
                bb = 18 + 4 * five + 2 * has_min
                zero = 0 if has_min else (16 if five else 8)
                blk = base + bb * ((k0 >> 5) + (q >> 1))
                half = q & 1
                w = _five_words(buf, blk + bb - 16)
                d, m = _f16(buf, blk), (_f16(buf, blk + 2) if has_min else 0.0)
                qh_at = blk + (4 if has_min else 2) + 2 * half
                ext = (int(buf[qh_at]) | int(buf[qh_at + 1]) << 8) if five else 0
                for i in range(4):
                    vm = ((w[i] >> 4) if half else w[i]) & 0x0F0F0F0F
                    if five:
                        vm |= _spread4(ext >> (4 * i)) << 4
                    for t, code in enumerate(_bytes4(vm)):
                        out[o + 4 * i + t] = f32(d) * f32(code - zero) + f32(m)
    return out


@pytest.mark.parametrize("fmt", ["Q6_K", "Q5_K", "Q4_0", "Q5_0", "Q4_1", "Q5_1", "Q2_K", "Q3_K"])
def test_grouped_gemm_producer_map(fmt):
    # K = 768: three super-blocks per row, so Q6_K / Q3_K rows (630 / 330 bytes) alternate between word-aligned and two
    # bytes off, and so do the 18- / 22-byte blocks of Q4_0 / Q5_0 inside a row
    rng = np.random.Generator(np.random.PCG64(12))
    k = 768
    raw = F.ggml_random_blocks(fmt, rng, 4, k)
    want = F.GGML_DEQUANT[fmt](raw, k)
    flat, row_bytes = raw.reshape(-1), raw.shape[1]
    for r in range(4):
        assert np.array_equal(producer_row(fmt, flat, r * row_bytes, k), want[r]), (fmt, r)
