"""The oracle is pinned before it is trusted: golden vectors produced by the
reference's own Python converter / gguf-py, and the reference's known-answer
tests restated (file:line cited per test)."""
import numpy as np
import pytest

from oracle import formats as F


def test_q4_k_dequant_matches_gguf_py_on_reference_bytes(golden):
    got = F.q4_k_dequant(golden["q4_bytes"], 512)
    assert np.array_equal(got, golden["q4_deq"])


def test_q4_k_quantizer_matches_reference_converter(golden):
    # same published procedure as scripts/convert_fp8_to_gguf.py:155-216
    mine = F.q4_k_quantize(golden["w4"])
    ref = golden["q4_bytes"]
    assert mine.shape == ref.shape
    same = (mine == ref).mean()
    assert same > 0.999, same
    # and it is a sane quantizer in its own right
    err = F.q4_k_dequant(mine, 512)[:3] - golden["w4"][:3]
    assert np.sqrt((err ** 2).mean()) / np.sqrt((golden["w4"][:3] ** 2).mean()) < 0.09


def test_q8_0_matches_gguf_py(golden):
    assert np.array_equal(F.q8_0_quantize(golden["w8"]), golden["q8_bytes"])
    assert np.array_equal(F.q8_0_dequant(golden["q8_bytes"], 256), golden["q8_deq"])


def test_e4m3_table_matches_torch(golden):
    ref = golden["e4m3_all"]
    assert np.array_equal(np.isnan(ref), np.isnan(F.E4M3_TABLE))
    ok = ~np.isnan(ref)
    assert np.array_equal(ref[ok], F.E4M3_TABLE[ok])


def test_fp8_block_dequant_matches_reference_converter(golden):
    got = F.fp8_block_dequant(golden["fp8_codes"], golden["fp8_scale"])
    assert np.array_equal(got, golden["fp8_deq"])


def test_fp8_blockwise_dequant_kat():
    # hanzo-quant/src/blockwise_fp8/ops.rs:1098-1118: ones(5,5) e4m3, 2x2 blocks, scales arange(9)
    ones = np.full((5, 5), 0x38, np.uint8)          # 1.0 in e4m3
    s = np.arange(9, dtype=np.float32).reshape(3, 3)
    got = F.fp8_block_dequant(ones, s, 2, 2)
    want = np.array([[0, 0, 1, 1, 2], [0, 0, 1, 1, 2], [3, 3, 4, 4, 5], [3, 3, 4, 4, 5], [6, 6, 7, 7, 8]], np.float32)
    assert np.array_equal(got, want)


def test_fp8_vector_dequant_kat():
    # hanzo-quant/src/vector_fp8/ops.rs:459-480
    ones = np.full(256, 0x38, np.uint8)
    got = F.fp8_vector_dequant(ones, np.array([2.0, 3.0], np.float32))
    assert np.all(got[:128] == 2.0) and np.all(got[128:] == 3.0)


def test_fp8_quant_roundtrip_bounds():
    # The reference bounds the round trip statistically on unseeded data (block quant < 0.16 on
    # randn*2 with 4x4 blocks, blockwise_fp8/ops.rs:1302-1343; vector quant < 0.27 on N(0,2),
    # vector_fp8/ops.rs:482-520).  The exact property behind both: the error never exceeds half
    # a step of the top binade, 16 * scale.
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((16, 16)) * 2).astype(np.float32)
    c, s = F.fp8_block_quant(w, 4, 4)
    err = np.abs(F.fp8_block_dequant(c, s, 4, 4) - w)
    assert np.all(err <= np.repeat(np.repeat(s, 4, 0), 4, 1) * 16 * (1 + 1e-6))
    assert err.max() < 0.27
    x = (rng.standard_normal(256) * 2).astype(np.float32)
    c, s = F.fp8_vector_quant(x)
    assert s.shape == (2,)
    assert np.abs(F.fp8_vector_dequant(c, s) - x).max() < 0.27


def test_e4m3_encode_is_nearest_even():
    import ml_dtypes
    rng = np.random.default_rng(5)
    x = np.concatenate([rng.uniform(-448, 448, 4000), rng.normal(0, 1, 4000), rng.normal(0, 0.01, 2000),
                        F.E4M3_TABLE[~np.isnan(F.E4M3_TABLE)],
                        # exact midpoints between neighbouring codes
                        (F.E4M3_TABLE[1:0x7E] + F.E4M3_TABLE[2:0x7F]) / 2]).astype(np.float32)
    want = x.astype(ml_dtypes.float8_e4m3fn).view(np.uint8)
    got = F.e4m3_encode(x)
    # +0/-0 codes are both zero
    assert np.array_equal(F.e4m3_decode(got), F.e4m3_decode(want))


def test_all_zero_fp8_block_uses_tiny_scale():
    c, s = F.fp8_block_quant(np.zeros((4, 4), np.float32), 4, 4)
    assert s[0, 0] == np.float32(1e-12) and not c.any()


def test_mxfp4_value_table_and_block_dot():
    # hanzo-quant/src/mxfp4/dp4a.rs:176-204: value table, and one block of nibble 5 (3.0) at
    # scale e=127 against ones -> 96.0
    want = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]
    assert list(F.FP4_VALUES) == want
    blocks = np.full((1, 16), 0x55, np.uint8)
    scales = np.full((1, 1), 127, np.uint8)
    w = F.mxfp4_dequant(blocks, scales)
    assert float((w @ np.ones(32, np.float32))[0]) == 96.0


def test_mxfp4_scale_edge_codes():
    # f32::from_bits(s << 23): s=0 -> 0.0, s=255 -> inf (hanzo-quant/src/mxfp4/mod.rs:480)
    assert F.e8m0_to_f32(np.array([0, 127, 128, 255], np.uint8)).tolist() == [0.0, 1.0, 2.0, np.inf]


def test_mxfp4_quantize_roundtrip():
    rng = np.random.default_rng(11)
    w = rng.normal(0, 0.02, (8, 96)).astype(np.float32)
    w[1, :32] = 0
    b, s = F.mxfp4_quantize(w)
    assert b.shape == (8, 48) and s.shape == (8, 3)
    assert s[1, 0] == 127 and not b[1, :16].any()
    dq = F.mxfp4_dequant(b, s)
    rel = np.linalg.norm(dq - w) / np.linalg.norm(w)
    assert rel < 0.2
    # nibble order: element 2i low, 2i+1 high (mxfp4/mod.rs:262-270)
    w2 = np.zeros((1, 32), np.float32)
    w2[0, 0], w2[0, 1] = 6.0, -3.0
    b2, s2 = F.mxfp4_quantize(w2)
    assert s2[0, 0] == 127 and b2[0, 0] == (7 | (0xD << 4))


def test_bf16_rounding_helpers():
    import torch
    x = np.random.default_rng(0).standard_normal(1000).astype(np.float32)
    want = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(F.round_bf16(x), want)
    assert np.array_equal(F.from_bf16_bits(F.to_bf16_bits(x)), want)


@pytest.mark.parametrize("fmt", ["Q6_K", "Q5_K", "Q4_0", "Q5_0", "Q4_1", "Q5_1", "Q2_K", "Q3_K"])
def test_ggml_dequant_matches_gguf_py_bit_for_bit(fmt):
    """Random valid blocks (and, where a quantizer exists, quantized N(0, 0.02^2) weights) against gguf-py's
    dequantize; vectors from tests/golden/make_golden_ggml.py."""
    import os
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "ggml_vectors.npz"))
    got = F.GGML_DEQUANT[fmt](z["raw_" + fmt], 512)
    assert np.array_equal(got, z["deq_" + fmt])


def test_q6_k_quantizer_round_trip():
    rng = np.random.Generator(np.random.PCG64(606))
    w = rng.normal(0.0, 0.02, (5, 768)).astype(np.float32)
    w[2, :32] = 0.0
    raw = F.q6_k_quantize(w)
    assert raw.shape == (5, 3 * 210) and raw.dtype == np.uint8
    back = F.q6_k_dequant(raw, 768)
    # 6-bit codes: half a step of absmax / 31 per 16-element sub-block, plus the 8-bit scale's own rounding
    blk = np.abs(w.reshape(5, 48, 16)).max(2, keepdims=True)
    assert (np.abs(back - w).reshape(5, 48, 16) <= blk / 31 * 0.55 + 1e-9).all()
    assert not back[2, :32].any()
    # quantizing the dequantized weights again reproduces the same values
    assert np.array_equal(F.q6_k_dequant(F.q6_k_quantize(back), 768), back)
