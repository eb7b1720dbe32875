"""The MXFP8 activation quantizer of the oracle (OCP microscaling rule for e4m3 elements; the reference has no
such quantizer, its structure follows MXFP4Layer::quantize, hanzo-quant/src/mxfp4/mod.rs:216-300)."""
import numpy as np

from oracle import formats as F


def test_shared_exponent_rule():
    x = np.zeros((1, 5 * 32), np.float32)
    x[0, 0] = 448.0            # 2^8 * 1.75: exponent 8 - 8 = 0
    x[0, 32] = 1.0             # 2^0: 0 - 8
    x[0, 64] = 3.0e-3          # 2^-9 * 1.536: -9 - 8
    x[0, 96] = 512.0           # 2^9: 9 - 8 = 1 (512 / 2 = 256, representable)
    # block 4 stays zero: exponent byte 127
    codes, scales = F.mxfp8_quant(x)
    assert scales.tolist() == [[127, 119, 110, 128, 127]]
    back = F.mxfp8_dequant(codes, scales)
    assert back[0, 0] == 448.0 and back[0, 32] == 1.0 and back[0, 96] == 512.0
    assert abs(back[0, 64] - 3.0e-3) <= 3.0e-3 / 16
    assert not back[0, 128:].any()


def test_round_trip_error_and_idempotence():
    rng = np.random.Generator(np.random.PCG64(77))
    x = (rng.standard_normal((16, 256)) * np.exp2(rng.integers(-20, 20, (16, 1)))).astype(np.float32)
    codes, scales = F.mxfp8_quant(x)
    back = F.mxfp8_dequant(codes, scales)
    # e4m3 keeps 3 mantissa bits (half a step = 1/16 of the element's binade); a block maximum between 448 and 512
    # times the shared scale saturates at 448, which costs up to 1/8
    blk = np.abs(x.reshape(16, 8, 32)).max(2, keepdims=True)
    err = np.abs(back - x).reshape(16, 8, 32)
    assert (err <= blk / 8 * 1.0001).all()
    assert (err <= np.maximum(np.abs(x).reshape(16, 8, 32) / 8, blk / 2 ** 9) * 1.0001).all()
    # quantizing the dequantized values again changes nothing
    c2, s2 = F.mxfp8_quant(back)
    assert np.array_equal(F.mxfp8_dequant(c2, s2), back)


def test_largest_and_smallest_inputs_saturate_and_flush():
    x = np.zeros((1, 64), np.float32)
    x[0, 0] = np.float32(3.0e38)
    x[0, 1] = np.float32(1.0)             # 1 / 2^119 underflows e4m3: becomes zero
    x[0, 32] = np.float32(1.0e-45)        # denormal absmax: exponent byte clamps at 0
    codes, scales = F.mxfp8_quant(x)
    assert scales[0, 0] == 127 + 127 - 8 and scales[0, 1] == 0
    back = F.mxfp8_dequant(codes, scales)
    assert np.isfinite(back).all() and back[0, 1] == 0.0
