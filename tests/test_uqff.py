"""UQFF byte format (engine_b200/uqff.py) against byte strings assembled by hand from the layout the reference
documents (hanzo-quant/src/gguf/mod.rs:401-425, mxfp4/mod.rs:729-740, utils/uqff.rs:88-102), and round trips through the
layer classes (on CPU tensors: the device check of the constructors is switched off for the test)."""
import struct

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from engine_b200 import uqff
from oracle import formats as F

VERSION = (0 << 16) | (2 << 8) | 0


def _tensor_record(code, dims, payload):
    return struct.pack("<III", len(payload), code, len(dims)) + struct.pack(f"<{len(dims)}I", *dims) + payload


def test_gguf_layer_bytes_follow_the_documented_layout():
    rng = np.random.Generator(np.random.PCG64(1))
    raw = rng.integers(0, 256, (6, 288), dtype=np.uint8)              # Q4_K, K = 512: two 144-byte super-blocks a row
    bias = rng.standard_normal(6).astype(np.float32)
    got = uqff.serialize_gguf(torch.from_numpy(raw), "Q4_K", 512, torch.from_numpy(bias))
    want = (struct.pack("<I", VERSION) + bytes([0]) + struct.pack("<I", raw.size) + bytes([1]) +
            struct.pack("<I", 12) + struct.pack("<I", 2) + struct.pack("<II", 6, 512) + raw.tobytes() +
            _tensor_record(6, (6,), bias.tobytes()))
    assert got == want
    assert uqff.serde_type(got) == uqff.SERDE_GGUF
    r, qtype, k, b = uqff.deserialize_gguf(got)
    assert qtype == "Q4_K" and k == 512 and np.array_equal(r.numpy(), raw) and np.array_equal(b.numpy(), bias)
    # expert bank, no bias: three dims, the has_bias byte is 0 and nothing follows the payload
    bank = F.ggml_random_blocks("Q6_K", rng, 8, 256).reshape(2, 4, 210)
    got = uqff.serialize_gguf(torch.from_numpy(bank), "Q6_K", 256)
    assert got == (struct.pack("<IBIBII", VERSION, 0, bank.size, 0, 14, 3) + struct.pack("<III", 2, 4, 256) +
                   bank.tobytes())
    r, qtype, k, b = uqff.deserialize_gguf(got)
    assert r.shape == (2, 4, 210) and qtype == "Q6_K" and k == 256 and b is None


@pytest.mark.parametrize("qtype", sorted(uqff.GGML_TYPE_ID))
def test_every_ggml_type_of_the_path_round_trips(qtype):
    rng = np.random.Generator(np.random.PCG64(2))
    per, bb = uqff._GGML_BLOCK[qtype]
    raw = rng.integers(0, 256, (3, 512 // per * bb), dtype=np.uint8)
    r, t, k, b = uqff.deserialize_gguf(uqff.serialize_gguf(torch.from_numpy(raw), qtype, 512))
    assert t == qtype and k == 512 and b is None and np.array_equal(r.numpy(), raw)


def test_mxfp4_layer_bytes_follow_the_documented_layout():
    rng = np.random.Generator(np.random.PCG64(3))
    blocks = rng.integers(0, 256, (2, 4, 32), dtype=np.uint8)         # E = 2, N = 4, K = 64
    scales = rng.integers(100, 140, (2, 4, 2), dtype=np.uint8)
    bias = torch.from_numpy(rng.standard_normal((2, 4)).astype(np.float32)).to(torch.bfloat16)
    got = uqff.serialize_mxfp4(torch.from_numpy(blocks), torch.from_numpy(scales), bias)
    want = (struct.pack("<IBB", VERSION, 6, 1) + _tensor_record(0, (2, 4, 32), blocks.tobytes()) +
            _tensor_record(0, (2, 4, 2), scales.tobytes()) +
            _tensor_record(5, (2, 4), bias.view(torch.uint8).numpy().tobytes()))
    assert got == want
    b, s, bi = uqff.deserialize_mxfp4(got)
    assert np.array_equal(b.numpy(), blocks) and np.array_equal(s.numpy(), scales) and torch.equal(bi, bias)


def test_version_and_type_checks():
    ok = uqff.serialize_mxfp4(torch.zeros((1, 16), dtype=torch.uint8), torch.zeros((1, 1), dtype=torch.uint8))
    uqff.deserialize_mxfp4(ok)
    older_minor = struct.pack("<I", (0 << 16) | (1 << 8) | 7) + ok[4:]
    uqff.deserialize_mxfp4(older_minor)                                # same major, older minor: accepted
    for bad in [struct.pack("<I", (1 << 16)) + ok[4:], struct.pack("<I", (0 << 16) | (3 << 8)) + ok[4:]]:
        with pytest.raises(uqff.UqffError):
            uqff.deserialize_mxfp4(bad)
    with pytest.raises(uqff.UqffError):
        uqff.deserialize_gguf(ok)                                      # an MXFP4 artifact is not a GGUF layer
    with pytest.raises(uqff.UqffError):
        uqff.deserialize_mxfp4(ok[:-3])                                # truncated
    bad_type = bytearray(uqff.serialize_gguf(torch.zeros((1, 34 * 8), dtype=torch.uint8), "Q8_0", 256))
    bad_type[10:14] = struct.pack("<I", 16)                            # IQ2_XXS: not a type of this path
    with pytest.raises(uqff.UqffError):
        uqff.deserialize_gguf(bytes(bad_type))


def test_layers_serialise_like_the_reference_trait(monkeypatch):
    from engine_b200 import quant
    monkeypatch.setattr(quant, "_require_cuda", lambda *a, **k: None)
    rng = np.random.Generator(np.random.PCG64(4))
    raw = torch.from_numpy(F.ggml_random_blocks("Q5_K", rng, 4, 256))
    bias = torch.from_numpy(rng.standard_normal(4).astype(np.float32))
    layer = quant.GgufMatMul(raw, "Q5_K", 256, bias)
    assert layer.isq_serde_supported() and layer.name() == "gguf"
    data = layer.serialize()
    back, ext = quant.GgufMatMul.deserialize_ext_bias(data, "cpu")
    assert back.qtype == "Q5_K" and back.n == 4 and back.k == 256 and torch.equal(back.data, raw)
    assert torch.equal(back.bias, bias) and torch.equal(ext, bias)
    assert layer.serialize_with_bias(None) == uqff.serialize_gguf(raw, "Q5_K", 256)
    blocks = torch.from_numpy(rng.integers(0, 256, (3, 8, 32), dtype=np.uint8))
    scales = torch.from_numpy(rng.integers(110, 130, (3, 8, 2), dtype=np.uint8))
    mx = quant.MXFP4Layer(blocks, scales)
    assert mx.isq_serde_supported() and mx.name() == "mxfp4-layer"
    again = quant.MXFP4Layer.deserialize(mx.serialize(), "cpu")
    assert torch.equal(again.blocks, blocks) and torch.equal(again.scales, scales) and again.bias is None
    # the reference does not serialise block-FP8 layers (blockwise_fp8/mod.rs:401-408)
    assert quant.BlockwiseFP8Linear.isq_serde_supported(object.__new__(quant.BlockwiseFP8Linear)) is False
