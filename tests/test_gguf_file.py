"""GGUF reader on a file written by gguf-py's own writer: directory, metadata and the raw block bytes of dense
matrices and expert banks come back byte for byte (no GPU needed)."""
import os

import numpy as np
import pytest

gguf = pytest.importorskip("gguf")

from oracle import formats as F


def _write(path, tensors, kv):
    w = gguf.GGUFWriter(path, "llama")
    for k, v in kv.items():
        if isinstance(v, str):
            w.add_string(k, v)
        else:
            w.add_uint32(k, v)
    for name, (raw, qtype) in tensors.items():
        if qtype is None:
            w.add_tensor(name, raw)
        else:
            w.add_tensor(name, raw, raw_dtype=qtype)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


def test_reader_returns_the_file_s_block_bytes(tmp_path):
    from engine_b200.gguf_file import GgufFile
    rng = np.random.Generator(np.random.PCG64(12))
    e, n, k = 3, 8, 512
    w = rng.normal(0, 0.02, (e * n, k)).astype(np.float32)
    q4 = F.q4_k_quantize(w).reshape(e, n, -1)
    q8 = F.q8_0_quantize(w[:n]).reshape(n, -1)
    bias = rng.standard_normal(n).astype(np.float32)
    path = os.path.join(tmp_path, "t.gguf")
    _write(path, {"blk.0.ffn_gate_exps.weight": (q4, gguf.GGMLQuantizationType.Q4_K),
                  "blk.0.attn_q.weight": (q8, gguf.GGMLQuantizationType.Q8_0),
                  "blk.0.attn_q.bias": (bias, None)},
           {"general.name": "tiny", "llama.expert_count": e})
    f = GgufFile(path)
    assert f.metadata["general.name"] == "tiny" and f.metadata["llama.expert_count"] == e
    t = f.tensors["blk.0.ffn_gate_exps.weight"]
    assert t.shape == (e, n, k) and t.type_name == "Q4_K" and t.row_bytes == k // 256 * 144
    assert np.array_equal(f.raw("blk.0.ffn_gate_exps.weight"), q4)
    assert np.array_equal(f.raw("blk.0.attn_q.weight"), q8)
    assert f.tensors["blk.0.attn_q.weight"].shape == (n, k)
    # the bytes dequantize to what was quantized, through the oracle
    np.testing.assert_array_equal(F.q4_k_dequant(f.raw("blk.0.ffn_gate_exps.weight").reshape(e * n, -1), k),
                                  F.q4_k_dequant(q4.reshape(e * n, -1), k))
    f.close()


def test_reader_rejects_what_it_does_not_know(tmp_path):
    from engine_b200.gguf_file import GgufError, GgufFile
    path = os.path.join(tmp_path, "bad.gguf")
    with open(path, "wb") as fh:
        fh.write(b"NOPE" + b"\0" * 64)
    with pytest.raises(GgufError):
        GgufFile(path)


def test_reader_knows_every_ggml_type_the_kernels_run(tmp_path):
    """One tensor of each type of the reference's decode list (hanzo-quant/src/gguf/fast_mmvq.rs:36-50), written by
    gguf-py: type name, block geometry and bytes come back, and the bytes dequantize (oracle) to what gguf-py says."""
    from engine_b200.gguf_file import GgufFile
    from gguf import quants
    rng = np.random.Generator(np.random.PCG64(13))
    n, k = 4, 512
    tensors, raws = {}, {}
    for name in ["Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q2_K", "Q3_K", "Q5_K", "Q6_K"]:
        raws[name] = F.ggml_random_blocks(name, rng, n, k)
        tensors[f"t.{name}.weight"] = (raws[name], getattr(gguf.GGMLQuantizationType, name))
    path = os.path.join(tmp_path, "types.gguf")
    _write(path, tensors, {"general.name": "types"})
    f = GgufFile(path)
    for name, raw in raws.items():
        t = f.tensors[f"t.{name}.weight"]
        assert t.type_name == name and t.shape == (n, k) and t.row_bytes == raw.shape[1]
        got = np.array(f.raw(f"t.{name}.weight"))                 # a copy: views keep the file mapped
        assert np.array_equal(got, raw)
        want = quants.dequantize(raw, getattr(gguf.GGMLQuantizationType, name)).astype(np.float32)
        assert np.array_equal(F.GGML_DEQUANT[name](got, k), want)
    f.close()
