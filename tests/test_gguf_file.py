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
