"""Generates tests/golden/ggml_vectors.npz: block bytes of the GGML types Q6_K, Q5_K, Q4_0, Q5_0, Q4_1, Q5_1, Q2_K and
Q3_K and what gguf-py (the GGML format's own Python package) dequantizes them to.  The bytes are random valid blocks
(every bit pattern of these types is valid) with finite f16 scale fields; for Q6_K blocks built by the oracle's plain
quantizer from N(0, 0.02^2) weights are added, for Q4_0 / Q5_0 / Q4_1 / Q5_1 blocks that gguf-py itself quantized.
Run where gguf-py is installed:  python tests/golden/make_golden_ggml.py"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    import gguf
    from gguf import quants
    from oracle import formats as F
    rng = np.random.default_rng(20240602)
    k = 512
    types = {"Q6_K": gguf.GGMLQuantizationType.Q6_K, "Q5_K": gguf.GGMLQuantizationType.Q5_K,
             "Q4_0": gguf.GGMLQuantizationType.Q4_0, "Q5_0": gguf.GGMLQuantizationType.Q5_0,
             "Q4_1": gguf.GGMLQuantizationType.Q4_1, "Q5_1": gguf.GGMLQuantizationType.Q5_1,
             "Q2_K": gguf.GGMLQuantizationType.Q2_K, "Q3_K": gguf.GGMLQuantizationType.Q3_K}
    out = {}
    w = rng.normal(0.0, 0.02, (3, k)).astype(np.float32)
    w[1, :16] = 0.0
    out["w"] = w
    for name, t in types.items():
        raw = F.ggml_random_blocks(name, rng, 4, k)
        if name == "Q6_K":
            raw = np.concatenate([raw, F.q6_k_quantize(w)])
        elif name in ("Q4_0", "Q5_0", "Q4_1", "Q5_1"):
            raw = np.concatenate([raw, quants.quantize(w, t)])
        out["raw_" + name] = raw
        out["deq_" + name] = quants.dequantize(raw, t).astype(np.float32)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ggml_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
