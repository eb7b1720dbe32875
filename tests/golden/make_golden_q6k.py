"""Generates tests/golden/q6k_vectors.npz: Q6_K block bytes and what gguf-py (the GGML format's own Python
package) dequantizes them to.  gguf-py has no Q6_K quantizer, so the bytes are random valid blocks (every bit
pattern of ql / qh / scales is valid) with a finite f16 d, plus blocks built by the oracle's plain quantizer
from N(0, 0.02^2) weights.  Run where gguf-py is installed:  python tests/golden/make_golden_q6k.py"""
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
    rand = rng.integers(0, 256, (4, k // 256, 210), dtype=np.uint8)
    rand[:, :, 208:210] = np.asarray(rng.uniform(1e-4, 3e-3, (4, k // 256, 1)), np.float16).view(np.uint8)
    rand = rand.reshape(4, -1)
    w = rng.normal(0.0, 0.02, (3, k)).astype(np.float32)
    w[1, :16] = 0.0
    made = F.q6_k_quantize(w)
    raw = np.concatenate([rand, made])
    deq = quants.dequantize(raw, gguf.GGMLQuantizationType.Q6_K).astype(np.float32)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "q6k_vectors.npz")
    np.savez_compressed(out, raw=raw, deq=deq, w=w)
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
