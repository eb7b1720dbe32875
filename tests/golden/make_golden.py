"""Generate tests/golden/reference_vectors.npz.

Runs ONLY where the reference checkout is present (path given by --reference):
it imports the reference's own Python converter (scripts/convert_fp8_to_gguf.py)
to produce Q4_K block bytes and an FP8 128x128 block dequantization from seeded
inputs, and uses gguf-py (the GGML format's own Python package) for the Q8_0 /
Q4_K dequantized values.  The committed .npz is what the tests read; this script
is kept so the vectors can be regenerated.

    python tests/golden/make_golden.py --reference /path/to/hanzo-engine
"""
import argparse
import importlib.util
import os
import sys

import numpy as np


def load_reference_converter(ref_root):
    path = os.path.join(ref_root, "scripts", "convert_fp8_to_gguf.py")
    spec = importlib.util.spec_from_file_location("ref_convert_fp8_to_gguf", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--out", default=os.path.join(os.path.dirname(__file__), "reference_vectors.npz"))
    args = ap.parse_args()

    import gguf
    import torch
    from gguf import quants

    ref = load_reference_converter(args.reference)
    rng = np.random.default_rng(20240601)

    # Q4_K: weights N(0, 0.02^2) plus rows with awkward content (zeros, constant, large range)
    w4 = rng.normal(0.0, 0.02, (6, 512)).astype(np.float32)
    w4[3, :256] = 0.0
    w4[4, :] = 0.0125
    w4[5, :] *= np.linspace(0.01, 40.0, 512, dtype=np.float32)
    q4_bytes = ref.quantize_q4_k(w4)
    q4_deq = quants.dequantize(q4_bytes, gguf.GGMLQuantizationType.Q4_K).astype(np.float32)

    # Q8_0 through gguf-py
    w8 = rng.normal(0.0, 0.02, (5, 256)).astype(np.float32)
    w8[2, :64] = 0.0
    q8_bytes = quants.quantize(w8, gguf.GGMLQuantizationType.Q8_0)
    q8_deq = quants.dequantize(q8_bytes, gguf.GGMLQuantizationType.Q8_0).astype(np.float32)

    # FP8 e4m3 with a 128x128 scale grid through the reference converter's dequantizer
    codes = rng.integers(0, 256, (130, 260), dtype=np.uint8)
    codes[(codes & 0x7F) == 0x7F] = 0x3C          # no NaN codes
    scale = rng.uniform(1e-4, 3e-3, (2, 3)).astype(np.float32)
    wt = torch.from_numpy(codes).view(torch.float8_e4m3fn)
    fp8_deq = ref._dequant_fp8_block(wt, torch.from_numpy(scale)).astype(np.float32)

    # every e4m3 code decoded by torch (pins the decode table)
    all_codes = np.arange(256, dtype=np.uint8)
    e4m3_all = torch.from_numpy(all_codes).view(torch.float8_e4m3fn).to(torch.float32).numpy()

    np.savez_compressed(args.out, w4=w4, q4_bytes=q4_bytes, q4_deq=q4_deq,
                        w8=w8, q8_bytes=q8_bytes, q8_deq=q8_deq,
                        fp8_codes=codes, fp8_scale=scale, fp8_deq=fp8_deq, e4m3_all=e4m3_all)
    print("wrote", args.out, os.path.getsize(args.out), "bytes")


if __name__ == "__main__":
    main()
