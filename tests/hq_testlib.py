"""Seeded synthetic inputs shared by the GPU parity tests, the smoke run and the benchmark's checks.
Weights N(0, 0.02^2) quantized by the oracle; activations N(0, 1)."""
import numpy as np

from oracle import formats as F


def rng_for(cfg: int, index: int = 0):
    return np.random.Generator(np.random.PCG64(1000 * cfg + index))


def rel_l2(got: np.ndarray, want: np.ndarray) -> float:
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    den = np.linalg.norm(want)
    return float(np.linalg.norm(got - want) / (den if den > 0 else 1.0))


def make_weight(fmt: str, rng, n: int, k: int, experts: int = 0, sigma: float = 0.02):
    """Returns (arrays for the layer constructor, dequantized f32 [E?, N, K])."""
    e = max(experts, 1)
    w = rng.normal(0.0, sigma, (e * n, k)).astype(np.float32)
    if fmt == "Q8_0":
        raw = F.q8_0_quantize(w)
        deq = F.q8_0_dequant(raw, k)
        arrays = {"data": raw.reshape(e, n, -1)}
    elif fmt == "Q4_K":
        raw = F.q4_k_quantize(w)
        deq = F.q4_k_dequant(raw, k)
        arrays = {"data": raw.reshape(e, n, -1)}
    elif fmt == "Q6_K":
        raw = F.q6_k_quantize(w)
        deq = F.q6_k_dequant(raw, k)
        arrays = {"data": raw.reshape(e, n, -1)}
    elif fmt in ("Q5_K", "Q4_0", "Q5_0", "Q4_1", "Q5_1", "Q2_K", "Q3_K"):
        # no quantizer for these types: random valid blocks whose scales give weights of the usual magnitude
        lo, hi = {"Q5_K": (2e-5, 1e-4), "Q2_K": (5e-4, 2e-3), "Q3_K": (1e-4, 4e-4)}.get(fmt, (1e-3, 4e-3))
        raw = F.ggml_random_blocks(fmt, rng, e * n, k, lo, hi)
        deq = F.GGML_DEQUANT[fmt](raw, k)
        arrays = {"data": raw.reshape(e, n, -1)}
    elif fmt == "FP8":
        codes, scales, deqs = [], [], []
        for i in range(e):
            c, s = F.fp8_block_quant(w[i * n:(i + 1) * n])
            codes.append(c), scales.append(s), deqs.append(F.fp8_block_dequant(c, s))
        arrays = {"weight": np.stack(codes), "scale": np.stack(scales)}
        deq = np.concatenate(deqs)
    elif fmt == "MXFP4":
        b, s = F.mxfp4_quantize(w)
        deq = F.mxfp4_dequant(b, s)
        arrays = {"blocks": b.reshape(e, n, -1), "scales": s.reshape(e, n, -1)}
    else:
        raise ValueError(fmt)
    deq = deq.reshape(e, n, k)
    if experts == 0:
        arrays = {k_: v[0] for k_, v in arrays.items()}
        deq = deq[0]
    return arrays, deq


def make_layer(fmt: str, arrays: dict, k: int, device, bias=None):
    import torch
    import engine_b200 as hq
    t = {k_: torch.from_numpy(np.ascontiguousarray(v)).to(device) for k_, v in arrays.items()}
    if fmt in F.GGML_DEQUANT:
        return hq.GgufMatMul(t["data"], fmt, k, bias)
    if fmt == "FP8":
        return hq.BlockwiseFP8Linear(t["weight"], t["scale"], bias)
    return hq.MXFP4Layer(t["blocks"], t["scales"], bias)


def to_dev(x: np.ndarray, dtype, device):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).to(device).to(dtype)
