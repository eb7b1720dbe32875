"""Synthetic layers at the benchmark configurations, built on the device (stand-ins for model checkpoints:
weights N(0, 0.02^2) quantized to the layer's format, seeded), and the CPU oracle of a token subset of such a
layer.  Shared by bench.py, the full-size parity tests and the smoke run.  The byte formats produced here are the
ones tests/ pins against the oracle; the oracle side of this file is test infrastructure."""
from __future__ import annotations

import numpy as np

MOE_CFGS = {
    # benchmark configurations 3-5: Qwen3-30B-A3B Q4_K, DeepSeek-V3 block-FP8, gpt-oss-120b MXFP4 layer shapes
    "moe_q4k": dict(fmt="Q4_K", e=128, k=8, h=2048, i=768, t=4096, router="softmax", inter=False,
                    label="cfg3_qwen3_30b_a3b_q4k_moe"),
    "moe_fp8": dict(fmt="FP8", e=256, k=8, h=7168, i=2048, t=4096, router="sigmoid_bias", inter=False,
                    shared=True, act_fp8=True, label="cfg4_deepseek_v3_block_fp8_moe"),
    "moe_mxfp4": dict(fmt="MXFP4", e=128, k=4, h=2880, i=2880, t=8192, router="topk_softmax", inter=True,
                      act_mx=True, label="cfg5_gpt_oss_120b_mxfp4_moe"),
}


def q8_0_matrix(torch, n, k, gen, device):
    """N(0, 0.02^2) weights quantized to GGUF Q8_0 blocks on the device: d = absmax/127 (fp16), q = round(x/d)."""
    out = torch.empty((n, k // 32, 34), dtype=torch.uint8, device=device)
    rows_per = max(1, (1 << 26) // k)
    for r0 in range(0, n, rows_per):
        r1 = min(n, r0 + rows_per)
        w = torch.randn((r1 - r0, k // 32, 32), generator=gen, device=device, dtype=torch.float32) * 0.02
        d = w.abs().amax(dim=2, keepdim=True) / 127.0
        q = torch.round(w / torch.where(d > 0, d, torch.ones_like(d))).clamp(-127, 127).to(torch.int8)
        out[r0:r1, :, 0:2] = d.to(torch.float16).view(torch.uint8).reshape(r1 - r0, k // 32, 2)
        out[r0:r1, :, 2:] = q.view(torch.uint8)
    return out.reshape(n, -1)


def q4k_bank(torch, e, n, k, gen, dev):
    """N(0, 0.02^2) weights -> GGUF Q4_K super-blocks with a plain min/max quantizer, one expert at a time: per
    32-element sub-block scale = (max - min)/15 and min <= 0, both coded in 6 bits against the super-block's
    d / dmin."""
    out = torch.empty((e, n, k // 256, 144), dtype=torch.uint8, device=dev)
    for ex in range(e):
        w = torch.randn((n, k // 256, 8, 32), generator=gen, device=dev) * 0.02
        mn = torch.clamp(w.amin(dim=3), max=0.0)
        sc = (w.amax(dim=3) - mn) / 15.0
        d = (sc.amax(dim=2, keepdim=True) / 63.0).to(torch.float16)
        dmin = ((-mn).amax(dim=2, keepdim=True) / 63.0).to(torch.float16)
        df, dmf = d.float().clamp_min(1e-12), dmin.float().clamp_min(1e-12)
        ls = torch.clamp(torch.round(sc / df), 0, 63).to(torch.int32)
        lm = torch.clamp(torch.round(-mn / dmf), 0, 63).to(torch.int32)
        d1 = (d.float() * ls).unsqueeze(-1)
        m1 = (dmin.float() * lm).unsqueeze(-1)
        q = torch.clamp(torch.round((w + m1) / d1.clamp_min(1e-12)), 0, 15).to(torch.uint8)
        blk = out[ex]
        blk[:, :, 0:2] = d.view(torch.uint8).reshape(n, k // 256, 2)
        blk[:, :, 2:4] = dmin.view(torch.uint8).reshape(n, k // 256, 2)
        sb = torch.zeros((n, k // 256, 12), dtype=torch.int32, device=dev)
        sb[:, :, 0:4] = ls[:, :, 0:4] | ((ls[:, :, 4:8] >> 4) << 6)
        sb[:, :, 4:8] = lm[:, :, 0:4] | ((lm[:, :, 4:8] >> 4) << 6)
        sb[:, :, 8:12] = (ls[:, :, 4:8] & 0xF) | ((lm[:, :, 4:8] & 0xF) << 4)
        blk[:, :, 4:16] = sb.to(torch.uint8)
        blk[:, :, 16:] = (q[:, :, 0::2, :] | (q[:, :, 1::2, :] << 4)).reshape(n, k // 256, 128)
    return out.reshape(e, n, -1)


def fp8_bank(torch, e, n, k, gen, dev):
    codes = torch.empty((e, n, k), dtype=torch.uint8, device=dev)
    scales = torch.empty((e, n // 128, k // 128), dtype=torch.float32, device=dev)
    for ex in range(e):
        w = (torch.randn((n // 128, 128, k // 128, 128), generator=gen, device=dev) * 0.02)
        s = w.abs().amax(dim=(1, 3)) / 448.0
        q = (w / s[:, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn)
        codes[ex] = q.view(torch.uint8).reshape(n, k)
        scales[ex] = s
    return codes, scales


def mxfp4_bank(torch, e, n, k, gen, dev):
    blocks = torch.empty((e, n, k // 2), dtype=torch.uint8, device=dev)
    scales = torch.empty((e, n, k // 32), dtype=torch.uint8, device=dev)
    for ex in range(e):
        w = torch.randn((n, k // 32, 32), generator=gen, device=dev) * 0.02
        amax = w.abs().amax(dim=2)
        ee = torch.clamp(torch.floor(torch.log2(amax / 6.0)) + 127, 0, 254)
        ee = torch.where(amax == 0, torch.full_like(ee, 127), ee)
        v = (w / torch.exp2(ee - 127).unsqueeze(-1)).abs()
        nib = ((v >= 0.25).int() + (v >= 0.75).int() + (v >= 1.25).int() + (v >= 1.75).int() + (v >= 2.5).int() +
               (v >= 3.5).int() + (v >= 5.0).int())
        nib = (nib | ((w < 0).int() << 3)).to(torch.uint8).reshape(n, k)
        blocks[ex] = nib[:, 0::2] | (nib[:, 1::2] << 4)
        scales[ex] = ee.to(torch.uint8)
    return blocks, scales


def build_moe_layer(torch, hq, cfg, gen, dev, e_local=None):
    """Banks for `e_local` experts of the layer (all experts when None)."""
    from engine_b200 import _lib as L
    e = e_local or cfg["e"]
    h, i, fmt = cfg["h"], cfg["i"], cfg["fmt"]

    def bank(n, k, bias):
        b = (torch.randn((e, n), generator=gen, device=dev) * 0.02).to(torch.bfloat16) if bias else None
        if fmt == "Q4_K":
            return hq.GgufMatMul(q4k_bank(torch, e, n, k, gen, dev), "Q4_K", k, b)
        if fmt == "FP8":
            c, s = fp8_bank(torch, e, n, k, gen, dev)
            return hq.BlockwiseFP8Linear(c, s, b)
        bl, sc = mxfp4_bank(torch, e, n, k, gen, dev)
        return hq.MXFP4Layer(bl, sc, b)

    down = bank(h, i, cfg["inter"])
    if cfg["inter"]:
        return hq.MoEExperts(down, gate_up_proj=bank(2 * i, h, True), act=L.ACT_GPTOSS, limit=7.0, alpha=1.702)
    return hq.MoEExperts(down, bank(i, h, False), bank(i, h, False), act=L.ACT_SWIGLU)


def router_config(hq, cfg):
    from engine_b200 import _lib as L
    if cfg["router"] == "softmax":
        return hq.MoeRouterTopKConfig(cfg["k"], L.SCORE_SOFTMAX, L.WEIGHT_SCORE, True)
    if cfg["router"] == "sigmoid_bias":
        return hq.MoeRouterTopKConfig(cfg["k"], L.SCORE_SIGMOID, L.WEIGHT_SCORE, True, 1e-20, 2.5)
    return hq.MoeRouterTopKConfig(cfg["k"], L.SCORE_RAW, L.WEIGHT_SOFTMAX, False)


def oracle_router(cfg, logits: np.ndarray, sel_bias: np.ndarray | None):
    from oracle import moe as M
    if cfg["router"] == "softmax":
        return M.router_topk(logits, cfg["k"], M.SCORE_SOFTMAX, M.WEIGHT_SCORE, True)
    if cfg["router"] == "sigmoid_bias":
        return M.router_topk(logits, cfg["k"], M.SCORE_SIGMOID, M.WEIGHT_SCORE, True, 1e-20, 2.5,
                             selection_bias=sel_bias)
    return M.router_topk(logits, cfg["k"], M.SCORE_RAW, M.WEIGHT_SOFTMAX, False)


# ---- CPU oracle of a token subset ---------------------------------------------------------------------
_FMT_NAME = {0: "Q8_0", 1: "Q4_K", 2: "FP8", 3: "MXFP4", 4: "Q6_K", 5: "Q5_K", 6: "Q4_0", 7: "Q5_0", 8: "Q4_1", 9: "Q5_1",
             10: "Q2_K", 11: "Q3_K"}


def _bank_slices(layer, experts):
    """Host copies of the listed experts of a quantized bank: (fmt name, bytes [n_e, N, row_bytes], scales, bias)."""
    import torch
    idx = torch.as_tensor(experts, dtype=torch.long, device=layer._device())
    fmt = _FMT_NAME[layer.format]
    bias = None if getattr(layer, "bias", None) is None else \
        layer.bias.index_select(0, idx).to(torch.float32).cpu().numpy()
    if fmt in ("Q8_0", "Q4_K"):
        return fmt, layer.data.index_select(0, idx).cpu().numpy(), None, bias
    if fmt == "FP8":
        return fmt, layer.weight.index_select(0, idx).cpu().numpy(), layer.scale.index_select(0, idx).cpu().numpy(), bias
    return fmt, layer.blocks.index_select(0, idx).cpu().numpy(), layer.scales.index_select(0, idx).cpu().numpy(), bias


def oracle_moe_host(first_banks, down_bank, n_used, act, x_sub, ids_c, w_sub, *, fp8_act=False, threads=0):
    """Expert block on host copies of `n_used` experts.  first_banks: [(fmt, bytes [n_used, N, row_bytes], scales,
    bias)] -- one interleaved gate/up bank, or the gate and the up bank; ids_c [S, k] index into the copies (-1 =
    skipped slot); act = (code, has_limit, limit, alpha).  Rounding points mirror the CUDA path: the 16-bit path
    rounds the activated intermediate to f16; the FP8-activation path quantizes x 1x128, rounds gate and up to f16,
    rounds the activated product to f16 and quantizes it 1x128; fp8_act="mx" is the MXFP8 path: x quantized per 32
    elements with a power-of-two scale, gate / up / product kept in f32, product quantized the same way.
    Returns f32 [S, H]."""
    from oracle import cbuild, formats as F, moe as M
    s, k = ids_c.shape
    f16 = lambda a: a.astype(np.float16).astype(np.float32)
    qdq = lambda a: F.fp8_vector_dequant(*F.fp8_vector_quant(np.ascontiguousarray(a).reshape(-1), 128), 128) \
        .reshape(a.shape).astype(np.float32)
    mx = fp8_act == "mx"
    if mx:
        f16 = lambda a: a
        qdq = lambda a: F.mxfp8_dequant(*F.mxfp8_quant(np.ascontiguousarray(a, dtype=np.float32))).astype(np.float32)
    # stable (token, slot) order grouped by expert
    flat = [(int(ids_c[t, sl]), t * k + sl) for t in range(s) for sl in range(k) if ids_c[t, sl] >= 0]
    flat.sort(key=lambda p: p[0])
    bounds = np.zeros(n_used + 1, np.int32)
    for e_c, _ in flat:
        bounds[e_c + 1] += 1
    bounds = np.cumsum(bounds).astype(np.int32)
    assign = np.array([a for _, a in flat], np.int32)
    tok = assign // k
    rows = np.arange(assign.size, dtype=np.int32)
    x_in = qdq(x_sub) if fp8_act else x_sub.astype(np.float32)
    outs = [cbuild.gather(fmt, data, scales, bias, x_in, n_used, bounds, tok, rows, assign.size, threads)
            for fmt, data, scales, bias in first_banks]
    if len(first_banks) == 1:
        g, u = outs[0][:, 0::2], outs[0][:, 1::2]
    else:
        g, u = outs
    if fp8_act:
        g, u = f16(g), f16(u)
    code, has_limit, limit, alpha = act
    if code == M.ACT_GPTOSS:
        hmid = M.gptoss_swiglu(g, u, alpha, limit)
    else:
        hmid = M.swiglu(g, u, limit if has_limit else None)
    hmid = qdq(f16(hmid.astype(np.float32))) if fp8_act else f16(hmid)
    fmt, data, scales, bias = down_bank
    y = cbuild.gather(fmt, data, scales, bias, hmid, n_used, bounds, rows, rows, assign.size, threads)
    out = np.zeros((s, y.shape[1]), np.float32)
    order = np.argsort(assign, kind="stable")            # add a token's slots in slot order, as the reduce does
    for pos in order:
        a = int(assign[pos])
        out[a // k] += np.float32(w_sub[a // k, a % k]) * y[pos]
    return out


def oracle_moe_subset(experts, x_sub: np.ndarray, ids_sub: np.ndarray, w_sub: np.ndarray, *, fp8_act=False,
                      threads=0, timer=None):
    """The expert block of `experts` (an engine_b200.MoEExperts living on the GPU) for the token rows x_sub
    [S, H] with routing ids_sub / w_sub [S, k], computed by the C oracle (dequantize each expert row to f32, f32
    dot) from host copies of the experts those tokens touch.  `timer`, if given, is called with the seconds spent
    in the oracle's arithmetic (bank copies excluded)."""
    import time
    used = sorted(set(int(v) for v in ids_sub.reshape(-1) if 0 <= int(v) < experts.n_experts))
    remap = {e: j for j, e in enumerate(used)}
    ids_c = np.array([[remap.get(int(v), -1) for v in row] for row in ids_sub], dtype=np.int64)
    interleaved = experts.gate_up is not None
    first = [_bank_slices(experts.gate_up, used)] if interleaved else \
        [_bank_slices(experts.gate, used), _bank_slices(experts.up, used)]
    down = _bank_slices(experts.down, used)
    act = (experts.act.act, experts.act.has_limit, experts.act.limit, experts.act.alpha)
    t0 = time.perf_counter()
    out = oracle_moe_host(first, down, len(used), act, x_sub, ids_c, w_sub, fp8_act=fp8_act, threads=threads)
    if timer is not None:
        timer(time.perf_counter() - t0)
    return out
