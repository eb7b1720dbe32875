"""CPU oracle: router, permutation, gated activations, gather/MoE math.

TEST INFRASTRUCTURE ONLY (see oracle/formats.py).  numpy restatement of the
reference's CPU semantics for the sparse-MoE path; each function cites the
reference file:line it follows.
"""
from __future__ import annotations

import numpy as np

# integer codes that cross the C boundary (hanzo-engine/src/ops.rs:194-222)
SCORE_RAW, SCORE_SOFTMAX, SCORE_SIGMOID = 0, 1, 2
WEIGHT_SCORE, WEIGHT_SOFTMAX, WEIGHT_SIGMOID = 0, 1, 2
# gated-activation codes of the new ABI
ACT_NONE, ACT_SWIGLU, ACT_GPTOSS = 0, 1, 2


def _softmax_rows(x: np.ndarray) -> np.ndarray:
    x = x.astype(np.float32)
    m = x.max(axis=-1, keepdims=True)
    e = np.exp((x - m).astype(np.float32)).astype(np.float32)
    return (e / e.sum(axis=-1, keepdims=True, dtype=np.float32)).astype(np.float32)


def _sigmoid(x: np.ndarray) -> np.ndarray:
    x = x.astype(np.float32)
    return (np.float32(1.0) / (np.float32(1.0) + np.exp(-x).astype(np.float32))).astype(np.float32)


def deterministic_topk_indices(scores: np.ndarray, k: int) -> np.ndarray:
    """Canonical selection: order each row by (score DESC, expert id ASC), take k
    (hanzo-engine/src/ops.rs:241-251).  NaN scores are treated as -inf, as the
    reference's CUDA kernel does (hanzo-engine/src/cuda/sort.cu:1084-1086); its CPU
    fallback sorts with f32::total_cmp, which would put a positive NaN first -- the
    two reference paths disagree there and this restatement follows the GPU one."""
    s = np.where(np.isnan(scores), -np.inf, scores).astype(np.float32)
    # stable argsort on -score keeps lower ids first among equals
    order = np.argsort(-s, axis=-1, kind="stable")
    return order[:, :k].astype(np.uint32)


def router_topk(logits: np.ndarray, top_k: int, score_mode: int, weight_mode: int,
                renormalize: bool, norm_min: float = 0.0, output_scale: float = 1.0,
                selection_bias: np.ndarray | None = None, expert_scale: np.ndarray | None = None,
                clamp: tuple[float, float] | None = None):
    """logits f32 [T, E] -> (ids uint32 [T, k] in descending selection order,
    weights f32 [T, k]).  Follows `moe_router_topk`
    (hanzo-engine/src/ops.rs:253-335) with the canonical tie-break always on."""
    lg = np.asarray(logits, dtype=np.float32)
    if clamp is not None:
        lg = np.clip(lg, np.float32(clamp[0]), np.float32(clamp[1]))
    if score_mode == SCORE_RAW:
        sc = lg.copy()
    elif score_mode == SCORE_SOFTMAX:
        sc = _softmax_rows(lg)
    else:
        sc = _sigmoid(lg)
    sel = sc + selection_bias.astype(np.float32)[None, :] if selection_bias is not None else sc
    ids = deterministic_topk_indices(sel, top_k)
    if weight_mode == WEIGHT_SCORE:
        vals = np.take_along_axis(sc, ids.astype(np.int64), axis=1)
    elif weight_mode == WEIGHT_SOFTMAX:
        vals = _softmax_rows(np.take_along_axis(lg, ids.astype(np.int64), axis=1))
    else:
        vals = _sigmoid(np.take_along_axis(lg, ids.astype(np.int64), axis=1))
    vals = vals.astype(np.float32)
    if renormalize:
        den = vals.sum(axis=1, keepdims=True, dtype=np.float32)
        if norm_min > 0.0:
            den = np.maximum(den, np.float32(norm_min))
        vals = (vals / den).astype(np.float32)
    if output_scale != 1.0:
        vals = (vals * np.float32(output_scale)).astype(np.float32)
    if expert_scale is not None:
        vals = (vals * expert_scale.astype(np.float32)[ids.astype(np.int64)]).astype(np.float32)
    return ids, vals


def router_topk_grouped(logits: np.ndarray, top_k: int, score_mode: int, n_group: int, topk_group: int,
                        group_score: str = "top2_sum", selection_bias: np.ndarray | None = None,
                        renormalize: bool = True, norm_min: float = 1e-20, output_scale: float = 1.0):
    """DeepSeek group-limited routing (hanzo-engine/src/models/deepseek3.rs:623-690): scores -> + bias -> group
    score (sum of the two best of a group for "top2_sum" / noaux_tc, the best one for "max" /
    group_limited_greedy) -> keep the topk_group best groups, zero the selection score elsewhere -> top-k ->
    weights = unbiased scores of the selected experts, renormalised, scaled.  Ties by (score DESC, index ASC)."""
    lg = np.asarray(logits, dtype=np.float32)
    t, e = lg.shape
    sc = _softmax_rows(lg) if score_mode == SCORE_SOFTMAX else (_sigmoid(lg) if score_mode == SCORE_SIGMOID else lg.copy())
    sel = sc + selection_bias.astype(np.float32)[None, :] if selection_bias is not None else sc.copy()
    gs = e // n_group
    grouped = sel.reshape(t, n_group, gs)
    if group_score == "top2_sum":
        srt = -np.sort(-grouped, axis=-1)
        gsc = (srt[..., 0] + srt[..., 1]).astype(np.float32)
    else:
        gsc = grouped.max(axis=-1)
    gidx = deterministic_topk_indices(gsc, topk_group).astype(np.int64)
    mask = np.zeros((t, n_group), dtype=bool)
    np.put_along_axis(mask, gidx, True, axis=1)
    tmp = np.where(np.repeat(mask, gs, axis=1), sel, np.float32(0.0)).astype(np.float32)
    ids = deterministic_topk_indices(tmp, top_k)
    vals = np.take_along_axis(sc, ids.astype(np.int64), axis=1).astype(np.float32)
    if renormalize:
        den = vals.sum(axis=1, keepdims=True, dtype=np.float32)
        if norm_min > 0.0:
            den = np.maximum(den, np.float32(norm_min))
        vals = (vals / den).astype(np.float32)
    if output_scale != 1.0:
        vals = (vals * np.float32(output_scale)).astype(np.float32)
    return ids, vals


def stable_permutation(ids: np.ndarray, n_experts: int):
    """Stable counting sort of the flat assignment index t*k+s by expert id: the
    reference's only deterministic grouping (hanzo-quant/src/mxfp4/ops.rs:237-271,
    same order as hanzo-engine/src/moe/experts/backends.rs:913-927).
    Returns (expert_bounds int32 [E+1], sorted_assign int32 [T*k] = flat index,
    sorted_token int32 [T*k] = token index)."""
    t, k = ids.shape
    flat = ids.reshape(-1).astype(np.int64)
    order = np.argsort(flat, kind="stable")
    counts = np.bincount(flat, minlength=n_experts)
    bounds = np.zeros(n_experts + 1, np.int32)
    bounds[1:] = np.cumsum(counts)
    return bounds, order.astype(np.int32), (order // k).astype(np.int32)


def silu(x: np.ndarray) -> np.ndarray:
    """x / (1 + exp(-x)) (hanzo-quant/src/utils/ops.rs:2587-2589)."""
    x = x.astype(np.float32)
    return (x / (np.float32(1.0) + np.exp(-x).astype(np.float32))).astype(np.float32)


def swiglu(gate: np.ndarray, up: np.ndarray, limit: float | None = None) -> np.ndarray:
    """silu(gate) * up in f32, with the optional clamp gate<=L, |up|<=L applied
    first (hanzo-engine/src/ops.rs:3545-3556; f32 form of the grouped route,
    hanzo-quant/kernels/mmq_gguf/mmq_quantize.cu:229-260)."""
    g = gate.astype(np.float32)
    u = up.astype(np.float32)
    if limit is not None:
        g = np.minimum(g, np.float32(limit))
        u = np.clip(u, -np.float32(limit), np.float32(limit))
    return (silu(g) * u).astype(np.float32)


def gptoss_swiglu(gate: np.ndarray, up: np.ndarray, alpha: float = 1.702, limit: float = 7.0) -> np.ndarray:
    """(clamp(up, +-L) + 1) * g * sigmoid(alpha*g), g = min(gate, L)
    (hanzo-engine/src/models/gpt_oss.rs:116-135)."""
    g = np.minimum(gate.astype(np.float32), np.float32(limit))
    u = np.clip(up.astype(np.float32), -np.float32(limit), np.float32(limit))
    glu = g * _sigmoid(g * np.float32(alpha))
    return ((u + np.float32(1.0)) * glu).astype(np.float32)


def dense_forward(x: np.ndarray, w_f32: np.ndarray, bias: np.ndarray | None = None) -> np.ndarray:
    """y = x . W^T (+ b) with f64 accumulation: the dequantize-then-matmul
    result every quantized `forward` is graded against
    (hanzo-quant/src/gguf/mod.rs:196-209, mxfp4/mod.rs:550-626)."""
    y = x.astype(np.float64) @ w_f32.astype(np.float64).T
    if bias is not None:
        y = y + bias.astype(np.float64)[None, :]
    return y.astype(np.float32)


def gather_forward(x: np.ndarray, ids: np.ndarray, bank_f32: np.ndarray,
                   bias: np.ndarray | None = None) -> np.ndarray:
    """Per-assignment matvec out of an expert bank [E, N, K].

    x is [T, K] / [T, 1, K] (one row per token, shared by its k slots) or
    [T, k, K] (one row per slot); ids [T, k]; returns [T, k, N] f32
    (hanzo-quant/src/unquantized/mod.rs:182-277, mxfp4/mod.rs:630-726)."""
    t, k = ids.shape
    if x.ndim == 2:
        x = x[:, None, :]
    per_slot = x.shape[1] > 1
    n = bank_f32.shape[1]
    out = np.zeros((t, k, n), np.float32)
    flat = ids.reshape(-1).astype(np.int64)
    for e in np.unique(flat):
        sel = np.nonzero(flat == e)[0]
        tok, slot = sel // k, sel % k
        rows = x[tok, slot if per_slot else 0, :]
        y = rows.astype(np.float64) @ bank_f32[e].astype(np.float64).T
        if bias is not None:
            y = y + bias[e].astype(np.float64)[None, :]
        out[tok, slot, :] = y.astype(np.float32)
    return out


def weighted_combine(y: np.ndarray, w: np.ndarray) -> np.ndarray:
    """out[t, :] = sum_s w[t, s] * y[t, s, :] in f32
    (hanzo-engine/src/moe/experts/backends.rs:601-604)."""
    return (y.astype(np.float32) * w.astype(np.float32)[:, :, None]).sum(axis=1, dtype=np.float32)


def moe_layer(x: np.ndarray, ids: np.ndarray, weights: np.ndarray,
              gate_bank: np.ndarray | None, up_bank: np.ndarray | None, down_bank: np.ndarray,
              act: int = ACT_SWIGLU, gate_up_bank: np.ndarray | None = None,
              gate_up_bias: np.ndarray | None = None, down_bias: np.ndarray | None = None,
              alpha: float = 1.702, limit: float | None = None,
              h_round=None, gu_round=None) -> np.ndarray:
    """Whole expert block in f32: gather gate/up -> gated activation -> gather
    down -> weighted sum over slots.  Separate gate/up banks (Qwen3, DeepSeek:
    hanzo-engine/src/moe/experts/backends.rs:560-605) or one interleaved bank
    with rows [gate0, up0, gate1, up1, ...] (gpt-oss:
    hanzo-engine/src/models/gpt_oss.rs:405-440).  `h_round`, if given, is applied
    to the activated intermediate (the rounding point of a 16-bit pipeline);
    `gu_round` to the gate and up projections before the activation (a pipeline
    that stores them in 16 bits first)."""
    if gate_up_bank is not None:
        gu = gather_forward(x, ids, gate_up_bank, gate_up_bias)
        g, u = gu[..., 0::2], gu[..., 1::2]
    else:
        g = gather_forward(x, ids, gate_bank)
        u = gather_forward(x, ids, up_bank)
    if gu_round is not None:
        g, u = gu_round(g), gu_round(u)
    if act == ACT_GPTOSS:
        h = gptoss_swiglu(g, u, alpha, limit if limit is not None else 7.0)
    else:
        h = swiglu(g, u, limit)
    if h_round is not None:
        h = h_round(h)
    y = gather_forward(h, ids, down_bank, down_bias)
    return weighted_combine(y, weights)
