"""Router, dispatch tables, gather_forward and the whole expert block against the oracle, through the C ABI.
Routing indices and the permutation are compared bit-exactly; outputs by rel-L2 (GGUF 1e-3, FP8/MXFP4 2e-3)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

import engine_b200 as hq
from engine_b200 import _lib as L
from oracle import formats as F
from oracle import moe as M
from tests import hq_testlib as T

DEV = "cuda:0"
TOL = {"Q8_0": 1e-3, "Q4_K": 1e-3, "Q6_K": 1e-3, "Q5_K": 1e-3, "Q4_0": 1e-3, "Q5_0": 1e-3, "Q4_1": 1e-3, "Q5_1": 1e-3,
       "Q2_K": 1e-3, "Q3_K": 1e-3, "FP8": 2e-3, "MXFP4": 2e-3}


def margin_ok_rows(sel: np.ndarray, k: int, ulps: int = 4):
    """Rows whose k-th and (k+1)-th selection scores differ by more than a few ulp: only those can be required
    to match when the two sides evaluate exp() with different last-bit rounding."""
    s = -np.sort(-sel, axis=1)
    gap = s[:, k - 1] - s[:, k] if sel.shape[1] > k else np.full(sel.shape[0], np.inf)
    inner = np.min(s[:, :k - 1] - s[:, 1:k], axis=1) if k > 1 else np.full(sel.shape[0], np.inf)
    eps = np.spacing(np.abs(s[:, 0]).astype(np.float32)) * ulps
    return (gap > eps) & (inner > eps)


ROUTER_CASES = [
    # (E, k, score, weight, renorm, norm_min, scale, bias)
    (128, 8, L.SCORE_SOFTMAX, L.WEIGHT_SCORE, True, 0.0, 1.0, False),      # Qwen3-style
    (256, 8, L.SCORE_SIGMOID, L.WEIGHT_SCORE, True, 1e-20, 2.5, True),     # DeepSeek-V3-style
    (128, 4, L.SCORE_RAW, L.WEIGHT_SOFTMAX, False, 0.0, 1.0, False),       # gpt-oss-style
    (60, 6, L.SCORE_SOFTMAX, L.WEIGHT_SIGMOID, False, 0.0, 1.0, False),    # E not a multiple of 32
    (5, 2, L.SCORE_RAW, L.WEIGHT_SCORE, False, 0.0, 1.0, False),
]


@pytest.mark.parametrize("case", ROUTER_CASES)
def test_router_matches_oracle(case):
    e, k, score, weight, renorm, nmin, scale, has_bias = case
    rng = T.rng_for(3, e + k)
    logits = rng.standard_normal((777, e)).astype(np.float32)
    bias = rng.normal(0, 0.01, e).astype(np.float32) if has_bias else None
    cfg = hq.MoeRouterTopKConfig(k, score, weight, renorm, nmin, scale)
    out = hq.moe_router_topk(T.to_dev(logits, torch.float32, DEV), cfg,
                             None if bias is None else T.to_dev(bias, torch.float32, DEV))
    ids = out.indices.cpu().numpy().astype(np.uint32)
    w = out.values.cpu().numpy()
    want_ids, want_w = M.router_topk(logits, k, score, weight, renorm, nmin, scale, bias)
    if score == L.SCORE_RAW:
        ok = np.ones(len(logits), bool)       # selection on the logits themselves: no rounding involved
    else:
        sc = M._softmax_rows(logits) if score == L.SCORE_SOFTMAX else M._sigmoid(logits)
        ok = margin_ok_rows(sc + (bias if bias is not None else 0), k)
    assert ok.mean() > 0.95
    assert np.array_equal(ids[ok], want_ids[ok])
    assert np.allclose(w[ok], want_w[ok], rtol=2e-6, atol=1e-9)


def test_router_exact_ties_follow_the_canonical_rule():
    # hanzo-engine/src/ops.rs:3728-3758 plus wider rows with duplicated logits
    cfg = hq.MoeRouterTopKConfig(2, L.SCORE_RAW, L.WEIGHT_SCORE)
    s = torch.tensor([[1, 5, 2, 5, 4], [7, 7, 7, 7, 7]], dtype=torch.float32, device=DEV)
    out = hq.moe_router_topk(s, cfg)
    assert out.indices.cpu().tolist() == [[1, 3], [0, 1]]
    assert out.values.cpu().tolist() == [[5, 5], [7, 7]]
    rng = T.rng_for(3, 99)
    base = rng.integers(-3, 4, (200, 128)).astype(np.float32)       # many exact ties
    for score in (L.SCORE_RAW, L.SCORE_SOFTMAX, L.SCORE_SIGMOID):
        cfg = hq.MoeRouterTopKConfig(8, score, L.WEIGHT_SCORE)
        got = hq.moe_router_topk(T.to_dev(base, torch.float32, DEV), cfg).indices.cpu().numpy()
        want, _ = M.router_topk(base, 8, L.SCORE_RAW, L.WEIGHT_SCORE, False)   # monotone scores: same order
        assert np.array_equal(got.astype(np.uint32), want)
    # bf16 / f16 logits select like their f32 values
    lg = T.to_dev(rng.standard_normal((64, 256)).astype(np.float32), torch.bfloat16, DEV)
    cfg = hq.MoeRouterTopKConfig(8, L.SCORE_RAW, L.WEIGHT_SCORE)
    a = hq.moe_router_topk(lg, cfg).indices
    b = hq.moe_router_topk(lg.to(torch.float32), cfg).indices
    assert torch.equal(a, b)


@pytest.mark.parametrize("t,k,e", [(1, 8, 128), (3, 2, 4), (33, 4, 128), (64, 8, 128), (1024, 8, 256), (5000, 8, 128)])
def test_dispatch_tables_bit_exact(t, k, e):
    rng = T.rng_for(3, t)
    # distinct experts per token, skewed so some experts get nothing and some get many
    p = rng.dirichlet(np.full(e, 0.3))
    ids = np.stack([rng.choice(e, size=k, replace=False, p=p) for _ in range(t)]).astype(np.int32)
    tb = hq.moe_dispatch_build(T.to_dev(ids, torch.int32, DEV), e)
    bounds, sa, st = M.stable_permutation(ids.astype(np.uint32), e)
    assert np.array_equal(tb.expert_bounds.cpu().numpy(), bounds)
    assert np.array_equal(tb.sorted_assign.cpu().numpy(), sa)
    assert np.array_equal(tb.sorted_token.cpu().numpy(), st)
    inv = tb.inv_perm.cpu().numpy()
    assert np.array_equal(sa[inv], np.arange(t * k))
    # run twice: identical tables (no atomics on outputs)
    tb2 = hq.moe_dispatch_build(T.to_dev(ids, torch.int32, DEV), e)
    assert torch.equal(tb.sorted_assign, tb2.sorted_assign)


def test_gather_forward_known_answers():
    # hanzo-quant/src/unquantized/mod.rs:603-645 with the [2,2,3] bank zero-padded to K = 256 and stored as
    # exactly representable Q8_0 blocks (d = 1)
    bank = np.zeros((2, 2, 256), np.float32)
    bank[:, :, :3] = np.array([1, 0, 0, 0, 1, 0, 0, 0, 1, 1, 1, 1], np.float32).reshape(2, 2, 3)
    raw = np.zeros((4, 8, 34), np.uint8)
    raw[:, :, 0:2] = np.frombuffer(np.float16(1.0).tobytes(), np.uint8)
    raw[:, :, 2:] = bank.reshape(4, 8, 32).astype(np.int8).view(np.uint8)
    layer = hq.GgufMatMul(torch.from_numpy(raw.reshape(2, 2, -1)).to(DEV), "Q8_0", 256)
    x = np.zeros((2, 1, 256), np.float32)
    x[:, 0, :3] = np.arange(1, 7).reshape(2, 3)
    ids = torch.tensor([[0, 1], [1, 0]], dtype=torch.int32, device=DEV)
    out = layer.gather_forward(T.to_dev(x, torch.float32, DEV), ids)
    assert out.shape == (2, 2, 2)
    assert out.reshape(-1).cpu().tolist() == [1, 2, 3, 6, 6, 15, 4, 5]
    x2 = x.reshape(1, 2, 256)
    out2 = layer.gather_forward(T.to_dev(x2, torch.float32, DEV), torch.tensor([[0, 1]], dtype=torch.int32, device=DEV))
    assert out2.reshape(-1).cpu().tolist() == [1, 2, 6, 15]


@pytest.mark.parametrize("fmt,k,n", [("Q4_K", 512, 192), ("Q8_0", 256, 64), ("FP8", 256, 128), ("MXFP4", 96, 80),
                                     ("Q6_K", 256, 72), ("Q5_K", 512, 64), ("Q4_0", 256, 40), ("Q5_0", 256, 40),
                                     ("Q4_1", 256, 40), ("Q5_1", 256, 40), ("Q2_K", 768, 72), ("Q3_K", 768, 72)])
@pytest.mark.parametrize("per_slot", [False, True])
def test_gather_forward_matches_oracle(fmt, k, n, per_slot):
    rng = T.rng_for(3, k + n)
    e, t, topk = 6, 19, 3
    arrays, deq = T.make_weight(fmt, rng, n, k, experts=e)
    bias = None
    bd = None
    if fmt == "MXFP4":
        bd = T.to_dev(rng.normal(0, 0.02, (e, n)).astype(np.float32), torch.bfloat16, DEV)
        bias = bd.to(torch.float32).cpu().numpy()
    layer = T.make_layer(fmt, arrays, k, DEV, bd)
    ids = np.stack([rng.choice(e, size=topk, replace=False) for _ in range(t)]).astype(np.int32)
    shape = (t, topk, k) if per_slot else ((t, k) if fmt == "MXFP4" else (t, 1, k))
    xd = T.to_dev(rng.standard_normal(shape).astype(np.float32), torch.bfloat16, DEV)
    out = layer.gather_forward_raw(xd, T.to_dev(ids, torch.int32, DEV), torch.float32)
    want = M.gather_forward(xd.to(torch.float32).cpu().numpy(), ids.astype(np.uint32), deq, bias)
    assert out.shape == (t, topk, n)
    assert T.rel_l2(out.cpu().numpy(), want) <= TOL[fmt]
    assert layer.device_status()[0] == 0


def _moe_case(fmt, t, e, k, h, i, interleaved, act, seed, limit=None, down_fmt=None):
    rng = T.rng_for(4, seed)
    down_fmt = down_fmt or fmt
    if interleaved:
        gu_a, gu_deq = T.make_weight(fmt, rng, 2 * i, h, experts=e)
        gub = T.to_dev(rng.normal(0, 0.02, (e, 2 * i)).astype(np.float32), torch.bfloat16, DEV)
        gate_up = T.make_layer(fmt, gu_a, h, DEV, gub)
    else:
        g_a, g_deq = T.make_weight(fmt, rng, i, h, experts=e)
        u_a, u_deq = T.make_weight(fmt, rng, i, h, experts=e)
        gate, up = T.make_layer(fmt, g_a, h, DEV), T.make_layer(fmt, u_a, h, DEV)
    d_a, d_deq = T.make_weight(down_fmt, rng, h, i, experts=e)
    db = T.to_dev(rng.normal(0, 0.02, (e, h)).astype(np.float32), torch.bfloat16, DEV) if interleaved else None
    down = T.make_layer(down_fmt, d_a, i, DEV, db)
    x = T.to_dev(rng.standard_normal((t, h)).astype(np.float32), torch.bfloat16, DEV)
    logits = rng.standard_normal((t, e)).astype(np.float32)
    ids, w = M.router_topk(logits, k, L.SCORE_SOFTMAX, L.WEIGHT_SCORE, True)
    ids_d, w_d = T.to_dev(ids.astype(np.int32), torch.int32, DEV), T.to_dev(w, torch.float32, DEV)
    x_np = x.to(torch.float32).cpu().numpy()
    f16 = lambda a: a.astype(np.float16).astype(np.float32)
    if interleaved:
        experts = hq.MoEExperts(down, gate_up_proj=gate_up, act=act, limit=limit)
        want = M.moe_layer(x_np, ids, w, None, None, d_deq, act, gate_up_bank=gu_deq,
                           gate_up_bias=gub.to(torch.float32).cpu().numpy(),
                           down_bias=db.to(torch.float32).cpu().numpy(), limit=limit, h_round=f16)
    else:
        experts = hq.MoEExperts(down, gate, up, act=act, limit=limit)
        want = M.moe_layer(x_np, ids, w, g_deq, u_deq, d_deq, act, limit=limit, h_round=f16)
    got = experts.forward(x, w_d, ids_d, out_dtype=torch.float32)
    # the one-call form of the same layer (router included) launches the same kernels as the separate calls: same bits
    rcfg = hq.MoeRouterTopKConfig(k, L.SCORE_SOFTMAX, L.WEIGHT_SCORE, True)
    logits_d = T.to_dev(logits, torch.float32, DEV)
    top = hq.moe_router_topk(logits_d, rcfg)
    assert np.array_equal(top.indices.cpu().numpy().astype(np.uint32), ids)
    split = experts.forward(x, top.values, top.indices, out_dtype=torch.float32)
    fused = experts.forward_layer(x, logits_d, rcfg, out_dtype=torch.float32)
    assert torch.equal(fused, split)
    return got.cpu().numpy(), want


@pytest.mark.parametrize("t", [1, 7, 64])
def test_moe_block_q4_k_swiglu(t):
    # Qwen3-30B-A3B-shaped layer at reduced width: separate gate/up banks, plain SwiGLU
    got, want = _moe_case("Q4_K", t, 16, 4, 512, 256, False, L.ACT_SWIGLU, t)
    assert T.rel_l2(got, want) <= 1e-3


@pytest.mark.parametrize("t", [5, 300])
def test_moe_block_q4_k_m_mix(t):
    # a Q4_K_M file's layer: gate / up experts in Q4_K, down experts in Q6_K; decode rows and prefill rows
    got, want = _moe_case("Q4_K", t, 8, 2, 512, 256, False, L.ACT_SWIGLU, 20 + t, down_fmt="Q6_K")
    assert T.rel_l2(got, want) <= 1e-3


@pytest.mark.parametrize("t", [3, 200])
def test_moe_block_q6_k_gate_and_up(t):
    got, want = _moe_case("Q6_K", t, 4, 2, 256, 256, False, L.ACT_SWIGLU, 30 + t)
    assert T.rel_l2(got, want) <= 1e-3


@pytest.mark.parametrize("fmt", ["Q5_K", "Q4_0", "Q5_0", "Q4_1", "Q5_1", "Q2_K", "Q3_K"])
@pytest.mark.parametrize("t", [3, 200])
def test_moe_block_further_ggml_types(fmt, t):
    # decode rows (the warp-MMA decode kernel) and prefill rows (the tcgen05 grouped GEMM: 200 tokens x top-2 over 4
    # experts is 100 rows per expert)
    got, want = _moe_case(fmt, t, 4, 2, 256, 256, False, L.ACT_SWIGLU, 40 + t)
    assert T.rel_l2(got, want) <= 1e-3


def test_moe_block_fp8_swiglu():
    got, want = _moe_case("FP8", 40, 8, 4, 512, 256, False, L.ACT_SWIGLU, 5)
    assert T.rel_l2(got, want) <= 2e-3


def test_moe_block_mxfp4_gptoss():
    # gpt-oss-shaped: interleaved gate/up rows, biases, clamp 7.0 / alpha 1.702
    got, want = _moe_case("MXFP4", 33, 8, 4, 288, 288, True, L.ACT_GPTOSS, 6, limit=7.0)
    assert T.rel_l2(got, want) <= 2e-3


def test_weighted_reduce_and_gated_act():
    rng = T.rng_for(4, 9)
    y = rng.standard_normal((10, 4, 200)).astype(np.float32)
    w = rng.random((10, 4)).astype(np.float32)
    add = rng.standard_normal((10, 200)).astype(np.float32)
    got = hq.moe_weighted_reduce(T.to_dev(y, torch.float32, DEV), T.to_dev(w, torch.float32, DEV), torch.float32,
                                 addend=T.to_dev(add, torch.float32, DEV))
    assert np.allclose(got.cpu().numpy(), M.weighted_combine(y, w) + add, rtol=1e-6, atol=1e-6)
    yb = T.to_dev(y, torch.bfloat16, DEV)
    got = hq.moe_weighted_reduce(yb, T.to_dev(w, torch.float32, DEV), torch.bfloat16)
    want = F.round_bf16(M.weighted_combine(yb.to(torch.float32).cpu().numpy(), w))
    assert np.abs(got.to(torch.float32).cpu().numpy() - want).max() <= np.abs(want).max() * 2 ** -7
    g = rng.standard_normal((6, 50)).astype(np.float32) * 4
    u = rng.standard_normal((6, 50)).astype(np.float32) * 4
    gd, ud = T.to_dev(g, torch.float32, DEV), T.to_dev(u, torch.float32, DEV)
    assert np.allclose(hq.gated_act(gd, ud, L.ACT_SWIGLU).cpu().numpy(), M.swiglu(g, u), rtol=1e-5, atol=1e-6)
    assert np.allclose(hq.gated_act(gd, ud, L.ACT_SWIGLU, limit=1.0).cpu().numpy(), M.swiglu(g, u, 1.0), rtol=1e-5,
                       atol=1e-6)
    assert np.allclose(hq.gated_act(gd, ud, L.ACT_GPTOSS, limit=7.0).cpu().numpy(), M.gptoss_swiglu(g, u), rtol=1e-5,
                       atol=1e-6)
    inter = np.stack([g, u], axis=-1)
    got = hq.gated_act(T.to_dev(inter, torch.float32, DEV), None, L.ACT_GPTOSS, limit=7.0, interleaved=True)
    assert np.allclose(got.cpu().numpy(), M.gptoss_swiglu(g, u), rtol=1e-5, atol=1e-6)


def test_fp8_quantizers_bit_exact():
    rng = T.rng_for(4, 11)
    x = (rng.standard_normal((37, 256)) * 2).astype(np.float32)
    x[3, :128] = 0
    codes, scales = hq.fp8_vector_quantize(T.to_dev(x, torch.float32, DEV))
    wc, ws = F.fp8_vector_quant(x)
    assert np.array_equal(scales.cpu().numpy(), ws.reshape(-1))
    assert np.array_equal(F.e4m3_decode(codes.cpu().numpy()), F.e4m3_decode(wc))
    back = hq.fp8_vector_dequantize(codes, scales, torch.float32).cpu().numpy()
    assert np.array_equal(back, F.fp8_vector_dequant(wc, ws))
    w = rng.normal(0, 0.02, (200, 300)).astype(np.float32)
    c, s = hq.fp8_blockwise_quantize(T.to_dev(w, torch.float32, DEV))
    oc, os_ = F.fp8_block_quant(w)
    assert np.array_equal(s.cpu().numpy(), os_)
    assert np.array_equal(F.e4m3_decode(c.cpu().numpy()), F.e4m3_decode(oc))
    deq = hq.fp8_blockwise_dequantize(c, s, (128, 128), torch.float32).cpu().numpy()
    assert np.array_equal(deq, F.fp8_block_dequant(oc, os_))
    # the reference's known answer: ones(5,5), 2x2 blocks, scales arange(9) (blockwise_fp8/ops.rs:1098-1118)
    ones = torch.full((5, 5), 0x38, dtype=torch.uint8, device=DEV)
    sc = torch.arange(9, dtype=torch.float32, device=DEV).reshape(3, 3)
    got = hq.fp8_blockwise_dequantize(ones, sc, (2, 2), torch.float32).cpu().tolist()
    assert got == [[0, 0, 1, 1, 2], [0, 0, 1, 1, 2], [3, 3, 4, 4, 5], [3, 3, 4, 4, 5], [6, 6, 7, 7, 8]]


# ---- tensor-core (tcgen05) grouped GEMM: forced on, checked against the oracle and the decode kernel ----------

@pytest.fixture
def tensor_path():
    lib = L.lib()
    old = (lib.hq_config_get(L.CFG_MOE_TENSOR_MIN_ROWS), lib.hq_config_get(L.CFG_DENSE_TENSOR_MIN_ROWS))
    lib.hq_config_set(L.CFG_MOE_TENSOR_MIN_ROWS, 0)
    lib.hq_config_set(L.CFG_DENSE_TENSOR_MIN_ROWS, 1)
    yield lib
    lib.hq_config_set(L.CFG_MOE_TENSOR_MIN_ROWS, old[0])
    lib.hq_config_set(L.CFG_DENSE_TENSOR_MIN_ROWS, old[1])


@pytest.mark.parametrize("fmt,n,k,m", [("Q4_K", 256, 512, 128), ("Q4_K", 200, 256, 37), ("FP8", 256, 384, 130),
                                       ("MXFP4", 192, 320, 64), ("MXFP4", 2880, 2880, 150), ("Q4_K", 4096, 4096, 16)])
def test_tensor_path_dense(tensor_path, fmt, n, k, m):
    rng = T.rng_for(5, n + k + m)
    arrays, deq = T.make_weight(fmt, rng, n, k)
    bd = T.to_dev(rng.normal(0, 0.02, n).astype(np.float32), torch.bfloat16, DEV) if fmt == "MXFP4" else None
    layer = T.make_layer(fmt, arrays, k, DEV, bd)
    xd = T.to_dev(rng.standard_normal((m, k)).astype(np.float32), torch.bfloat16, DEV)
    got = layer.forward_raw(xd, torch.float32)
    torch.cuda.synchronize()
    assert layer.device_status()[0] == 0, layer.device_status()
    want = M.dense_forward(xd.to(torch.float32).cpu().numpy(), deq,
                           None if bd is None else bd.to(torch.float32).cpu().numpy())
    assert T.rel_l2(got.cpu().numpy(), want) <= TOL[fmt]
    # and it agrees with the decode kernel on the same inputs
    tensor_path.hq_config_set(L.CFG_DENSE_TENSOR_MIN_ROWS, 1 << 40)
    ref = layer.forward_raw(xd, torch.float32)
    assert T.rel_l2(got.cpu().numpy(), ref.cpu().numpy()) <= TOL[fmt]


@pytest.mark.parametrize("fmt,k,n", [("Q4_K", 512, 192), ("FP8", 256, 128), ("MXFP4", 128, 144)])
def test_tensor_path_gather_forward(tensor_path, fmt, k, n):
    rng = T.rng_for(5, k + n)
    e, t, topk = 5, 300, 2          # expert 4 gets nothing, expert 0 gets several 128-row tiles
    arrays, deq = T.make_weight(fmt, rng, n, k, experts=e)
    layer = T.make_layer(fmt, arrays, k, DEV)
    p = np.array([0.7, 0.15, 0.1, 0.05, 0.0])
    ids = np.stack([rng.choice(e, size=topk, replace=False, p=p) for _ in range(t)]).astype(np.int32)
    xd = T.to_dev(rng.standard_normal((t, k)).astype(np.float32), torch.bfloat16, DEV)
    out = layer.gather_forward_raw(xd, T.to_dev(ids, torch.int32, DEV), torch.float32)
    torch.cuda.synchronize()
    assert layer.device_status()[0] == 0, layer.device_status()
    want = M.gather_forward(xd.to(torch.float32).cpu().numpy(), ids.astype(np.uint32), deq)
    assert T.rel_l2(out.cpu().numpy(), want) <= TOL[fmt]
    again = layer.gather_forward_raw(xd, T.to_dev(ids, torch.int32, DEV), torch.float32)
    assert torch.equal(out, again)            # no atomics anywhere: bit-reproducible


def test_tensor_path_moe_blocks(tensor_path):
    got, want = _moe_case("Q4_K", 200, 8, 4, 512, 256, False, L.ACT_SWIGLU, 21)
    assert T.rel_l2(got, want) <= 1e-3
    got, want = _moe_case("FP8", 150, 8, 4, 512, 256, False, L.ACT_SWIGLU, 22)
    assert T.rel_l2(got, want) <= 2e-3
    got, want = _moe_case("MXFP4", 140, 8, 4, 320, 320, True, L.ACT_GPTOSS, 23, limit=7.0)
    assert T.rel_l2(got, want) <= 2e-3


def test_tensor_path_wide_token_tiles(tensor_path):
    # enough rows per expert on average for the 256-token tiles (f16 rows copied with cp.async)
    rng = T.rng_for(5, 91)
    e, t, topk, k, n = 4, 700, 2, 256, 192
    arrays, deq = T.make_weight("Q4_K", rng, n, k, experts=e)
    layer = T.make_layer("Q4_K", arrays, k, DEV)
    p = np.array([0.55, 0.3, 0.15, 0.0])
    ids = np.stack([rng.choice(e, size=topk, replace=False, p=p) for _ in range(t)]).astype(np.int32)
    xd = T.to_dev(rng.standard_normal((t, k)).astype(np.float32), torch.bfloat16, DEV)
    out = layer.gather_forward_raw(xd, T.to_dev(ids, torch.int32, DEV), torch.float32)
    torch.cuda.synchronize()
    assert layer.device_status()[0] == 0, layer.device_status()
    want = M.gather_forward(xd.to(torch.float32).cpu().numpy(), ids.astype(np.uint32), deq)
    assert T.rel_l2(out.cpu().numpy(), want) <= 1e-3
    got, want = _moe_case("Q4_K", 450, 8, 4, 512, 256, False, L.ACT_SWIGLU, 31)
    assert T.rel_l2(got, want) <= 1e-3
    got, want = _moe_case("MXFP4", 450, 8, 4, 320, 320, True, L.ACT_GPTOSS, 32, limit=7.0)
    assert T.rel_l2(got, want) <= 2e-3
    got, want = _moe_case("FP8", 450, 8, 4, 512, 256, False, L.ACT_SWIGLU, 33)
    assert T.rel_l2(got, want) <= 2e-3


def test_tensor_path_short_k_and_partial_feature_tiles(tensor_path):
    # the kernel that expands the weights into tensor memory, at its edges: K of one, three and five 64-column
    # stages (fewer stages than producer groups: a group's next stage lies in a later tile), 64-feature gate/up
    # tiles with a partly filled last tile, a 128-lane tile with 64 valid rows, token tiles with a few rows
    got, want = _moe_case("MXFP4", 300, 8, 4, 64, 192, True, L.ACT_GPTOSS, 41, limit=7.0)
    assert T.rel_l2(got, want) <= 2e-3
    got, want = _moe_case("MXFP4", 131, 4, 2, 320, 64, True, L.ACT_GPTOSS, 42, limit=7.0)
    assert T.rel_l2(got, want) <= 2e-3
    got, want = _moe_case("Q4_K", 260, 4, 2, 256, 256, False, L.ACT_SWIGLU, 43)
    assert T.rel_l2(got, want) <= 1e-3
    for fmt, n, k, m in [("MXFP4", 72, 64, 300), ("MXFP4", 200, 192, 129), ("Q4_K", 72, 256, 260)]:
        rng = T.rng_for(5, 1000 + n + k + m)
        arrays, deq = T.make_weight(fmt, rng, n, k)
        layer = T.make_layer(fmt, arrays, k, DEV)
        xd = T.to_dev(rng.standard_normal((m, k)).astype(np.float32), torch.bfloat16, DEV)
        got = layer.forward_raw(xd, torch.float32)
        torch.cuda.synchronize()
        assert layer.device_status()[0] == 0, layer.device_status()
        want = M.dense_forward(xd.to(torch.float32).cpu().numpy(), deq, None)
        assert T.rel_l2(got.cpu().numpy(), want) <= TOL[fmt], (fmt, n, k, m)
        assert torch.equal(got, layer.forward_raw(xd, torch.float32))


@pytest.mark.parametrize("group_score", ["top2_sum", "max"])
def test_group_limited_router_matches_oracle(group_score):
    """DeepSeek-V3 routing: 256 experts in 8 groups, 4 groups kept, top-8, sigmoid scores + selection bias,
    renormalised and scaled by 2.5 (hanzo-engine/src/models/deepseek3.rs:623-702)."""
    import engine_b200 as hq
    from engine_b200 import _lib as L
    rng = T.rng_for(4, 77)
    t, e, k = 500, 256, 8
    logits = rng.standard_normal((t, e)).astype(np.float32)
    logits[7] = logits[7, 0]                 # a row of exact ties: decided by index order alone
    bias = (rng.standard_normal(e) * 0.01).astype(np.float32)
    cfg = hq.MoeRouterTopKConfig(k, L.SCORE_SIGMOID, L.WEIGHT_SCORE, True, 1e-20, 2.5)
    top = hq.moe_router_topk(T.to_dev(logits, torch.float32, DEV), cfg, T.to_dev(bias, torch.float32, DEV),
                             n_group=8, topk_group=4, group_score=group_score)
    ids, w = M.router_topk_grouped(logits, k, M.SCORE_SIGMOID, 8, 4, group_score, bias, True, 1e-20, 2.5)
    got = top.indices.cpu().numpy().astype(np.uint32)
    same = (got == ids).all(axis=1)
    assert same.mean() >= 0.995 and same[7]
    assert np.allclose(top.values.cpu().numpy()[same], w[same], rtol=2e-6, atol=1e-9)
    # the selected experts come from at most 4 groups
    assert all(len(set(int(v) // 32 for v in row)) <= 4 for row in got)
