"""Router / permutation / gather known answers restated from the reference's tests."""
import numpy as np

from oracle import moe as M


def test_tie_break_lowest_expert():
    # hanzo-engine/src/ops.rs:3728-3758
    s = np.array([[1, 5, 2, 5, 4], [7, 7, 7, 7, 7]], np.float32)
    assert M.deterministic_topk_indices(s, 2).tolist() == [[1, 3], [0, 1]]
    ids, w = M.router_topk(s, 2, M.SCORE_RAW, M.WEIGHT_SCORE, False)
    assert ids.tolist() == [[1, 3], [0, 1]] and w.tolist() == [[5, 5], [7, 7]]


def test_topk_descending():
    # hanzo-engine/src/ops.rs:3824-3851
    x = np.array([[1, 3, 5], [2, 4, 6]], np.float32)
    ids, w = M.router_topk(x, 2, M.SCORE_RAW, M.WEIGHT_SCORE, False)
    assert ids.tolist() == [[2, 1], [2, 1]] and w.tolist() == [[5, 3], [6, 4]]


def test_swiglu_clamp_kat():
    # hanzo-engine/src/ops.rs:3805-3821 (limit 1.0 clamps gate above, up both sides)
    g = np.array([[10.0, -10.0, 0.5]], np.float32)
    u = np.array([[10.0, -10.0, 0.5]], np.float32)
    out = M.swiglu(g, u, 1.0)
    want = M.silu(np.array([[1.0, -10.0, 0.5]], np.float32)) * np.array([[1.0, -1.0, 0.5]], np.float32)
    assert np.array_equal(out, want)
    assert np.array_equal(M.swiglu(g, u, None), M.silu(g) * u)


def _bank():
    # hanzo-quant/src/unquantized/mod.rs:603-610: [2,2,3]
    return np.array([1, 0, 0, 0, 1, 0, 0, 0, 1, 1, 1, 1], np.float32).reshape(2, 2, 3)


def test_gather_forward_single_route_input():
    # hanzo-quant/src/unquantized/mod.rs:616-631
    x = np.arange(1, 7, dtype=np.float32).reshape(2, 1, 3)
    ids = np.array([[0, 1], [1, 0]], np.uint32)
    out = M.gather_forward(x, ids, _bank())
    assert out.shape == (2, 2, 2)
    assert out.reshape(-1).tolist() == [1, 2, 3, 6, 6, 15, 4, 5]


def test_gather_forward_per_route_input():
    # hanzo-quant/src/unquantized/mod.rs:633-645
    x = np.arange(1, 7, dtype=np.float32).reshape(1, 2, 3)
    ids = np.array([[0, 1]], np.uint32)
    out = M.gather_forward(x, ids, _bank())
    assert out.reshape(-1).tolist() == [1, 2, 6, 15]


def test_stable_permutation():
    ids = np.array([[2, 0], [0, 2], [1, 0]], np.uint32)
    bounds, sa, st = M.stable_permutation(ids, 4)
    assert bounds.tolist() == [0, 3, 4, 6, 6]
    assert sa.tolist() == [1, 2, 5, 4, 0, 3]
    assert st.tolist() == [0, 1, 2, 2, 0, 1]


def test_router_modes():
    rng = np.random.default_rng(1)
    lg = rng.standard_normal((16, 32)).astype(np.float32)
    ids, w = M.router_topk(lg, 4, M.SCORE_SOFTMAX, M.WEIGHT_SCORE, True)
    assert np.allclose(w.sum(1), 1, atol=1e-6)
    # gpt-oss: top-k on logits then softmax over the k values (hanzo-engine/src/models/gpt_oss.rs:396-403)
    ids2, w2 = M.router_topk(lg, 4, M.SCORE_RAW, M.WEIGHT_SOFTMAX, False)
    assert np.array_equal(ids, ids2)
    assert np.allclose(w, w2, atol=1e-6)
    # DeepSeek: sigmoid + selection bias, unbiased weights (hanzo-engine/src/models/deepseek3.rs:620-700)
    bias = rng.normal(0, 1, 32).astype(np.float32)
    ids3, w3 = M.router_topk(lg, 4, M.SCORE_SIGMOID, M.WEIGHT_SCORE, True, 1e-20, 2.5, bias)
    sg = 1 / (1 + np.exp(-lg))
    assert np.array_equal(ids3, M.deterministic_topk_indices(sg + bias, 4))
    assert np.allclose(w3.sum(1), 2.5, atol=1e-5)


def test_moe_layer_matches_dense_loop():
    rng = np.random.default_rng(2)
    t, k, e, h, i = 5, 2, 4, 8, 6
    x = rng.standard_normal((t, h)).astype(np.float32)
    gb, ub = rng.standard_normal((2, e, i, h)).astype(np.float32)
    db = rng.standard_normal((e, h, i)).astype(np.float32)
    ids, w = M.router_topk(rng.standard_normal((t, e)).astype(np.float32), k, M.SCORE_SOFTMAX, M.WEIGHT_SCORE, True)
    got = M.moe_layer(x, ids, w, gb, ub, db)
    want = np.zeros((t, h), np.float32)
    for ti in range(t):
        for s in range(k):
            ex = ids[ti, s]
            hh = M.silu(gb[ex] @ x[ti]) * (ub[ex] @ x[ti])
            want[ti] += w[ti, s] * (db[ex] @ hh)
    assert np.allclose(got, want, rtol=1e-4, atol=1e-4)
    # interleaved gate/up bank gives the same answer
    gu = np.empty((e, 2 * i, h), np.float32)
    gu[:, 0::2], gu[:, 1::2] = gb, ub
    got2 = M.moe_layer(x, ids, w, None, None, db, gate_up_bank=gu)
    assert np.allclose(got, got2, rtol=1e-5, atol=1e-5)


def test_group_limited_routing_hand_case():
    """hanzo-engine/src/models/deepseek3.rs:623-660 on a case small enough to do by hand: 8 experts in 4 groups of
    2, keep the 2 best groups by the sum of their two scores, then top-3 among what is left."""
    from oracle import moe as M
    scores = np.array([[0.9, 0.1, 0.5, 0.6, 0.2, 0.95, 0.3, 0.3]], np.float32)    # raw scores, no bias
    # group sums: 1.0, 1.1, 1.15, 0.6 -> groups 2 and 1 stay -> candidates 2, 3, 4, 5 (the rest score 0)
    ids, w = M.router_topk_grouped(scores, 3, M.SCORE_RAW, 4, 2, "top2_sum", renormalize=True, norm_min=0.0)
    assert ids.tolist() == [[5, 3, 2]]
    np.testing.assert_allclose(w[0], np.array([0.95, 0.6, 0.5], np.float32) / np.float32(2.05), rtol=1e-6)
    # group_limited_greedy: group score = its best expert: 0.9, 0.6, 0.95, 0.3 -> groups 2 and 0
    ids, _ = M.router_topk_grouped(scores, 3, M.SCORE_RAW, 4, 2, "max", renormalize=False)
    assert ids.tolist() == [[5, 0, 4]]
