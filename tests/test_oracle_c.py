"""The C restatement of the oracle agrees with the numpy one (which is pinned against the golden vectors)."""
import numpy as np
import pytest

from oracle import cbuild
from oracle import moe as M
from tests import hq_testlib as T


@pytest.mark.parametrize("fmt,k", [("Q8_0", 512), ("Q4_K", 512), ("FP8", 384), ("MXFP4", 96), ("Q6_K", 512), ("Q5_K", 512),
                                   ("Q4_0", 256), ("Q5_0", 256), ("Q4_1", 256), ("Q5_1", 256), ("Q2_K", 768),
                                   ("Q3_K", 768)])
def test_c_linear_matches_numpy(fmt, k):
    rng = T.rng_for(7, k)
    n = 256 if fmt == "FP8" else 70
    arrays, deq = T.make_weight(fmt, rng, n, k)
    x = rng.standard_normal((5, k)).astype(np.float32)
    w = arrays.get("data", arrays.get("weight", arrays.get("blocks")))
    sc = arrays.get("scale", arrays.get("scales"))
    got = cbuild.linear(fmt, w, sc, None, x)
    assert T.rel_l2(got, M.dense_forward(x, deq)) < 2e-6


def test_c_gather_matches_numpy():
    rng = T.rng_for(7, 1)
    e, n, k, t, topk = 5, 48, 256, 13, 2
    arrays, deq = T.make_weight("Q4_K", rng, n, k, experts=e)
    x = rng.standard_normal((t, k)).astype(np.float32)
    ids = np.stack([rng.choice(e, size=topk, replace=False) for _ in range(t)]).astype(np.uint32)
    bounds, sa, st = M.stable_permutation(ids, e)
    got = cbuild.gather("Q4_K", arrays["data"], None, None, x, e, bounds, st, sa, t * topk)
    want = M.gather_forward(x, ids, deq).reshape(t * topk, n)
    assert T.rel_l2(got, want) < 2e-6
