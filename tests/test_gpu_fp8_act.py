"""Block-FP8 layers with block-scaled FP8 activations (the FP8 tensor-core path): against the oracle with the
reference's 1x128 activation quantizer applied first (hanzo-quant/src/vector_fp8/ops.rs:235-287).  Products of
e4m3 values are exact, so what remains is f32 summation order and the rare code that flips where an intermediate
sits on a rounding boundary: rel-L2 <= 2e-3, the FP8 tolerance."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

from oracle import formats as F
from oracle import moe as M
from tests import hq_testlib as T

DEV = "cuda:0"


def _qdq(a):
    codes, scale = F.fp8_vector_quant(a.reshape(-1), 128)
    return F.fp8_vector_dequant(codes, scale, 128).reshape(a.shape).astype(np.float32)


def test_row_quantizer_matches_the_oracle_bit_for_bit():
    import engine_b200 as hq
    rng = T.rng_for(9, 1)
    x = rng.standard_normal((37, 512)).astype(np.float32)
    x[3] = 0.0
    rows = rng.integers(0, 37, 90).astype(np.int32)
    codes, scales = hq.fp8_quantize_rows(T.to_dev(x, torch.float32, DEV), torch.from_numpy(rows).to(DEV))
    want_c, want_s = F.fp8_vector_quant(x[rows].reshape(-1), 128)
    assert np.array_equal(codes.cpu().numpy().reshape(-1), want_c)
    assert np.array_equal(scales.cpu().numpy().reshape(-1), want_s)


@pytest.mark.parametrize("m", [1, 100, 128, 300])
def test_dense_layer_over_quantized_rows(m):
    import engine_b200 as hq
    n, k = 256, 1024
    rng = T.rng_for(9, 2)
    arrays, deq = T.make_weight("FP8", rng, n, k)
    layer = T.make_layer("FP8", arrays, k, DEV)
    x = rng.standard_normal((m, k)).astype(np.float32)
    codes, scales = hq.fp8_quantize_rows(T.to_dev(x, torch.float32, DEV))
    y = layer.forward_fp8_rows(codes, scales, torch.float32)
    torch.cuda.synchronize()
    assert layer.device_status()[0] == 0
    want = M.dense_forward(_qdq(x), deq, None)
    assert T.rel_l2(y.cpu().numpy(), want) <= 1e-5     # exact products: only the summation order differs


def test_expert_block_with_fp8_activations():
    import engine_b200 as hq
    from engine_b200 import _lib as L
    e, k, h, i, t = 8, 2, 1024, 512, 300
    rng = T.rng_for(9, 3)
    ga, gd = T.make_weight("FP8", rng, i, h, experts=e)
    ua, ud = T.make_weight("FP8", rng, i, h, experts=e)
    da, dd = T.make_weight("FP8", rng, h, i, experts=e)
    experts = hq.MoEExperts(T.make_layer("FP8", da, i, DEV), T.make_layer("FP8", ga, h, DEV),
                            T.make_layer("FP8", ua, h, DEV))
    x = rng.standard_normal((t, h)).astype(np.float32)
    logits = rng.standard_normal((t, e)).astype(np.float32)
    logits[:, 0] += 2.0                      # uneven experts: some tiles full, one expert nearly empty
    logits[:, 5] -= 6.0
    ids, w = M.router_topk(logits, k, M.SCORE_SOFTMAX, M.WEIGHT_SCORE, True)
    xd = T.to_dev(x, torch.bfloat16, DEV)
    out = experts.forward_fp8_act(xd, T.to_dev(w, torch.float32, DEV),
                                  torch.from_numpy(ids.astype(np.int32)).to(DEV), out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert experts.gate.device_status()[0] == 0
    x_used = _qdq(xd.to(torch.float32).cpu().numpy())
    f16 = lambda a: a.astype(np.float16).astype(np.float32)
    want = M.moe_layer(x_used, ids, w, gd, ud, dd, h_round=_qdq, gu_round=f16)
    assert T.rel_l2(out.cpu().numpy(), want) <= 2e-3
