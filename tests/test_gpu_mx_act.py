"""MXFP4 layers with MXFP8 activations (the block-scaled tensor-core path): against the oracle with the same
activation quantizer applied first (e4m3 elements, one power-of-two scale per 32 elements).  Products of e4m3 and
e2m1 values and the power-of-two scales are exact, so what remains is f32 summation order and the rare code that
flips where an intermediate sits on a rounding boundary: rel-L2 <= 2e-3, the MXFP4 tolerance."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

from oracle import formats as F
from oracle import moe as M
from tests import hq_testlib as T

DEV = "cuda:0"


def _qdq(a):
    return F.mxfp8_dequant(*F.mxfp8_quant(np.ascontiguousarray(a, dtype=np.float32))).astype(np.float32)


def test_row_quantizer_matches_the_oracle_bit_for_bit():
    import engine_b200 as hq
    rng = T.rng_for(11, 1)
    x = (rng.standard_normal((37, 320)) * rng.choice([1e-4, 1.0, 500.0], (37, 1))).astype(np.float32)
    x[3] = 0.0
    x[5, :32] = 0.0
    rows = rng.integers(0, 37, 90).astype(np.int32)
    codes, scales = hq.mxfp8_quantize_rows(T.to_dev(x, torch.float32, DEV), torch.from_numpy(rows).to(DEV))
    want_c, want_s = F.mxfp8_quant(x[rows])
    assert np.array_equal(scales.cpu().numpy(), want_s)
    assert np.array_equal(codes.cpu().numpy(), want_c)


@pytest.mark.parametrize("m,n,k", [(1, 256, 256), (100, 192, 512), (128, 128, 128), (300, 320, 2880), (77, 72, 192)])
def test_dense_layer_over_quantized_rows(m, n, k):
    # K = 2880 (gpt-oss) ends in a 64-element stage; K = 192 in one of 64; N = 72 / 192 / 320 end in partial tiles
    import engine_b200 as hq
    rng = T.rng_for(11, 2)
    arrays, deq = T.make_weight("MXFP4", rng, n, k)
    bias = rng.standard_normal(n).astype(np.float32) * 0.1
    layer = T.make_layer("MXFP4", arrays, k, DEV, T.to_dev(bias, torch.float32, DEV))
    x = rng.standard_normal((m, k)).astype(np.float32)
    codes, scales = hq.mxfp8_quantize_rows(T.to_dev(x, torch.float32, DEV))
    y = layer.forward_mx_rows(codes, scales, torch.float32)
    torch.cuda.synchronize()
    assert layer.device_status()[0] == 0
    want = M.dense_forward(_qdq(x), deq, bias)
    assert T.rel_l2(y.cpu().numpy(), want) <= 1e-5     # exact products: only the summation order differs


def test_scale_bytes_reach_the_right_rows_and_columns():
    # every weight row and every K block with its own exponent, every token with its own magnitude: a scale byte
    # that lands on the wrong lane, column or K block changes the result by a power of two
    import engine_b200 as hq
    n, k, m = 256, 512, 130
    rng = T.rng_for(11, 3)
    w = rng.standard_normal((n, k)).astype(np.float32)
    w *= np.exp2(rng.integers(-6, 7, (n, k // 32))).repeat(32, axis=1).astype(np.float32)
    b, s = F.mxfp4_quantize(w)
    deq = F.mxfp4_dequant(b, s)
    layer = T.make_layer("MXFP4", {"blocks": b, "scales": s}, k, DEV)
    x = rng.standard_normal((m, k)).astype(np.float32)
    x *= np.exp2(rng.integers(-8, 9, (m, k // 32))).repeat(32, axis=1).astype(np.float32)
    codes, scales = hq.mxfp8_quantize_rows(T.to_dev(x, torch.float32, DEV))
    y = layer.forward_mx_rows(codes, scales, torch.float32)
    torch.cuda.synchronize()
    want = M.dense_forward(_qdq(x), deq, None)
    assert T.rel_l2(y.cpu().numpy(), want) <= 1e-5
    # row by row as well: a global norm would hide a few misplaced rows
    err = np.abs(y.cpu().numpy() - want).max(axis=1) / (np.abs(want).max(axis=1) + 1e-30)
    assert err.max() <= 1e-4


def _expert_block_case(e, k, h, i, t, seed, interleaved=True, skew=None, out_dtype=None, pad_slot=False):
    import engine_b200 as hq
    from engine_b200 import _lib as L
    rng = T.rng_for(11, seed)
    x = rng.standard_normal((t, h)).astype(np.float32)
    logits = rng.standard_normal((t, e)).astype(np.float32)
    for col, shift in (skew or {}).items():
        logits[:, col] += shift
    ids, w = M.router_topk(logits, k, M.SCORE_RAW, M.WEIGHT_SOFTMAX, False)
    ids_dev = ids.astype(np.int32)
    if pad_slot:
        ids_dev = ids_dev.copy()
        ids_dev[::7, -1] = -1
        w = w.copy()
        w[::7, -1] = 0.0
    da, dd = T.make_weight("MXFP4", rng, h, i, experts=e)
    if interleaved:
        gua, gud = T.make_weight("MXFP4", rng, 2 * i, h, experts=e)
        gub = (rng.standard_normal((e, 2 * i)) * 0.05).astype(np.float32)
        db = (rng.standard_normal((e, h)) * 0.05).astype(np.float32)
        experts = hq.MoEExperts(T.make_layer("MXFP4", da, i, DEV, T.to_dev(db, torch.float32, DEV)),
                                gate_up_proj=T.make_layer("MXFP4", gua, h, DEV, T.to_dev(gub, torch.float32, DEV)),
                                act=L.ACT_GPTOSS, limit=7.0, alpha=1.702)
    else:
        ga, gd = T.make_weight("MXFP4", rng, i, h, experts=e)
        ua, ud = T.make_weight("MXFP4", rng, i, h, experts=e)
        experts = hq.MoEExperts(T.make_layer("MXFP4", da, i, DEV), T.make_layer("MXFP4", ga, h, DEV),
                                T.make_layer("MXFP4", ua, h, DEV))
    xd = T.to_dev(x, torch.bfloat16, DEV)
    out = experts.forward_mx_act(xd, T.to_dev(w, torch.float32, DEV), torch.from_numpy(ids_dev).to(DEV),
                                 out_dtype=out_dtype or torch.float32)
    torch.cuda.synchronize()
    assert experts.down.device_status()[0] == 0
    x_used = _qdq(xd.to(torch.float32).cpu().numpy())
    if interleaved:
        want = M.moe_layer(x_used, ids, w, None, None, dd, act=M.ACT_GPTOSS, gate_up_bank=gud, gate_up_bias=gub,
                           down_bias=db, alpha=1.702, limit=7.0, h_round=_qdq)
    else:
        want = M.moe_layer(x_used, ids, w, gd, ud, dd, h_round=_qdq)
    return out.to(torch.float32).cpu().numpy(), want


def test_expert_block_interleaved_gate_up():
    # gpt-oss form: one bank whose rows interleave gate and up, biases, clamped activation; expert 0 holds more
    # than one 128-row tile, expert 5 is nearly empty
    got, want = _expert_block_case(8, 2, 512, 256, 300, 4, skew={0: 2.0, 5: -6.0})
    assert T.rel_l2(got, want) <= 2e-3


def test_expert_block_gpt_oss_width():
    # hidden = intermediate = 2880: 22 full K stages and one of 64 elements; 2 * 2880 = 5760 weight rows = 45 tiles
    got, want = _expert_block_case(4, 2, 2880, 2880, 48, 5, pad_slot=True)
    assert T.rel_l2(got, want) <= 2e-3


def test_expert_block_separate_gate_and_up():
    got, want = _expert_block_case(8, 2, 256, 384, 200, 6, interleaved=False)
    assert T.rel_l2(got, want) <= 2e-3


def test_expert_block_16_bit_rows():
    got, want = _expert_block_case(8, 2, 512, 256, 333, 7, out_dtype=torch.bfloat16)
    assert T.rel_l2(got, want) <= 2e-3 + 4.5e-3        # + two roundings to bf16 (rows, result)


def test_bounded_wait_runs_out_and_the_call_returns():
    """The copy-issuing warp is told to issue nothing (test hook), so no copy and no MMA is in flight; every other
    warp's first wait runs out after the (shortened) poll limit.  The call must return, report the time-out with
    the tag of the wait that gave up, and leave the output untouched."""
    import engine_b200 as hq
    from engine_b200 import _lib as L
    lib = L.lib()
    rng = T.rng_for(11, 8)
    arrays, _ = T.make_weight("MXFP4", rng, 256, 512)
    layer = T.make_layer("MXFP4", arrays, 512, DEV)
    x = rng.standard_normal((64, 512)).astype(np.float32)
    codes, scales = hq.mxfp8_quantize_rows(T.to_dev(x, torch.float32, DEV))
    old_spin, old_skip = lib.hq_config_get(L.CFG_SPIN_LIMIT), lib.hq_config_get(L.CFG_TEST_SKIP_PRODUCER)
    y = torch.full((64, 256), 7.0, dtype=torch.float32, device=DEV)
    try:
        lib.hq_config_set(L.CFG_SPIN_LIMIT, 64)
        lib.hq_config_set(L.CFG_TEST_SKIP_PRODUCER, 1)
        w = layer._weight_struct()
        rc = lib.hq_mx_linear_forward(C.byref(w), codes.data_ptr(), scales.data_ptr(), 64, y.data_ptr(), L.DT_F32,
                                      256, layer._status_buf(codes.device).data_ptr(),
                                      torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
    finally:
        lib.hq_config_set(L.CFG_SPIN_LIMIT, old_spin)
        lib.hq_config_set(L.CFG_TEST_SKIP_PRODUCER, old_skip)
    st = layer.device_status()
    assert st[0] == L.DEV_WAIT_TIMEOUT and 810 <= st[3] < 870, st
    assert bool((y == 7.0).all())              # nothing was stored
    layer._status.zero_()
    y2 = layer.forward_mx_rows(codes, scales, torch.float32)
    torch.cuda.synchronize()
    assert layer.device_status()[0] == 0
