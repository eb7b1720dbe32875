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


def _expert_block_case(e, k, h, i, t, seed, skew=None, out_dtype=None, pad_slot=False):
    import engine_b200 as hq
    rng = T.rng_for(9, seed)
    ga, gd = T.make_weight("FP8", rng, i, h, experts=e)
    ua, ud = T.make_weight("FP8", rng, i, h, experts=e)
    da, dd = T.make_weight("FP8", rng, h, i, experts=e)
    experts = hq.MoEExperts(T.make_layer("FP8", da, i, DEV), T.make_layer("FP8", ga, h, DEV),
                            T.make_layer("FP8", ua, h, DEV))
    x = rng.standard_normal((t, h)).astype(np.float32)
    logits = rng.standard_normal((t, e)).astype(np.float32)
    for col, shift in (skew or {}).items():
        logits[:, col] += shift
    ids, w = M.router_topk(logits, k, M.SCORE_SOFTMAX, M.WEIGHT_SCORE, True)
    ids_dev = ids.astype(np.int32)
    if pad_slot:                              # a padding slot (id -1) contributes nothing
        ids_dev = ids_dev.copy()
        ids_dev[::7, -1] = -1
        w = w.copy()
        w[::7, -1] = 0.0
    xd = T.to_dev(x, torch.bfloat16, DEV)
    out = experts.forward_fp8_act(xd, T.to_dev(w, torch.float32, DEV), torch.from_numpy(ids_dev).to(DEV),
                                  out_dtype=out_dtype or torch.float32)
    torch.cuda.synchronize()
    assert experts.gate.device_status()[0] == 0
    x_used = _qdq(xd.to(torch.float32).cpu().numpy())
    f16 = lambda a: a.astype(np.float16).astype(np.float32)
    # gate and up rounded to f16, the activated product rounded to f16, then the 1x128 quantizer: the kernel's
    # rounding points (the reference's gather route rounds the same three values to the activation dtype,
    # hanzo-quant/kernels/ops/ops.cu:845-858)
    want = M.moe_layer(x_used, ids, w, gd, ud, dd, h_round=lambda a: _qdq(f16(a)), gu_round=f16)
    return out.to(torch.float32).cpu().numpy(), want


def test_expert_block_with_fp8_activations():
    # uneven experts: expert 0 holds more than one 144-row tile, expert 5 is nearly empty
    got, want = _expert_block_case(8, 2, 1024, 512, 300, 3, skew={0: 2.0, 5: -6.0})
    assert T.rel_l2(got, want) <= 2e-3


def test_expert_block_tile_edges_and_padding_slots():
    # 2 experts, top-1, logits pushed so that expert 0 gets 145 of 160 rows (two tiles of 80) and expert 1 the
    # rest; a padding slot every 7th token
    got, want = _expert_block_case(4, 2, 512, 512, 160, 4, skew={0: 3.0, 3: -8.0}, pad_slot=True)
    assert T.rel_l2(got, want) <= 2e-3


@pytest.mark.parametrize("dt", ["bfloat16", "float16"])
def test_expert_block_16_bit_rows(dt):
    # 16-bit output: the down projection's rows leave through the shared-memory transpose as 16-bit values
    out_dtype = getattr(torch, dt)
    got, want = _expert_block_case(8, 2, 512, 512, 333, 5, out_dtype=out_dtype)
    tol = 2e-3 + (4.5e-3 if dt == "bfloat16" else 6e-4)     # + two roundings of the output dtype (rows, result)
    assert T.rel_l2(got, want) <= tol


def test_bounded_wait_runs_out_and_the_call_returns():
    """The copy-issuing warp is told to issue nothing (test hook), so no copy and no MMA is in flight; every other
    warp's first wait runs out after the (shortened) poll limit.  The call must return, report the time-out with
    the tag of the wait that gave up, and leave the output untouched."""
    import engine_b200 as hq
    from engine_b200 import _lib as L
    lib = L.lib()
    rng = T.rng_for(9, 6)
    arrays, _ = T.make_weight("FP8", rng, 256, 512)
    layer = T.make_layer("FP8", arrays, 512, DEV)
    x = rng.standard_normal((64, 512)).astype(np.float32)
    codes, scales = hq.fp8_quantize_rows(T.to_dev(x, torch.float32, DEV))
    old_spin, old_skip = lib.hq_config_get(L.CFG_SPIN_LIMIT), lib.hq_config_get(L.CFG_TEST_SKIP_PRODUCER)
    y = torch.full((64, 256), 7.0, dtype=torch.float32, device=DEV)
    try:
        lib.hq_config_set(L.CFG_SPIN_LIMIT, 64)
        lib.hq_config_set(L.CFG_TEST_SKIP_PRODUCER, 1)
        w = layer._weight_struct()
        import ctypes as C
        rc = lib.hq_fp8_linear_forward(C.byref(w), codes.data_ptr(), scales.data_ptr(), 64, y.data_ptr(), L.DT_F32,
                                       256, layer._status_buf(codes.device).data_ptr(),
                                       torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
    finally:
        lib.hq_config_set(L.CFG_SPIN_LIMIT, old_spin)
        lib.hq_config_set(L.CFG_TEST_SKIP_PRODUCER, old_skip)
    st = layer.device_status()
    assert st[0] == L.DEV_WAIT_TIMEOUT and 720 <= st[3] < 770, st
    assert bool((y == 7.0).all())              # nothing was stored
    layer._status.zero_()
    # and the same layer works again afterwards
    y2 = layer.forward_fp8_rows(codes, scales, torch.float32)
    torch.cuda.synchronize()
    assert layer.device_status()[0] == 0
    assert bool(torch.isfinite(y2).all())
