"""Edge values: activations beyond the f16 range, MXFP4 exponents outside the range the f16-expanding tensor path
takes, FP8 quantizer groups with a tiny absmax, and NaN router logits."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

from oracle import formats as F
from oracle import moe as M
from tests import hq_testlib as T

DEV = "cuda:0"


def test_values_beyond_f16_are_clamped_and_flagged():
    """The tensor-core paths multiply in f16 (the reference feeds its kernels bf16 / f32 and has no such limit): a
    finite value beyond +-65504 is clamped by the conversion and HQ_DEV_F16_RANGE is left in the status word."""
    import engine_b200 as hq
    from engine_b200 import _lib as L
    from engine_b200.quant import convert
    x = torch.randn((4, 256), device=DEV).to(torch.bfloat16)
    x[2, 17] = 1.0e5
    x[3, 5] = -3.0e6
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    y = convert(x, torch.float16, status)
    torch.cuda.synchronize()
    assert int(status[0]) == L.DEV_F16_RANGE
    assert float(y[2, 17]) == 65504.0 and float(y[3, 5]) == -65504.0
    assert bool(torch.isfinite(y).all())
    keep = torch.ones_like(x, dtype=torch.bool)
    keep[2, 17] = keep[3, 5] = False
    assert torch.equal(y[keep], x.to(torch.float16)[keep])
    # in range: no flag
    status.zero_()
    convert(x.clamp(-100, 100), torch.float16, status)
    torch.cuda.synchronize()
    assert int(status[0]) == 0


def test_prefill_layer_reports_the_f16_limit():
    import engine_b200 as hq
    from engine_b200 import _lib as L
    n, k, m = 256, 512, 64
    rng = T.rng_for(12, 1)
    arrays, deq = T.make_weight("Q4_K", rng, n, k)
    layer = T.make_layer("Q4_K", arrays, k, DEV)
    x = rng.standard_normal((m, k)).astype(np.float32)
    x[7, 3] = 1.0e5
    y = layer.forward_raw(T.to_dev(x, torch.bfloat16, DEV), torch.float32)
    torch.cuda.synchronize()
    assert layer.device_status()[0] == L.DEV_F16_RANGE
    assert bool(torch.isfinite(y).all())
    # every other row is unaffected
    xb = T.to_dev(x, torch.bfloat16, DEV).to(torch.float32).cpu().numpy()
    want = M.dense_forward(xb, deq, None)
    rows = [r for r in range(m) if r != 7]
    assert T.rel_l2(y.cpu().numpy()[rows], want[rows]) <= 1e-3


def _mxfp4_with_extreme_exponents(rng, n, k):
    w = rng.normal(0.0, 0.02, (n, k)).astype(np.float32)
    b, s = F.mxfp4_quantize(w)
    s = s.copy()
    s[3, 1] = 100       # 2^-27: below what the f16 expansion can carry
    s[9, 0] = 150       # 2^23: above it
    return b, s


def test_mxfp4_extreme_exponents_decode_and_block_scaled_paths_are_exact():
    """e8m0 exponents 100 and 150 are valid.  The decode kernel applies 2^(e-127) in f32 and the block-scaled MMA
    takes the exponent as it is; both must agree with the oracle."""
    import engine_b200 as hq
    n, k = 128, 256
    rng = T.rng_for(12, 2)
    b, s = _mxfp4_with_extreme_exponents(rng, n, k)
    deq = F.mxfp4_dequant(b, s)
    layer = T.make_layer("MXFP4", {"blocks": b, "scales": s}, k, DEV)
    x = rng.standard_normal((1, k)).astype(np.float32)
    y = layer.forward_raw(T.to_dev(x, torch.float32, DEV), torch.float32)
    torch.cuda.synchronize()
    assert layer.device_status()[0] == 0
    assert T.rel_l2(y.cpu().numpy(), M.dense_forward(x, deq, None)) <= 2e-3
    xm = rng.standard_normal((40, k)).astype(np.float32)
    codes, scales = hq.mxfp8_quantize_rows(T.to_dev(xm, torch.float32, DEV))
    ym = layer.forward_mx_rows(codes, scales, torch.float32)
    torch.cuda.synchronize()
    assert layer.device_status()[0] == 0
    xq = F.mxfp8_dequant(*F.mxfp8_quant(xm)).astype(np.float32)
    assert T.rel_l2(ym.cpu().numpy(), M.dense_forward(xq, deq, None)) <= 1e-5


def test_mxfp4_extreme_exponents_are_reported_by_the_f16_expanding_path():
    """The prefill path with 16-bit activations expands e2m1 x 2^(e-127) to f16 and takes exponents 113..140 (and
    0); a block outside that range is expanded as zero and HQ_DEV_SCALE_RANGE is left in the status word."""
    from engine_b200 import _lib as L
    n, k, m = 128, 256, 64
    rng = T.rng_for(12, 2)
    b, s = _mxfp4_with_extreme_exponents(rng, n, k)
    layer = T.make_layer("MXFP4", {"blocks": b, "scales": s}, k, DEV)
    x = rng.standard_normal((m, k)).astype(np.float32)
    y = layer.forward_raw(T.to_dev(x, torch.float16, DEV), torch.float32)
    torch.cuda.synchronize()
    assert layer.device_status()[0] == L.DEV_SCALE_RANGE
    # rows without an out-of-range block are unaffected
    deq = F.mxfp4_dequant(b, s)
    xh = x.astype(np.float16).astype(np.float32)
    want = M.dense_forward(xh, deq, None)
    cols = [c for c in range(n) if c not in (3, 9)]
    assert T.rel_l2(y.cpu().numpy()[:, cols], want[:, cols]) <= 2e-3


def test_fp8_quantizer_groups_with_tiny_absmax():
    """scale = absmax / 448 for every absmax > 0 (the reference's CPU rule, hanzo-quant/src/vector_fp8/ops.rs:235-287;
    its CUDA kernel clamps the scale at 1e-12 instead): groups with absmax 1e-11, 1e-20 and a denormal."""
    import engine_b200 as hq
    rng = T.rng_for(12, 3)
    x = rng.standard_normal((6, 256)).astype(np.float32)
    x[0] *= 1e-11
    x[1] *= 1e-20
    x[2] *= 1e-38
    x[3, :128] = 0.0
    x[4, 130] = 0.0
    codes, scales = hq.fp8_quantize_rows(T.to_dev(x, torch.float32, DEV))
    want_c, want_s = F.fp8_vector_quant(x.reshape(-1), 128)
    assert np.array_equal(scales.cpu().numpy().reshape(-1), want_s)
    assert np.array_equal(codes.cpu().numpy().reshape(-1), want_c)


def test_nan_logits_are_never_preferred():
    """A NaN score is ordered last (as -inf), in the kernel and in the oracle alike; ids stay bit-exact."""
    import engine_b200 as hq
    from engine_b200 import _lib as L
    rng = T.rng_for(12, 4)
    lg = rng.standard_normal((33, 16)).astype(np.float32)
    lg[::3, 5] = np.nan
    lg[1, :] = np.nan
    lg[1, 2] = 0.5
    cfg = hq.MoeRouterTopKConfig(4, L.SCORE_RAW, L.WEIGHT_SOFTMAX, False)
    top = hq.moe_router_topk(T.to_dev(lg, torch.float32, DEV), cfg)
    torch.cuda.synchronize()
    ids, _ = M.router_topk(lg, 4, M.SCORE_RAW, M.WEIGHT_SOFTMAX, False)
    assert np.array_equal(top.indices.cpu().numpy().astype(np.uint32), ids)
    rows = np.arange(0, 33, 3)
    rows = rows[rows != 1]
    assert not (top.indices.cpu().numpy()[rows] == 5).any()
