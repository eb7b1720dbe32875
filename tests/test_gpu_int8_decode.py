"""The Q8_0 / Q4_K decode kernel on the integer MMA: split K through the caller's scratch, the two-term int8
activations (outliers, f32 / f16 / bf16 input, non-finite input), against the dequantize-then-matmul oracle.
Tolerance as for every GGUF case: rel-L2 <= 1e-3 of the f32 output."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

from oracle import moe as M
from tests import hq_testlib as T

DEV = "cuda:0"


def _layer(fmt, n, k, seed):
    rng = T.rng_for(7, seed)
    arrays, deq = T.make_weight(fmt, rng, n, k)
    return T.make_layer(fmt, arrays, k, DEV), deq, rng


@pytest.mark.parametrize("fmt", ["Q8_0", "Q4_K"])
@pytest.mark.parametrize("m", [1, 5, 8, 11])
def test_long_k_takes_the_split_and_matches(fmt, m):
    # K = 14336 does not fit beside the ring: with the layer's scratch the kernel splits K across CTAs
    if fmt == "Q4_K" and m > 8:
        pytest.skip("Q4_K with more than 8 rows runs on the tensor-core kernel, not the decode kernel")
    from engine_b200 import _lib as L
    n, k = 1000, 14336
    layer, deq, rng = _layer(fmt, n, k, 1)
    x = T.to_dev(rng.standard_normal((m, k)).astype(np.float32), torch.bfloat16, DEV)
    w = layer._weight_struct()
    assert L.lib().hq_linear_workspace_bytes(C.byref(w), m) > 0
    y = layer.forward_raw(x, torch.float32)
    torch.cuda.synchronize()
    assert layer.device_status()[0] == 0
    want = M.dense_forward(x.to(torch.float32).cpu().numpy(), deq, None)
    assert T.rel_l2(y.cpu().numpy(), want) <= 1e-3
    # every call leaves the arrival counters (the first 1024 bytes of the scratch) at zero, and a second call
    # gives the same bits
    for buf in layer._ws.values():
        assert int(buf[:1024].count_nonzero()) == 0
    y2 = layer.forward_raw(x, torch.float32)
    assert torch.equal(y, y2)
    # without a scratch the same call runs unsplit and agrees within the tolerance
    y3 = torch.empty_like(y)
    rc = L.lib().hq_linear_forward(C.byref(w), x.data_ptr(), L.DT_BF16, k, y3.data_ptr(), L.DT_F32, n, m, None,
                                   torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert T.rel_l2(y3.cpu().numpy(), want) <= 1e-3


@pytest.mark.parametrize("fmt", ["Q8_0", "Q4_K"])
@pytest.mark.parametrize("x_dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_activation_dtypes_and_outliers(fmt, x_dtype):
    # one activation per row a thousand times the rest: the step of its 128- or 256-element group is coarse, the
    # error it causes stays far below what the outlier itself contributes
    n, k, m = 256, 2048, 6
    layer, deq, rng = _layer(fmt, n, k, 2)
    x = rng.standard_normal((m, k)).astype(np.float32)
    x[np.arange(m), rng.integers(0, k, m)] *= 1000.0
    xd = T.to_dev(x, x_dtype, DEV)
    y = layer.forward_raw(xd, torch.float32)
    want = M.dense_forward(xd.to(torch.float32).cpu().numpy(), deq, None)
    assert T.rel_l2(y.cpu().numpy(), want) <= 1e-3
    # tiny and zero activations
    x2 = (rng.standard_normal((m, k)) * 1e-20).astype(np.float32)
    x2[0] = 0.0
    xd2 = T.to_dev(x2, torch.float32, DEV)
    y2 = layer.forward_raw(xd2, torch.float32).cpu().numpy()
    want2 = M.dense_forward(x2, deq, None)
    assert np.all(y2[0] == 0.0)
    assert T.rel_l2(y2[1:], want2[1:]) <= 1e-3


@pytest.mark.parametrize("fmt", ["Q8_0", "Q4_K"])
def test_non_finite_activations_do_not_turn_finite(fmt):
    n, k = 64, 1024
    layer, deq, rng = _layer(fmt, n, k, 3)
    x = rng.standard_normal((3, k)).astype(np.float32)
    x[0, 17] = np.nan
    x[1, 900] = np.inf
    y = layer.forward_raw(T.to_dev(x, torch.float32, DEV), torch.float32).cpu().numpy()
    assert np.all(~np.isfinite(y[0])) and np.all(~np.isfinite(y[1]))
    want = M.dense_forward(x[2:3], deq, None)
    assert T.rel_l2(y[2:3], want) <= 1e-3


def test_one_hot_rows_pass_exactly():
    # power-of-two steps: a row with a single 1.0 reads one weight column back without any rounding
    for fmt in ["Q8_0", "Q4_K"]:
        n, k = 128, 512
        layer, deq, rng = _layer(fmt, n, k, 4)
        x = np.zeros((4, k), dtype=np.float32)
        cols = [0, 31, 255, 511]
        x[np.arange(4), cols] = 1.0
        y = layer.forward_raw(T.to_dev(x, torch.bfloat16, DEV), torch.float32).cpu().numpy()
        assert np.array_equal(y, deq[:, cols].T.astype(np.float32)), fmt


@pytest.mark.parametrize("m", [1, 2])
@pytest.mark.parametrize("x_dtype", [torch.float32, torch.bfloat16])
def test_fp8_one_and_two_rows_on_the_fp8_warp_mma(m, x_dtype):
    # block-FP8 with one or two activation rows: e4m3 weights unconverted, activations as three e4m3 terms;
    # K = 7168 is too long to stay staged, so the layer's scratch brings in the K split as well
    n, k = 512, 7168
    layer, deq, rng = _layer("FP8", n, k, 5)
    x = rng.standard_normal((m, k)).astype(np.float32)
    x[0, 100] *= 300.0
    xd = T.to_dev(x, x_dtype, DEV)
    y = layer.forward_raw(xd, torch.float32)
    torch.cuda.synchronize()
    assert layer.device_status()[0] == 0
    want = M.dense_forward(xd.to(torch.float32).cpu().numpy(), deq, None)
    assert T.rel_l2(y.cpu().numpy(), want) <= 2e-3
    assert torch.equal(y, layer.forward_raw(xd, torch.float32))
    x[m - 1, 5] = np.nan
    y2 = layer.forward_raw(T.to_dev(x, torch.float32, DEV), torch.float32).cpu().numpy()
    assert np.all(~np.isfinite(y2[m - 1]))
