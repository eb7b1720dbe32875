"""Fused dense decode set: gate+up GLU in one launch, the three attention projections in one call, and the
unquantized mat-vec, each against the oracle (hanzo-quant/src/lib.rs:1116-1204, gemv/mod.rs)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

from oracle import moe as M
from tests import hq_testlib as T

DEV = "cuda:0"


@pytest.mark.parametrize("fmt,tol", [("Q8_0", 1e-3), ("Q4_K", 1e-3), ("FP8", 2e-3), ("MXFP4", 2e-3)])
@pytest.mark.parametrize("m", [1, 5, 8])
def test_fused_gate_up_decode(fmt, tol, m):
    import engine_b200 as hq
    rng = T.rng_for(6, 1)
    n, k = 1536, 2048
    ga, gd = T.make_weight(fmt, rng, n, k)
    ua, ud = T.make_weight(fmt, rng, n, k)
    gate, up = T.make_layer(fmt, ga, k, DEV), T.make_layer(fmt, ua, k, DEV)
    x = T.to_dev(rng.standard_normal((m, k)).astype(np.float32), torch.bfloat16, DEV)
    y = hq.try_fused_quantized_gate_up(x, gate, up, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert gate.device_status()[0] == 0
    xf = x.to(torch.float32).cpu().numpy()
    want = M.swiglu(M.dense_forward(xf, gd), M.dense_forward(xf, ud))
    assert T.rel_l2(y.cpu().numpy(), want) <= tol
    # and it equals the two separate projections followed by the activation kernel's arithmetic
    g = gate.forward_raw(x, torch.float32)
    u = up.forward_raw(x, torch.float32)
    sep = (g / (1 + torch.exp(-g))) * u
    assert T.rel_l2(y.cpu().numpy(), sep.cpu().numpy()) <= 1e-5


def test_fused_gate_up_prefill_rows_take_the_tensor_cores():
    import engine_b200 as hq
    rng = T.rng_for(6, 2)
    n, k, m = 1024, 2048, 200
    ga, gd = T.make_weight("Q4_K", rng, n, k)
    ua, ud = T.make_weight("Q4_K", rng, n, k)
    gate, up = T.make_layer("Q4_K", ga, k, DEV), T.make_layer("Q4_K", ua, k, DEV)
    x = T.to_dev(rng.standard_normal((m, k)).astype(np.float32), torch.bfloat16, DEV)
    y = hq.try_fused_quantized_gate_up(x, gate, up, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert gate.device_status()[0] == 0
    xf = x.to(torch.float32).cpu().numpy()
    want = M.swiglu(M.dense_forward(xf, gd), M.dense_forward(xf, ud))
    assert T.rel_l2(y.cpu().numpy(), want) <= 1e-3


def test_fused_gate_up_declines_what_the_reference_declines():
    import engine_b200 as hq
    rng = T.rng_for(6, 3)
    a, _ = T.make_weight("Q8_0", rng, 256, 512)
    b, _ = T.make_weight("Q4_K", rng, 256, 512)
    x = T.to_dev(rng.standard_normal((1, 512)).astype(np.float32), torch.bfloat16, DEV)
    assert hq.try_fused_quantized_gate_up(x, T.make_layer("Q8_0", a, 512, DEV), T.make_layer("Q4_K", b, 512, DEV)) is None
    bias = torch.zeros(256, dtype=torch.bfloat16, device=DEV)
    assert hq.try_fused_quantized_gate_up(x, T.make_layer("Q8_0", a, 512, DEV, bias),
                                          T.make_layer("Q8_0", a, 512, DEV)) is None


def test_fused_qkv():
    import engine_b200 as hq
    rng = T.rng_for(6, 4)
    k = 2048
    shapes = (2048, 512, 512)        # grouped-query attention: fewer key / value heads
    layers, deqs = [], []
    for n in shapes:
        a, d = T.make_weight("Q8_0", rng, n, k)
        layers.append(T.make_layer("Q8_0", a, k, DEV))
        deqs.append(d)
    x = T.to_dev(rng.standard_normal((3, k)).astype(np.float32), torch.bfloat16, DEV)
    outs = hq.try_fused_quantized_qkv(x, *layers, out_dtype=torch.float32)
    torch.cuda.synchronize()
    xf = x.to(torch.float32).cpu().numpy()
    for o, d, layer in zip(outs, deqs, layers):
        assert T.rel_l2(o.cpu().numpy(), M.dense_forward(xf, d)) <= 1e-3
        assert torch.equal(o, layer.forward_raw(x, torch.float32))


@pytest.mark.parametrize("wdt", ["bfloat16", "float16", "float32"])
@pytest.mark.parametrize("m", [1, 3, 8])
def test_unquantized_gemv(wdt, m):
    import engine_b200 as hq
    rng = T.rng_for(6, 5)
    n, k = 1000, 4104          # rows that are not a multiple of the block's 16, K with a partial chunk
    w = torch.from_numpy(rng.normal(0, 0.02, (n, k)).astype(np.float32)).to(DEV).to(getattr(torch, wdt))
    bias = torch.from_numpy(rng.standard_normal(n).astype(np.float32)).to(DEV).to(getattr(torch, wdt))
    x = T.to_dev(rng.standard_normal((m, k)).astype(np.float32), torch.bfloat16, DEV)
    assert hq.should_use_gemv(x, w)
    y = hq.gemv(x, w, bias, out_dtype=torch.float32)
    torch.cuda.synchronize()
    want = M.dense_forward(x.to(torch.float32).cpu().numpy(), w.to(torch.float32).cpu().numpy(),
                           bias.to(torch.float32).cpu().numpy())
    assert T.rel_l2(y.cpu().numpy(), want) <= 1e-5
    assert not hq.should_use_gemv(torch.zeros((9, k), device=DEV), w)
