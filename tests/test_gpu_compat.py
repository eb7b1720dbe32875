"""Reference-named entry points (include/hanzoquant_compat.h): each shim is called through ctypes with the
reference's argument order and compared with the hq_* result (same kernels behind both, so equality is exact
unless a path switch is stated)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

from oracle import moe as M
from tests import hq_testlib as T

DEV = "cuda:0"
P = C.c_void_p


def _lib():
    from engine_b200 import _lib as L
    return L.lib()


def _s():
    return P(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return P(t.data_ptr())


def test_dispatch_and_reduce_shims():
    import engine_b200 as hq
    lib = _lib()
    rng = T.rng_for(7, 1)
    t, k, e, h = 50, 4, 16, 256
    ids = torch.from_numpy(rng.integers(0, e, (t, k)).astype(np.int32)).to(DEV)
    tab = hq.moe_dispatch_build(ids, e)
    bounds = torch.empty(e + 1, dtype=torch.int32, device=DEV)
    sa = torch.empty(t * k, dtype=torch.int32, device=DEV)
    st = torch.empty(t * k, dtype=torch.int32, device=DEV)
    lib.launch_moe_dispatch(_p(ids), _p(bounds), _p(sa), _p(st), C.c_int32(t * k), C.c_int32(e), C.c_int32(k), None,
                            None, _s())
    torch.cuda.synchronize()
    assert torch.equal(bounds, tab.expert_bounds) and torch.equal(sa, tab.sorted_assign)
    assert torch.equal(st, tab.sorted_token)
    y = torch.from_numpy(rng.standard_normal((t * k, h)).astype(np.float32)).to(DEV)
    w = torch.from_numpy(rng.random((t, k)).astype(np.float32)).to(DEV)
    want = hq.moe_weighted_reduce(y, w, torch.float32)
    out = torch.empty((t, h), dtype=torch.float32, device=DEV)
    lib.launch_moe_weighted_reduce_flat(_p(y), _p(w), _p(out), C.c_int32(t), C.c_int32(h), C.c_int32(k), _s())
    out16 = torch.empty((t, h), dtype=torch.bfloat16, device=DEV)
    lib.launch_moe_weighted_reduce_flat_bf16(_p(y), _p(w), _p(out16), C.c_int32(t), C.c_int32(h), C.c_int32(k), _s())
    torch.cuda.synchronize()
    assert torch.equal(out, want)
    assert torch.equal(out16, hq.moe_weighted_reduce(y, w, torch.bfloat16))


@pytest.mark.parametrize("fmt,sym", [("Q8_0", "q8_0"), ("Q4_K", "q4_k"), ("Q6_K", "q6_k"), ("Q5_K", "q5_k"),
                                     ("Q4_0", "q4_0"), ("Q5_0", "q5_0"), ("Q4_1", "q4_1"), ("Q5_1", "q5_1"),
                                     ("Q2_K", "q2_k"), ("Q3_K", "q3_k")])
def test_q8_1_pair_runs_the_mat_vec_on_the_original_activations(fmt, sym):
    lib = _lib()
    rng = T.rng_for(7, 2)
    n, k, m = 512, 1024, 3
    arrays, deq = T.make_weight(fmt, rng, n, k)
    layer = T.make_layer(fmt, arrays, k, DEV)
    x = T.to_dev(rng.standard_normal((m, k)).astype(np.float32), torch.bfloat16, DEV)
    scratch = torch.empty(m * (k // 32) * 36, dtype=torch.uint8, device=DEV)     # what the reference would size
    out = torch.empty((m, n), dtype=torch.bfloat16, device=DEV)
    lib.launch_mmvq_gguf_quantize_q8_1_bf16(_p(x), _p(scratch), C.c_int32(k), C.c_int32(k), C.c_int32(m), _s())
    getattr(lib, f"launch_mmvq_gguf_{sym}_bf16_plain")(_p(layer.data), _p(scratch), _p(out), C.c_int32(k),
                                                      C.c_int32(n), C.c_int32(k // 32), C.c_int32(n), C.c_int32(m),
                                                      _s())
    torch.cuda.synchronize()
    assert torch.equal(out, layer.forward_raw(x, torch.bfloat16))
    want = M.dense_forward(x.to(torch.float32).cpu().numpy(), deq)
    assert T.rel_l2(out.to(torch.float32).cpu().numpy(), want) <= 5e-3      # bf16 output rounding


def test_indexed_moe_forward_q4k_shim():
    import engine_b200 as hq
    lib = _lib()
    rng = T.rng_for(7, 3)
    e, n, k, t, topk = 6, 256, 512, 9, 2
    arrays, deq = T.make_weight("Q4_K", rng, n, k, experts=e)
    bank = T.make_layer("Q4_K", arrays, k, DEV)
    x = T.to_dev(rng.standard_normal((t, k)).astype(np.float32), torch.float32, DEV)
    ids = torch.from_numpy(rng.integers(0, e, (t, topk)).astype(np.int32)).to(DEV)
    scratch = torch.empty(64, dtype=torch.uint8, device=DEV)
    out = torch.empty((t, topk, n), dtype=torch.float32, device=DEV)
    lib.launch_quantize_q8_1(_p(x), _p(scratch), C.c_int32(k), C.c_int32(k), C.c_int32(k // 32), C.c_int32(t), _s())
    lib.launch_indexed_moe_forward_q4k_q8_1(_p(bank.data), _p(scratch), _p(ids), _p(out), C.c_int32(n), C.c_int32(k),
                                            C.c_int32(t), C.c_int32(topk), C.c_int32(k), C.c_int32(1), _s())
    torch.cuda.synchronize()
    want = M.gather_forward(x.cpu().numpy(), ids.cpu().numpy().astype(np.uint32), deq)
    assert T.rel_l2(out.cpu().numpy(), want) <= 1e-3


def test_fp8_shims():
    import engine_b200 as hq
    lib = _lib()
    rng = T.rng_for(7, 4)
    e, n, k, t, topk = 4, 256, 512, 7, 2
    arrays, deq = T.make_weight("FP8", rng, n, k, experts=e)
    bank = T.make_layer("FP8", arrays, k, DEV)
    x = T.to_dev(rng.standard_normal((t, k)).astype(np.float32), torch.bfloat16, DEV)
    ids = torch.from_numpy(rng.integers(0, e, (t, topk)).astype(np.int32)).to(DEV)
    out = torch.empty((t, topk, n), dtype=torch.bfloat16, device=DEV)
    lib.launch_fp8_indexed_moe_gemm_bf16(_p(x), _p(bank.weight), _p(bank.scale), _p(ids), _p(out), C.c_int32(t),
                                         C.c_int32(topk), C.c_int32(e), C.c_int32(n), C.c_int32(k), C.c_int32(k // 128),
                                         C.c_int32(128), C.c_int32(128), C.c_bool(False), _s())
    torch.cuda.synchronize()
    assert torch.equal(out, bank.gather_forward(x, ids))
    dense = bank._expert_view(1)
    y = torch.empty((t, n), dtype=torch.bfloat16, device=DEV)
    lib.launch_fp8_matmul_bf16(_p(x), _p(dense.weight), _p(dense.scale), _p(y), C.c_int32(t), C.c_int32(n), C.c_int32(k),
                               C.c_int32(k // 128), C.c_int32(128), C.c_int32(128), _s())
    torch.cuda.synchronize()
    assert torch.equal(y, dense.forward(x))
    # quantizers
    v = T.to_dev(rng.standard_normal(1024).astype(np.float32), torch.float32, DEV)
    codes = torch.empty(1024, dtype=torch.uint8, device=DEV)
    scales = torch.empty(8, dtype=torch.float32, device=DEV)
    lib.launch_quant_fp8_vector_kernel_f32(_p(v), _p(codes), _p(scales), C.c_size_t(1024), _s())
    back = torch.empty(1024, dtype=torch.float32, device=DEV)
    lib.launch_dequant_fp8_vector_kernel_f32(_p(codes), _p(scales), _p(back), C.c_size_t(1024), _s())
    torch.cuda.synchronize()
    c2, s2 = hq.fp8_vector_quantize(v)
    assert torch.equal(codes, c2) and torch.equal(scales, s2)
    assert torch.equal(back, hq.fp8_vector_dequantize(c2, s2, torch.float32))
    wm = T.to_dev(rng.standard_normal((256, 384)).astype(np.float32), torch.float32, DEV)
    bc = torch.empty((256, 384), dtype=torch.uint8, device=DEV)
    bs = torch.empty((2, 3), dtype=torch.float32, device=DEV)
    lib.launch_quant_fp8_blockwise_kernel_f32(_p(wm), _p(bc), _p(bs), C.c_int32(256), C.c_int32(384), C.c_int32(384),
                                              C.c_int32(3), C.c_int32(128), C.c_int32(128), _s())
    torch.cuda.synchronize()
    c3, s3 = hq.fp8_blockwise_quantize(wm)
    assert torch.equal(bc, c3) and torch.equal(bs, s3)


def test_mxfp4_router_and_activation_shims():
    import engine_b200 as hq
    from engine_b200 import _lib as L
    lib = _lib()
    rng = T.rng_for(7, 5)
    e, n, k, t, topk = 4, 128, 256, 5, 2
    arrays, deq = T.make_weight("MXFP4", rng, n, k, experts=e)
    bias = torch.from_numpy(rng.standard_normal((e, n)).astype(np.float32)).to(DEV).to(torch.bfloat16)
    bank = T.make_layer("MXFP4", arrays, k, DEV, bias)
    x = T.to_dev(rng.standard_normal((t, k)).astype(np.float32), torch.bfloat16, DEV)
    ids = torch.from_numpy(rng.integers(0, e, (t, topk)).astype(np.int32)).to(DEV)
    for sym in ("launch_mxfp4_indexed_moe_gemm_bf16", "launch_mxfp4_moe_grouped_gemm_bf16",
                "launch_mxfp4_moe_grouped_gemm_wmma_bf16"):
        out = torch.empty((t, topk, n), dtype=torch.bfloat16, device=DEV)
        getattr(lib, sym)(_p(x), _p(bank.blocks), _p(bank.scales), _p(bias), _p(ids), _p(out), C.c_int32(t),
                          C.c_int32(topk), C.c_int32(e), C.c_int32(n), C.c_int32(k), C.c_bool(True), C.c_bool(False),
                          _s())
        torch.cuda.synchronize()
        assert torch.equal(out, bank.gather_forward(x, ids)), sym
    lib.mxfp4_get_max_smem_optin.restype = C.c_int32
    assert lib.mxfp4_get_max_smem_optin() >= 200 * 1024
    # router
    logits = T.to_dev(rng.standard_normal((33, 64)).astype(np.float32), torch.float32, DEV)
    want = hq.moe_router_topk(logits, hq.MoeRouterTopKConfig(6, L.SCORE_SOFTMAX, L.WEIGHT_SCORE, True))
    w = torch.empty((33, 6), dtype=torch.float32, device=DEV)
    i = torch.empty((33, 6), dtype=torch.int32, device=DEV)
    lib.moe_router_topk_f32(_p(logits), _p(w), _p(i), None, None, C.c_int32(33), C.c_int32(64), C.c_int32(6),
                            C.c_int32(L.SCORE_SOFTMAX), C.c_int32(L.WEIGHT_SCORE), C.c_bool(True), C.c_bool(False),
                            C.c_float(0), C.c_float(0), C.c_float(0), C.c_float(1.0),
                            C.c_int64(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert torch.equal(i, want.indices) and torch.equal(w, want.values)
    # activations
    gu = T.to_dev(rng.standard_normal((10, 64, 2)).astype(np.float32), torch.float32, DEV)
    o = torch.empty((10, 64), dtype=torch.float32, device=DEV)
    lib.gptoss_swiglu_interleaved_f32(_p(gu), _p(o), C.c_uint32(10), C.c_uint32(64), C.c_float(1.702), C.c_float(7.0),
                                      _s())
    a, b = gu[..., 0].contiguous(), gu[..., 1].contiguous()
    o2 = torch.empty((10, 64), dtype=torch.float32, device=DEV)
    lib.fused_glu_f32(_p(a), _p(b), _p(o2), C.c_uint32(640), C.c_int32(0), _s())
    torch.cuda.synchronize()
    assert torch.equal(o, hq.gated_act(gu, None, L.ACT_GPTOSS, 7.0, 1.702, interleaved=True))
    assert torch.equal(o2, hq.gated_act(a, b, L.ACT_SWIGLU))
