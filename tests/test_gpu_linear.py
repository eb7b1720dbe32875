"""Dense quantized linear (QuantMethod::forward) against the dequantize-then-matmul oracle, through the C ABI.
Tolerances (rel-L2 of the f32-output kernel vs the unrounded oracle): GGUF 1e-3, FP8 / MXFP4 2e-3."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

from oracle import formats as F
from oracle import moe as M
from tests import hq_testlib as T

TOL = {"Q8_0": 1e-3, "Q4_K": 1e-3, "Q6_K": 1e-3, "Q5_K": 1e-3, "Q4_0": 1e-3, "Q5_0": 1e-3, "Q4_1": 1e-3, "Q5_1": 1e-3,
       "Q2_K": 1e-3, "Q3_K": 1e-3, "FP8": 2e-3, "MXFP4": 2e-3}
FURTHER = ["Q5_K", "Q4_0", "Q5_0", "Q4_1", "Q5_1", "Q2_K", "Q3_K"]     # the GGML types beyond Q8_0 / Q4_K / Q6_K
DEV = "cuda:0"


def run_case(fmt, n, k, m, x_dtype, out_dtype, seed, bias=False):
    rng = T.rng_for(1, seed)
    arrays, deq = T.make_weight(fmt, rng, n, k)
    x = rng.standard_normal((m, k)).astype(np.float32)
    xd = T.to_dev(x, x_dtype, DEV)
    x_used = xd.to(torch.float32).cpu().numpy()
    b = bd = None
    if bias:
        b = rng.normal(0, 0.02, n).astype(np.float32)
        bd = T.to_dev(b, torch.bfloat16, DEV)
        b = bd.to(torch.float32).cpu().numpy()
    layer = T.make_layer(fmt, arrays, k, DEV, bd)
    y = layer.forward_raw(xd, out_dtype)
    torch.cuda.synchronize()
    assert layer.device_status()[0] == 0
    want = M.dense_forward(x_used, deq, b)
    return y.to(torch.float32).cpu().numpy(), want


@pytest.mark.parametrize("fmt", ["Q8_0", "Q4_K", "Q6_K"] + FURTHER + ["FP8", "MXFP4"])
@pytest.mark.parametrize("m", [1, 2, 4, 8])
def test_decode_rows_f32_out(fmt, m):
    got, want = run_case(fmt, 512, 1024, m, torch.bfloat16, torch.float32, 10 + m)
    assert T.rel_l2(got, want) <= TOL[fmt]


@pytest.mark.parametrize("fmt,n,k", [("Q8_0", 4096, 4096), ("Q4_K", 4096, 4096), ("Q8_0", 1000, 14336),
                                     ("FP8", 2048, 7168), ("MXFP4", 5760, 2880), ("Q4_K", 2048, 768),
                                     ("Q6_K", 2048, 768), ("Q6_K", 1000, 4096),
                                     # rows staged four 256-weight spans at a time: a last stretch of one span
                                     # (K = 1280, 2304) and rows that start 2, 4, .. 14 bytes off a 16-byte boundary
                                     ("Q6_K", 520, 1280), ("Q5_0", 520, 1280), ("Q4_0", 1000, 4096),
                                     ("Q5_K", 520, 2304),
                                     # Q2_K rows of 420 bytes (4-byte aligned), Q3_K rows of 550 (2-byte aligned)
                                     ("Q2_K", 520, 1280), ("Q3_K", 520, 1280), ("Q4_1", 520, 1280), ("Q5_1", 520, 1280),
                                     ("Q2_K", 1000, 4096), ("Q3_K", 1000, 4096)])
def test_model_shapes(fmt, n, k):
    got, want = run_case(fmt, n, k, 3, torch.bfloat16, torch.float32, 20, bias=(fmt == "MXFP4"))
    assert T.rel_l2(got, want) <= TOL[fmt]


@pytest.mark.parametrize("m", [1, 16, 128])
def test_q4_k_config_f32_activations(m):
    # the CPU-runnable reference case: W Q4_K [4096, 4096], x f32 [M, 4096], out f32
    got, want = run_case("Q4_K", 4096, 4096, m, torch.float32, torch.float32, 30 + m)
    assert T.rel_l2(got, want) <= 1e-3


@pytest.mark.parametrize("m", [36, 128, 300, 700])
@pytest.mark.parametrize("dt", ["float16", "bfloat16"])
def test_q8_0_prefill_rows_on_the_tensor_cores(m, dt):
    # more than 32 rows: the 34-byte blocks are expanded to f16 (q x d rounded once) and multiplied by tcgen05,
    # instead of streaming the weights once per 8 rows; N = 1000 ends in a partial 128-row tile
    got, want = run_case("Q8_0", 1000, 2048, m, getattr(torch, dt), torch.float32, 60 + m)
    assert T.rel_l2(got, want) <= 1e-3


@pytest.mark.parametrize("m", [9, 130, 600])
@pytest.mark.parametrize("k", [768, 2048])
def test_q6_k_prefill_rows_on_the_tensor_cores(m, k):
    # K = 768 has three super-blocks per row, so rows alternate between 4-byte aligned and 2 bytes off: both forms
    # of the producers' word loads are exercised
    got, want = run_case("Q6_K", 1000, k, m, torch.bfloat16, torch.float32, 70 + m)
    assert T.rel_l2(got, want) <= 1e-3


@pytest.mark.parametrize("fmt", FURTHER)
@pytest.mark.parametrize("dt", ["float32", "float16"])
def test_further_ggml_types_any_row_count(fmt, dt):
    # 21 rows: past the eight of a decode work item, so these go to the tensor-core GEMM; N = 1000 is not a multiple
    # of its 128-row tiles
    got, want = run_case(fmt, 1000, 768, 21, getattr(torch, dt), torch.float32, 80)
    assert T.rel_l2(got, want) <= 1e-3


@pytest.mark.parametrize("fmt", FURTHER)
@pytest.mark.parametrize("m", [9, 130, 600])
@pytest.mark.parametrize("k", [768, 2048])
def test_further_ggml_types_prefill_rows_on_the_tensor_cores(fmt, m, k):
    # the blocks are expanded to f16 by the producer warps (Q5_K / Q2_K: d sc q - dmin m in split f16 arithmetic;
    # Q4_0 / Q5_0 / Q4_1 / Q5_1: (q - zero) x d [+ m] rounded once; Q3_K: (q - 4) x (d scale)) and multiplied by
    # tcgen05; K = 768 gives Q4_0 / Q5_0 rows whose 18- / 22-byte blocks alternate between 4-byte aligned and 2 bytes
    # off, and Q3_K rows of 330 bytes that do the same: both forms of the producers' word loads
    got, want = run_case(fmt, 1000, k, m, torch.bfloat16, torch.float32, 90 + m)
    assert T.rel_l2(got, want) <= 1e-3


@pytest.mark.parametrize("fmt", ["Q6_K"] + FURTHER)
def test_further_ggml_types_decode_kernel_beyond_eight_rows(fmt):
    # with the tensor path switched off the decode kernel serves any row count, eight rows per work item
    from engine_b200 import _lib as L
    lib = L.lib()
    old = lib.hq_config_get(L.CFG_DENSE_TENSOR_MIN_ROWS)
    lib.hq_config_set(L.CFG_DENSE_TENSOR_MIN_ROWS, 1 << 40)
    try:
        got, want = run_case(fmt, 520, 1024, 21, torch.bfloat16, torch.float32, 95)
    finally:
        lib.hq_config_set(L.CFG_DENSE_TENSOR_MIN_ROWS, old)
    assert T.rel_l2(got, want) <= 1e-3


@pytest.mark.parametrize("fmt", ["Q8_0", "Q4_K", "Q6_K", "FP8", "MXFP4"])
def test_ragged_rows_and_tile_heights(fmt):
    # N not a multiple of the row tile, M not a multiple of 8, and an N large enough for the tall tiles
    for n, m in [(40, 11), (9472 + 24, 1), (19000, 2)]:
        if fmt == "FP8" and n % 128:
            n = (n // 128 + 1) * 128
        got, want = run_case(fmt, n, 512, m, torch.float16, torch.float32, 40)
        assert T.rel_l2(got, want) <= TOL[fmt], (n, m)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16])
def test_16bit_output_is_the_rounded_f32_result(out_dtype):
    rng = T.rng_for(1, 50)
    arrays, deq = T.make_weight("Q8_0", rng, 256, 512)
    xd = T.to_dev(rng.standard_normal((4, 512)).astype(np.float32), torch.bfloat16, DEV)
    layer = T.make_layer("Q8_0", arrays, 512, DEV)
    y32 = layer.forward_raw(xd, torch.float32)
    y16 = layer.forward_raw(xd, out_dtype)
    assert torch.equal(y32.to(out_dtype), y16)


def test_run_twice_is_bit_identical():
    rng = T.rng_for(1, 60)
    arrays, _ = T.make_weight("Q4_K", rng, 4096, 4096)
    xd = T.to_dev(rng.standard_normal((8, 4096)).astype(np.float32), torch.bfloat16, DEV)
    layer = T.make_layer("Q4_K", arrays, 4096, DEV)
    a = layer.forward_raw(xd, torch.float32).clone()
    b = layer.forward_raw(xd, torch.float32)
    assert torch.equal(a, b)


def test_dequantize_w_is_exact():
    rng = T.rng_for(1, 70)
    for fmt in ["Q8_0", "Q4_K", "Q6_K"] + FURTHER + ["FP8", "MXFP4"]:
        arrays, deq = T.make_weight(fmt, rng, 128, 256)
        layer = T.make_layer(fmt, arrays, 256, DEV)
        got = layer.dequantize_w().cpu().numpy()
        assert np.array_equal(got, deq), fmt


def test_empty_and_bad_arguments():
    import engine_b200 as hq
    rng = T.rng_for(1, 80)
    arrays, _ = T.make_weight("Q8_0", rng, 64, 256)
    layer = T.make_layer("Q8_0", arrays, 256, DEV)
    y = layer.forward_raw(torch.empty((0, 256), dtype=torch.bfloat16, device=DEV))
    assert y.shape == (0, 64)
    with pytest.raises(hq.HqError):
        layer.forward_raw(torch.zeros((2, 128), dtype=torch.bfloat16, device=DEV))
    with pytest.raises(hq.HqError):
        layer.forward_raw(torch.zeros((2, 256), dtype=torch.bfloat16))   # CPU tensor: no fallback
    with pytest.raises(hq.HqError):
        hq.GgufMatMul(torch.zeros((4, 34 * 4), dtype=torch.uint8, device=DEV), "Q8_0", 128)  # K % 256
