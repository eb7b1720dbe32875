"""Parity at the benchmark configurations' own sizes (full expert count, hidden and intermediate widths): the
layer runs once on the GPU over all tokens; a token subset spread over the batch is recomputed by the C oracle
(oracle/hq_oracle.c: dequantize each expert row to f32, f32 dot) from host copies of the experts those tokens
touch.  Router ids are compared for every token, bit for bit.  f32 outputs against the unrounded oracle:
rel-L2 <= 1e-3 (GGUF), <= 2e-3 (FP8 / MXFP4).  Mode A = 16-bit activations; mode B = per-token 1x128 FP8
activations, the oracle applying the identical quantizer first.  Data are seeded synthetic stand-ins."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

from tests import hq_synth as S
from tests import hq_testlib as T

DEV = "cuda:0"


def _run_layer(name, tokens, n_chk, seed, mode_b=False):
    import engine_b200 as hq
    cfg = dict(S.MOE_CFGS[name])
    gen = torch.Generator(device=DEV)
    gen.manual_seed(seed)
    e, k, h = cfg["e"], cfg["k"], cfg["h"]
    experts = S.build_moe_layer(torch, hq, cfg, gen, DEV)
    rcfg = S.router_config(hq, cfg)
    sel_bias = (torch.randn(e, generator=gen, device=DEV) * 0.01) if cfg["router"] == "sigmoid_bias" else None
    x = torch.randn((tokens, h), generator=gen, device=DEV).to(torch.bfloat16)
    logits = torch.randn((tokens, e), generator=gen, device=DEV)
    top = hq.moe_router_topk(logits, rcfg, sel_bias)
    ids_o, w_o = S.oracle_router(cfg, logits.cpu().numpy(), None if sel_bias is None else sel_bias.cpu().numpy())
    ids_g = top.indices.cpu().numpy().astype(np.uint32)
    # rows whose k-th and (k+1)-th scores are within a few ulp may legitimately differ between expf
    # implementations; everything else must agree bit for bit
    same = (ids_g == ids_o).all(axis=1)
    assert same.mean() >= 0.999, f"router ids differ on {(~same).sum()} of {tokens} rows"
    assert np.allclose(top.values.cpu().numpy()[same], w_o[same], rtol=2e-6, atol=1e-9)
    shared = S.build_moe_layer(torch, hq, cfg, gen, DEV, 1) if cfg.get("shared") else None
    add = None
    if shared is not None:
        add = shared.forward_fp8_dense(x, torch.float32) if mode_b else \
            shared.forward(x, torch.ones((tokens, 1), device=DEV), torch.zeros((tokens, 1), dtype=torch.int32, device=DEV),
                           out_dtype=torch.float32)
    fwd = experts.forward_fp8_act if mode_b else experts.forward
    out = fwd(x, top.values, top.indices, shared_out=add, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert experts.down.device_status()[0] == 0
    sel = np.linspace(0, tokens - 1, n_chk).astype(np.int64)
    sel = sel[same[sel]]
    x_np = x.to(torch.float32).cpu().numpy()[sel]
    want = S.oracle_moe_subset(experts, x_np, ids_g[sel], top.values.cpu().numpy()[sel], fp8_act=mode_b)
    if shared is not None:
        want = want + S.oracle_moe_subset(shared, x_np, np.zeros((len(sel), 1), np.int64),
                                          np.ones((len(sel), 1), np.float32), fp8_act=mode_b)
    return T.rel_l2(out.cpu().numpy()[sel], want)


@pytest.mark.parametrize("tokens", [64, 1024])
def test_cfg3_q4k_layer_at_full_size(tokens):
    # Qwen3-30B-A3B shape: 128 experts, top-8, hidden 2048, intermediate 768, Q4_K banks; mode A
    assert _run_layer("moe_q4k", tokens, 32, 31) <= 1e-3


@pytest.mark.parametrize("tokens", [128, 2048])
def test_cfg5_mxfp4_layer_at_full_size(tokens):
    # gpt-oss-120b shape: 128 experts, top-4, hidden = intermediate = 2880, interleaved gate/up with biases; mode A
    assert _run_layer("moe_mxfp4", tokens, 32, 51) <= 2e-3


def test_cfg4_block_fp8_layer_at_full_size_mode_b():
    # DeepSeek-V3 shape: 256 experts + shared expert, top-8, hidden 7168, intermediate 2048, sigmoid router with
    # bias; mode B (the FP8 x FP8 tensor-core path)
    assert _run_layer("moe_fp8", 256, 8, 41, mode_b=True) <= 2e-3


def test_cfg4_block_fp8_layer_at_full_size_mode_a():
    # the same layer with 16-bit activations (the reference's own arithmetic for this format)
    assert _run_layer("moe_fp8", 256, 6, 41, mode_b=False) <= 2e-3


def test_cfg2_vocabulary_projection_q8_0():
    # 4096 -> 128256 Q8_0 (the sweep's largest launch): sampled output features against the oracle
    import engine_b200 as hq
    from oracle import formats as F
    from oracle import moe as M
    gen = torch.Generator(device=DEV)
    gen.manual_seed(21)
    k, n = 4096, 128256
    w = S.q8_0_matrix(torch, n, k, gen, DEV)
    layer = hq.GgufMatMul(w, "Q8_0", k)
    for m in (1, 8):
        x = torch.randn((m, k), generator=gen, device=DEV).to(torch.bfloat16)
        y = layer.forward_raw(x, torch.float32)
        torch.cuda.synchronize()
        assert layer.device_status()[0] == 0
        rows = np.unique(np.concatenate([np.arange(0, 64), np.arange(n - 64, n),
                                         np.linspace(0, n - 1, 384).astype(np.int64)]))
        deq = F.q8_0_dequant(w[torch.as_tensor(rows, device=DEV)].cpu().numpy(), k)
        want = M.dense_forward(x.to(torch.float32).cpu().numpy(), deq)
        assert T.rel_l2(y.cpu().numpy()[:, rows], want) <= 1e-3
