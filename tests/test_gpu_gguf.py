"""A .gguf file's expert banks go from disk to the expert block without conversion and give the oracle's result."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
gguf = pytest.importorskip("gguf")

from oracle import formats as F
from oracle import moe as M
from tests import hq_testlib as T
from tests.test_gguf_file import _write

DEV = "cuda:0"


def test_expert_banks_from_a_gguf_file(tmp_path):
    from engine_b200.gguf_file import GgufFile
    rng = T.rng_for(5, 9)
    e, k, h, i, t = 4, 2, 512, 256, 12
    mats, deq = {}, {}
    for name, (n, kk) in {"gate": (i, h), "up": (i, h), "down": (h, i)}.items():
        w = rng.normal(0, 0.02, (e * n, kk)).astype(np.float32)
        raw = F.q4_k_quantize(w)
        deq[name] = F.q4_k_dequant(raw, kk).reshape(e, n, kk)
        mats[f"blk.3.ffn_{name}_exps.weight"] = (raw.reshape(e, n, -1), gguf.GGMLQuantizationType.Q4_K)
    path = os.path.join(tmp_path, "moe.gguf")
    _write(path, mats, {"general.name": "tiny-moe"})
    experts = GgufFile(path).moe_experts(3, DEV)
    x = T.to_dev(rng.standard_normal((t, h)).astype(np.float32), torch.bfloat16, DEV)
    logits = rng.standard_normal((t, e)).astype(np.float32)
    ids, w = M.router_topk(logits, k, M.SCORE_SOFTMAX, M.WEIGHT_SCORE, True)
    out = experts.forward(x, T.to_dev(w, torch.float32, DEV), torch.from_numpy(ids.astype(np.int32)).to(DEV),
                          out_dtype=torch.float32)
    torch.cuda.synchronize()
    want = M.moe_layer(x.to(torch.float32).cpu().numpy(), ids, w, deq["gate"], deq["up"], deq["down"],
                       h_round=lambda a: a.astype(np.float16).astype(np.float32))
    assert T.rel_l2(out.cpu().numpy(), want) <= 1e-3
