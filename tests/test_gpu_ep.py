"""Expert-parallel MoE on two GPUs over NCCL: every rank's output equals the oracle result for its tokens.
Skipped when fewer than two GPUs are visible."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import engine_b200 as hq
        from engine_b200 import _lib as L
        from engine_b200.ep import ExpertParallelMoE
        from oracle import moe as M
        from tests import hq_testlib as T
        e, k, h, i, t_local = 8, 2, 512, 256, 96 + 32 * rank
        rng = T.rng_for(8, 1)                      # same banks on every rank; each keeps its slice
        ga, gd = T.make_weight("Q4_K", rng, i, h, experts=e)
        ua, ud = T.make_weight("Q4_K", rng, i, h, experts=e)
        da, dd = T.make_weight("Q4_K", rng, h, i, experts=e)
        el = e // world
        sl = slice(rank * el, (rank + 1) * el)
        cut = lambda a: {key: v[sl] for key, v in a.items()}
        experts = hq.MoEExperts(T.make_layer("Q4_K", cut(da), i, dev), T.make_layer("Q4_K", cut(ga), h, dev),
                                T.make_layer("Q4_K", cut(ua), h, dev))
        ep = ExpertParallelMoE(e, experts)
        rr = T.rng_for(8, 10 + rank)
        x = T.to_dev(rr.standard_normal((t_local, h)).astype(np.float32), torch.bfloat16, dev)
        logits = rr.standard_normal((t_local, e)).astype(np.float32)
        top = hq.moe_router_topk(T.to_dev(logits, torch.float32, dev),
                                 hq.MoeRouterTopKConfig(k, L.SCORE_SOFTMAX, L.WEIGHT_SCORE, True))
        ids, w = M.router_topk(logits, k, L.SCORE_SOFTMAX, L.WEIGHT_SCORE, True)
        out = ep.forward(x, top.values, top.indices, out_dtype=torch.float32)
        torch.cuda.synchronize()
        want = M.moe_layer(x.to(torch.float32).cpu().numpy(), ids, w, gd, ud, dd,
                           h_round=lambda a: a.astype(np.float16).astype(np.float32))
        # the chunked form (exchange of one token chunk overlapping the experts of another) gives the same rows
        ep2 = ExpertParallelMoE(e, experts, chunks=2)
        out2 = ep2.forward(x, top.values, top.indices, out_dtype=torch.float32)
        torch.cuda.synchronize()
        results[rank] = (max(T.rel_l2(out.cpu().numpy(), want), T.rel_l2(out2.cpu().numpy(), want)),
                         bool(np.array_equal(top.indices.cpu().numpy().astype(np.uint32), ids)))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_expert_parallel_two_gpus():
    import torch.multiprocessing as mp
    world = 2
    port = 29600 + (os.getpid() % 1000)
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        res = dict(results)
    assert set(res) == {0, 1}
    for rank, (err, ids_ok) in res.items():
        assert ids_ok, rank
        assert err <= 1e-3, (rank, err)
