"""Expert-parallel dispatch/combine protocol with two CPU ranks over gloo: every rank's output must equal the
single-rank oracle result for its tokens.  The expert block and the reduce are stand-ins built on the oracle
(this is the host logic under test: ordering, split sizes, the two all-to-all-v exchanges, un-permute)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, results, chunks=1):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from engine_b200.ep import ExpertParallelMoE
        from oracle import moe as M
        e, k, h, i, t_local = 8, 3, 16, 12, 11 + rank      # ragged: ranks own different token counts
        rng = np.random.Generator(np.random.PCG64(77))
        gate, up = rng.standard_normal((2, e, i, h)).astype(np.float32)
        down = rng.standard_normal((e, h, i)).astype(np.float32)
        rng_r = np.random.Generator(np.random.PCG64(100 + rank))
        x = rng_r.standard_normal((t_local, h)).astype(np.float32)
        logits = rng_r.standard_normal((t_local, e)).astype(np.float32)
        if rank == 1:
            logits[:, :4] += 50.0          # rank 1 routes everything to rank 0's experts: empty splits appear
        ids, w = M.router_topk(logits, k, M.SCORE_SOFTMAX, M.WEIGHT_SCORE, True)

        ep = ExpertParallelMoE(e, expert_fn=None, reduce_fn=None, experts=object(), chunks=chunks)
        lo, hi = ep.local_expert_range()

        def expert_fn(rows, local_ids):
            rows_np, ids_np = rows.numpy(), local_ids.numpy().astype(np.int64)
            assert ((ids_np >= 0) & (ids_np < hi - lo)).all()
            gids = (ids_np + lo).reshape(-1, 1).astype(np.uint32)
            ones = np.ones((rows_np.shape[0], 1), np.float32)
            if rows_np.shape[0] == 0:
                return torch.zeros((0, h), dtype=torch.float32)
            return torch.from_numpy(M.moe_layer(rows_np, gids, ones, gate, up, down))

        def reduce_fn(y_rows, weights, row_map, out_dtype, addend):
            y = y_rows.numpy()[row_map.numpy().astype(np.int64)].reshape(weights.shape[0], weights.shape[1], -1)
            return torch.from_numpy(M.weighted_combine(y, weights.numpy())).to(out_dtype)

        ep.expert_fn, ep.reduce_fn = expert_fn, reduce_fn
        out = ep.forward(torch.from_numpy(x), torch.from_numpy(w), torch.from_numpy(ids.astype(np.int64)))
        want = M.moe_layer(x, ids, w, gate, up, down)
        err = float(np.abs(out.numpy() - want).max() / np.abs(want).max())
        send, recv = ep.last_counts
        results[rank] = (err, send, recv, t_local * k)
    finally:
        dist.destroy_process_group()


import pytest


@pytest.mark.parametrize("chunks", [1, 3])
def test_ep_protocol_two_cpu_ranks(chunks):
    # chunks > 1: the same exchange in token chunks (the form that overlaps exchange and experts on the GPU)
    world = 2
    port = 29500 + (os.getpid() % 2000) + 7 * chunks
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, port, results, chunks), nprocs=world, join=True)
        res = dict(results)
    assert set(res) == {0, 1}
    for rank, (err, send, recv, total) in res.items():
        assert err < 1e-5, (rank, err)
        assert sum(send) == total
    # what rank a sends to b is what b receives from a
    assert res[0][1][1] == res[1][2][0] and res[1][1][0] == res[0][2][1]
    assert res[1][1][1] == 0            # rank 1 kept nothing for itself


def test_ep_plan_is_stable_and_invertible():
    sys.path.insert(0, ROOT)
    from engine_b200.ep import ExpertParallelMoE
    ep = ExpertParallelMoE(8, experts=object())
    ep.world, ep.e_local = 4, 2
    ids = torch.tensor([[7, 0, 3], [1, 6, 2], [0, 1, 5]])
    order, counts, local_ids, row_map = ep.plan(ids)
    assert counts.tolist() == [4, 2, 1, 2]
    assert order.tolist() == [1, 3, 6, 7, 2, 5, 8, 0, 4]
    assert local_ids.tolist() == [0, 1, 0, 1, 1, 0, 1, 1, 0]
    assert order[row_map.long()].tolist() == list(range(9))
