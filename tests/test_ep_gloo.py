"""Expert-parallel dispatch/combine protocol with two CPU ranks over gloo: every rank's output must equal the
single-rank oracle result for its tokens.  Pack, unpack, the expert block and the reduce are numpy stand-ins
(tests/ep_cpu_ref.py, the oracle); what is under test is the host logic: slab geometry, the two equal-split
all-to-all exchanges, one row per (token, destination rank), the partial sums coming back to the right rows."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, results, t_by_rank):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import __graft_entry__ as g
        g.build()
        from engine_b200.ep import ExpertParallelMoE
        from oracle import moe as M
        from tests import ep_cpu_ref as R
        e, k, h, i = 8, 3, 16, 12
        t_local = t_by_rank[rank]                      # ragged: ranks own different token counts
        rng = np.random.Generator(np.random.PCG64(77))
        gate, up = rng.standard_normal((2, e, i, h)).astype(np.float32)
        down = rng.standard_normal((e, h, i)).astype(np.float32)
        rng_r = np.random.Generator(np.random.PCG64(100 + rank))
        x = rng_r.standard_normal((t_local, h)).astype(np.float32)
        x = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()      # exact on the 16-bit wire
        logits = rng_r.standard_normal((t_local, e)).astype(np.float32)
        if rank == 1:
            logits[:, :4] += 50.0          # rank 1 routes everything to rank 0's experts: rows that travel nowhere
        ids, w = M.router_topk(logits, k, M.SCORE_SOFTMAX, M.WEIGHT_SCORE, True)

        ep = ExpertParallelMoE(e, experts=object(), top_k=k, hidden=h, capacity=max(t_by_rank),
                               wire_dtype=torch.bfloat16, pack_fn=R.cpu_pack, unpack_fn=R.cpu_unpack,
                               reduce_fn=R.cpu_reduce)
        lo, hi = ep.local_expert_range()
        seen = {}

        def expert_fn(lay, recv, ids_l, w_l):
            rows = R.cpu_rows(lay, recv).numpy()
            ids_np, w_np = ids_l.numpy().astype(np.int64), w_l.numpy()
            assert (ids_np < hi - lo).all()
            seen["rows_with_work"] = int((ids_np >= 0).any(axis=1).sum())
            out = np.zeros((rows.shape[0], h), np.float32)
            for r in range(rows.shape[0]):
                sel = ids_np[r] >= 0
                if sel.any():
                    gids = (ids_np[r][sel] + lo).reshape(1, -1).astype(np.uint32)
                    out[r] = M.moe_layer(rows[r:r + 1], gids, w_np[r][sel].reshape(1, -1), gate, up, down)[0]
            return torch.from_numpy(out).to(torch.float32).to(lay_wire(lay))

        def lay_wire(lay):
            return torch.bfloat16 if lay.wire_dtype == 2 else torch.float16

        ep.expert_fn = expert_fn
        shared = torch.from_numpy(rng_r.standard_normal((t_local, h)).astype(np.float32))
        out = ep.forward(torch.from_numpy(x), torch.from_numpy(w), torch.from_numpy(ids.astype(np.int32)),
                         out_dtype=torch.float32, shared_fn=lambda: shared)
        want = M.moe_layer(x, ids, w, gate, up, down) + shared.numpy()
        err = float(np.abs(out.numpy() - want).max() / np.abs(want).max())
        # one row per (token, destination rank): tokens of all ranks that have an expert here
        results[rank] = (err, seen["rows_with_work"],
                         [int(((ids // (e // world)) == d).any(axis=1).sum()) for d in range(world)])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("t_by_rank", [(11, 12), (1, 64)])
def test_ep_protocol_two_cpu_ranks(t_by_rank):
    # (1, 64): ranks that bring very different token counts still issue the same collectives
    world = 2
    port = 29500 + (os.getpid() % 2000) + 7 * t_by_rank[0]
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, port, results, t_by_rank), nprocs=world, join=True)
        res = dict(results)
    assert set(res) == {0, 1}
    for rank, (err, rows_here, sent) in res.items():
        assert err < 2e-2, (rank, err)         # partial sums travel back in bf16
    # rows a rank worked on = rows both ranks sent it, each token once however many of its experts live there
    for d in range(world):
        assert res[d][1] == res[0][2][d] + res[1][2][d]
    assert res[1][2][1] == 0            # rank 1 kept nothing for itself


def test_layout_arithmetic():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as g
    g.build()
    from engine_b200.ep import make_layout
    lay = make_layout(8, 8, 32, 512, 7168, torch.bfloat16, True)
    assert lay.row_bytes == 7168 + 56 * 4
    assert lay.pad_rows == -(-512 * 8 * 8 // lay.row_bytes)
    assert lay.rows_per_peer == 512 + lay.pad_rows
    assert lay.message_bytes == lay.rows_per_peer * lay.row_bytes
    lay = make_layout(2, 4, 64, 100, 2880, torch.float16, False)
    assert lay.row_bytes == 5760 and lay.pad_rows == 1
