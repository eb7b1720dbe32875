"""Expert-parallel MoE on the GPU.  One-GPU cases check the pack / unpack kernels against the numpy restatement
of the slab layout and run the whole exchange as a single rank (pack -> unpack -> local block -> reduce) against
the oracle; the two-GPU case runs it over NCCL (skipped when fewer than two GPUs are visible)."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = "cuda:0"


def test_pack_and_unpack_match_the_layout_restatement():
    from engine_b200 import ep as EP
    from tests import ep_cpu_ref as R
    world, k, e_local, cap, h, t = 4, 3, 2, 40, 64, 33
    lay = EP.make_layout(world, k, e_local, cap, h, torch.bfloat16, False)
    rng = np.random.Generator(np.random.PCG64(5))
    x = torch.from_numpy(rng.standard_normal((t, h)).astype(np.float32)).to(torch.bfloat16)
    ids = rng.integers(0, world * e_local, (t, k)).astype(np.int32)
    ids[3] = [-1, 5, -1]                       # padding slots
    ids[4] = 2                                 # all of a token's experts on one rank: it travels once
    w = rng.random((t, k)).astype(np.float32)
    send = torch.zeros((world, lay.rows_per_peer, lay.row_bytes), dtype=torch.uint8, device=DEV)
    bm = EP._gpu_pack(lay, x.to(DEV), torch.from_numpy(ids).to(DEV), torch.from_numpy(w).to(DEV), send)
    want = torch.zeros((world, lay.rows_per_peer, lay.row_bytes), dtype=torch.uint8)
    want_bm = R.cpu_pack(lay, x, torch.from_numpy(ids), torch.from_numpy(w), want)
    assert np.array_equal(bm.cpu().numpy(), want_bm.numpy())
    assert np.array_equal(send.cpu().numpy(), want.numpy())
    assert (bm.cpu().numpy()[4] >= 0).sum() == 1
    ids_l, w_l = EP._gpu_unpack(lay, send)
    want_ids, want_w = R.cpu_unpack(lay, want)
    assert np.array_equal(ids_l.cpu().numpy(), want_ids.numpy())
    assert np.array_equal(w_l.cpu().numpy(), want_w.numpy())


def test_pack_fp8_wire_carries_the_vector_quantizer_bit_for_bit():
    from engine_b200 import ep as EP
    from oracle import formats as F
    world, k, e_local, cap, h, t = 2, 2, 4, 16, 512, 9
    lay = EP.make_layout(world, k, e_local, cap, h, torch.bfloat16, True)
    rng = np.random.Generator(np.random.PCG64(6))
    x = rng.standard_normal((t, h)).astype(np.float32)
    x[2] = 0.0
    ids = np.stack([rng.integers(0, 4, t), rng.integers(4, 8, t)], axis=1).astype(np.int32)   # every token to both
    send = torch.zeros((world, lay.rows_per_peer, lay.row_bytes), dtype=torch.uint8, device=DEV)
    EP._gpu_pack(lay, torch.from_numpy(x).to(DEV), torch.from_numpy(ids).to(DEV),
                 torch.ones((t, k), device=DEV), send)
    codes, scales = F.fp8_vector_quant(x.reshape(-1), 128)
    got = send.cpu().numpy()
    for d in range(world):
        assert np.array_equal(got[d, :t, :h].reshape(-1), codes)
        assert np.array_equal(got[d, :t, h:].copy().view(np.float32).reshape(-1), scales)


@pytest.mark.parametrize("fmt,fp8", [("Q4_K", False), ("FP8", True)])
def test_single_rank_exchange_matches_the_oracle(fmt, fp8):
    """world = 1: no collective, but every kernel of the sharded path runs (pack, meta unpack, dispatch build that
    skips padding slots, row gather / quantizer bounded by the valid count, experts, both reduces)."""
    import engine_b200 as hq
    from engine_b200 import _lib as L
    from engine_b200.ep import ExpertParallelMoE
    from oracle import formats as F
    from oracle import moe as M
    from tests import hq_testlib as T
    e, k, h, i, t = 8, 2, 512, 512 if fp8 else 256, 200      # the FP8 MMA path needs K % 512 == 0
    rng = T.rng_for(8, 3)
    ga, gd = T.make_weight(fmt, rng, i, h, experts=e)
    ua, ud = T.make_weight(fmt, rng, i, h, experts=e)
    da, dd = T.make_weight(fmt, rng, h, i, experts=e)
    experts = hq.MoEExperts(T.make_layer(fmt, da, i, DEV), T.make_layer(fmt, ga, h, DEV), T.make_layer(fmt, ua, h, DEV))
    ep = ExpertParallelMoE(e, experts, top_k=k, hidden=h, capacity=256, wire_dtype=torch.float16, fp8_act=fp8)
    x = rng.standard_normal((t, h)).astype(np.float32)
    logits = rng.standard_normal((t, e)).astype(np.float32)
    ids, w = M.router_topk(logits, k, M.SCORE_SOFTMAX, M.WEIGHT_SCORE, True)
    xd = T.to_dev(x, torch.bfloat16, DEV)
    shared = T.to_dev(rng.standard_normal((t, h)).astype(np.float32), torch.float32, DEV)
    out = ep.forward(xd, T.to_dev(w, torch.float32, DEV), torch.from_numpy(ids.astype(np.int32)).to(DEV),
                     out_dtype=torch.float32, shared_fn=lambda: shared)
    torch.cuda.synchronize()
    assert experts.gate.device_status()[0] == 0
    f16 = lambda a: a.astype(np.float16).astype(np.float32)
    x_used = xd.to(torch.float32).cpu().numpy()
    if fp8:
        qdq = lambda a: F.fp8_vector_dequant(*F.fp8_vector_quant(a.reshape(-1), 128), 128).reshape(a.shape).astype(np.float32)
        want = M.moe_layer(qdq(x_used), ids, w, gd, ud, dd, h_round=lambda a: qdq(f16(a)), gu_round=f16)
    else:
        want = M.moe_layer(f16(x_used), ids, w, gd, ud, dd, h_round=f16)
    want = want + shared.cpu().numpy()
    # the partial sum of a token's experts crosses the wire in f16: 2.8e-4 of rounding on top of the kernel's error
    assert T.rel_l2(out.cpu().numpy(), want) <= (2e-3 if fp8 else 1e-3)


def test_push_moves_slab_d_to_slot_rank_of_peer_d():
    """hq_ep_push with the peers of a three-rank exchange emulated by three local buffers: after every rank has
    pushed, buffer d holds in slot r the slab d of rank r's send buffer (the all-to-all's result); the barrier
    entry point is exercised as a one-rank exchange (it signals and waits for itself)."""
    import ctypes as C
    from engine_b200 import _lib as L
    lib = L.lib()
    world, slab = 3, 4096 + 48                      # a slab size that is not a multiple of the CTA's stride
    rng = np.random.Generator(np.random.PCG64(11))
    sends = [torch.from_numpy(rng.integers(0, 256, (world, slab), dtype=np.uint8)).to(DEV) for _ in range(world)]
    recvs = [torch.zeros((world, slab), dtype=torch.uint8, device=DEV) for _ in range(world)]
    table = torch.tensor([r.data_ptr() for r in recvs], dtype=torch.int64, device=DEV)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for rank in range(world):
        assert lib.hq_ep_push(sends[rank].data_ptr(), table.data_ptr(), world, rank, slab, stream) == 0
    torch.cuda.synchronize()
    for d in range(world):
        for r in range(world):
            assert torch.equal(recvs[d][r], sends[r][d]), (d, r)
    flags = torch.zeros(64, dtype=torch.int32, device=DEV)
    ftable = torch.tensor([flags.data_ptr()], dtype=torch.int64, device=DEV)
    seq = torch.zeros(1, dtype=torch.int32, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    for n in range(1, 4):
        assert lib.hq_ep_barrier(ftable.data_ptr(), 1, 0, seq.data_ptr(), status.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        assert int(seq[0]) == n and int(flags[0]) == n and int(status[0]) == 0


def test_push_rows_sends_only_the_rows_somebody_reads():
    """hq_ep_push_rows on emulated peers: dispatch filter (back_map, meta rows always) and return filter (slot ids)."""
    import ctypes as C
    from engine_b200 import _lib as L
    lib = L.lib()
    world, rows, row_bytes, cap, k, n_tok = 2, 6, 64, 4, 2, 3
    rng = np.random.Generator(np.random.PCG64(12))
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    send = torch.from_numpy(rng.integers(1, 256, (world, rows, row_bytes), dtype=np.uint8)).to(DEV)
    recvs = [torch.zeros((world, rows, row_bytes), dtype=torch.uint8, device=DEV) for _ in range(world)]
    table = torch.tensor([r.data_ptr() for r in recvs], dtype=torch.int64, device=DEV)
    back_map = torch.tensor([[0, -1], [-1, 7], [2, 8], [3, 9]], dtype=torch.int32, device=DEV)   # row 3 >= n_tok
    rank = 1
    assert lib.hq_ep_push_rows(send.data_ptr(), table.data_ptr(), world, rank, rows, row_bytes, cap,
                               back_map.data_ptr(), n_tok, None, k, stream) == 0
    torch.cuda.synchronize()
    for d in range(world):
        for r in range(rows):
            sent = r >= cap or (r < n_tok and int(back_map[r, d]) >= 0)
            got = recvs[d][rank, r]
            assert torch.equal(got, send[d, r]) if sent else not bool(got.any()), (d, r)
        assert not bool(recvs[d][0].any())                 # slot of the other rank untouched
    # return direction: a row travels when one of its slots names an expert
    for r_ in recvs:
        r_.zero_()
    ids = torch.full((world * rows, k), 0xFFFFFFFF, dtype=torch.int64, device=DEV).to(torch.uint32)
    ids_np = np.full((world * rows, k), 0xFFFFFFFF, np.uint32)
    ids_np[1, 0] = 3
    ids_np[8, 1] = 0
    ids = torch.from_numpy(ids_np.view(np.int32)).to(DEV)
    assert lib.hq_ep_push_rows(send.data_ptr(), table.data_ptr(), world, rank, rows, row_bytes, rows, None, 0,
                               ids.data_ptr(), k, stream) == 0
    torch.cuda.synchronize()
    for d in range(world):
        for r in range(rows):
            sent = (d * rows + r) in (1, 8)
            got = recvs[d][rank, r]
            assert torch.equal(got, send[d, r]) if sent else not bool(got.any()), (d, r)


def _worker(rank, world, port, results, exchange="nccl"):
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
        ep = ExpertParallelMoE(e, experts, top_k=k, hidden=h, capacity=128, wire_dtype=torch.float16,
                               exchange=exchange)
        rr = T.rng_for(8, 10 + rank)
        x = T.to_dev(rr.standard_normal((t_local, h)).astype(np.float32), torch.bfloat16, dev)
        logits = rr.standard_normal((t_local, e)).astype(np.float32)
        top = hq.moe_router_topk(T.to_dev(logits, torch.float32, dev),
                                 hq.MoeRouterTopKConfig(k, L.SCORE_SOFTMAX, L.WEIGHT_SCORE, True))
        ids, w = M.router_topk(logits, k, L.SCORE_SOFTMAX, L.WEIGHT_SCORE, True)
        out = ep.forward(x, top.values, top.indices, out_dtype=torch.float32)
        out = ep.forward(x, top.values, top.indices, out_dtype=torch.float32)     # twice: the buffers are reused
        torch.cuda.synchronize()
        assert ep.exchange_status()[0] == 0
        f16 = lambda a: a.astype(np.float16).astype(np.float32)
        want = M.moe_layer(f16(x.to(torch.float32).cpu().numpy()), ids, w, gd, ud, dd, h_round=f16)
        results[rank] = (T.rel_l2(out.cpu().numpy(), want),
                         bool(np.array_equal(top.indices.cpu().numpy().astype(np.uint32), ids)))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("exchange", ["nccl", "p2p"])
def test_expert_parallel_two_gpus(exchange):
    import torch.multiprocessing as mp
    world = 2
    port = 29600 + (os.getpid() % 1000) + (7 if exchange == "p2p" else 0)
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, port, results, exchange), nprocs=world, join=True)
        res = dict(results)
    assert set(res) == {0, 1}
    for rank, (err, ids_ok) in res.items():
        assert ids_ok, rank
        assert err <= 1e-3, (rank, err)
