"""Expert-parallel MoE over the GPUs of one box: experts are sharded in contiguous ranges (E / world per rank),
tokens stay data-parallel, and two all-to-all exchanges per layer move token rows to the ranks that own their
experts and bring the expert outputs back (NCCL over NVLink through torch.distributed).

The reference has no expert parallelism (its only MoE collective is the tensor-parallel all-reduce at
hanzo-engine/src/moe/experts/mod.rs:260-263, hanzo-quant/src/distributed/mod.rs:360-411); this module is the
exchange step the sharded path needs, built around the same local kernels.

Per layer and rank:
  1. assignments (t, s) are ordered by destination rank (stable), counts are exchanged (one small all-to-all);
  2. token rows + local expert ids go out in one all-to-all-v each;
  3. the local expert block runs on the received rows (one row per assignment, top_k = 1);
  4. outputs return by the mirrored all-to-all-v;
  5. the source rank un-permutes and takes the router-weighted sum over its k slots.
Results equal the single-GPU result up to f32 summation order (none: every (t, s) output is computed once,
by the rank that owns the expert, and summed in slot order at the source).

`expert_fn` and `reduce_fn` are injectable so the protocol can be exercised with CPU ranks (gloo).
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


def _gpu_expert_fn(experts, fp8_act: bool = False):
    def run(rows: torch.Tensor, local_ids: torch.Tensor) -> torch.Tensor:
        if rows.shape[0] == 0:
            return torch.empty((0, experts.down.n), dtype=torch.float32, device=rows.device)
        ones = torch.ones((rows.shape[0], 1), dtype=torch.float32, device=rows.device)
        fwd = experts.forward_fp8_act if fp8_act else experts.forward
        return fwd(rows, ones, local_ids.reshape(-1, 1).to(torch.int32), out_dtype=torch.float32)
    return run


def _gpu_reduce_fn(y_rows, weights, row_map, out_dtype, addend):
    from .moe import moe_weighted_reduce
    return moe_weighted_reduce(y_rows, weights, out_dtype, row_map, addend)


class ExpertParallelMoE:
    def __init__(self, n_experts_global: int, experts=None, group=None,
                 expert_fn: Callable | None = None, reduce_fn: Callable | None = None,
                 wire_dtype: torch.dtype | None = None, fp8_act: bool = False, chunks: int = 1):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if n_experts_global % self.world:
            raise ValueError(f"{n_experts_global} experts do not split over {self.world} ranks")
        self.n_experts = n_experts_global
        self.e_local = n_experts_global // self.world
        self.expert_fn = expert_fn or _gpu_expert_fn(experts, fp8_act)
        self.reduce_fn = reduce_fn or _gpu_reduce_fn
        # dtype the expert outputs travel back in (None = as computed, f32: the result then equals the single-GPU
        # layer; torch.float16 halves the return traffic at 5e-4 relative rounding per expert output)
        self.wire_dtype = wire_dtype
        # token chunks per layer call: with more than one, the exchange of a chunk runs on a second stream while
        # the experts work on another chunk
        self.chunks = max(1, int(chunks))
        self._comm_stream = None
        self.last_counts = None      # (send_counts, recv_counts) of the last call, for traffic accounting

    def local_expert_range(self):
        return self.rank * self.e_local, (self.rank + 1) * self.e_local

    def plan(self, topk_ids: torch.Tensor):
        """Order the flat assignment list by destination rank (stable).  Returns (order, send_counts, local_ids,
        row_map): order[i] = flat index t*k+s of the i-th row sent; row_map[t*k+s] = its position.
        On the GPU the ordering is the library's own stable dispatch build with ranks in the place of experts
        (three small kernels instead of a sort)."""
        if topk_ids.is_cuda:
            from .quant import moe_dispatch_build
            ids32 = topk_ids.to(torch.int32)
            dest = torch.div(ids32, self.e_local, rounding_mode="floor")
            tab = moe_dispatch_build(dest, self.world)
            order = tab.sorted_assign
            send_counts = (tab.expert_bounds[1:] - tab.expert_bounds[:-1]).to(torch.int64)
            local_ids = (ids32 - dest * self.e_local).reshape(-1).index_select(0, order)
            return order, send_counts, local_ids, tab.inv_perm
        flat = topk_ids.reshape(-1).to(torch.int64)
        dest = torch.div(flat, self.e_local, rounding_mode="floor")
        order = torch.argsort(dest, stable=True)
        send_counts = torch.bincount(dest, minlength=self.world)
        row_map = torch.empty_like(order)
        row_map[order] = torch.arange(order.numel(), device=order.device)
        local_ids = (flat - dest * self.e_local)[order]
        return order, send_counts, local_ids, row_map.to(torch.int32)

    def _exchange_counts(self, send_counts: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return send_counts.clone()
        recv = torch.empty_like(send_counts)
        dist.all_to_all_single(recv, send_counts, group=self.group)
        return recv

    def _all_to_all_v(self, send: torch.Tensor, send_splits, recv_splits) -> torch.Tensor:
        out = torch.empty((sum(recv_splits),) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
        if self.world == 1:
            out.copy_(send)
            return out
        dist.all_to_all_single(out, send.contiguous(), recv_splits, send_splits, group=self.group)
        return out

    def forward(self, xs: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                shared_out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        t, k = topk_ids.shape
        if self.chunks > 1 and t >= 2 * self.chunks:
            return self._forward_chunked(xs, topk_weights, topk_ids, shared_out, out_dtype)
        x = xs.reshape(t, -1)
        order, send_counts, local_ids, row_map = self.plan(topk_ids)
        recv_counts = self._exchange_counts(send_counts)
        # split sizes are needed on the host by the collective: one small device->host read per layer
        both = torch.stack([send_counts, recv_counts]).tolist()
        send_splits = [int(v) for v in both[0]]
        recv_splits = [int(v) for v in both[1]]
        self.last_counts = (send_splits, recv_splits)
        rows = x.index_select(0, torch.div(order, k, rounding_mode="floor"))
        got_rows = self._all_to_all_v(rows, send_splits, recv_splits)
        got_ids = self._all_to_all_v(local_ids, send_splits, recv_splits)
        y = self.expert_fn(got_rows, got_ids)
        if self.wire_dtype is not None and y.dtype != self.wire_dtype:
            y = y.to(self.wire_dtype)
        back = self._all_to_all_v(y, recv_splits, send_splits)
        out = self.reduce_fn(back, topk_weights.to(torch.float32), row_map, out_dtype or xs.dtype, shared_out)
        return out.reshape(*xs.shape[:-1], out.shape[-1])

    def _forward_chunked(self, xs, topk_weights, topk_ids, shared_out, out_dtype):
        """The same exchange in `chunks` contiguous token chunks: all plans and split sizes first (one host read),
        then every chunk's dispatch is queued on a second stream, and each chunk's return is queued behind its
        expert block, so the experts of one chunk overlap the exchange of its neighbours.  Every rank issues the
        collectives in the same order."""
        t, k = topk_ids.shape
        x = xs.reshape(t, -1)
        c_n = self.chunks
        cuts = [t * c // c_n for c in range(c_n + 1)]
        plans = [self.plan(topk_ids[cuts[c]:cuts[c + 1]]) for c in range(c_n)]
        send_counts = torch.stack([p[1] for p in plans], dim=1).contiguous()          # [world, chunks]
        if self.world == 1:
            recv_counts = send_counts.clone()
        else:
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        both = torch.stack([send_counts, recv_counts]).tolist()
        send_splits = [[int(both[0][r][c]) for r in range(self.world)] for c in range(c_n)]
        recv_splits = [[int(both[1][r][c]) for r in range(self.world)] for c in range(c_n)]
        self.last_counts = ([sum(v) for v in zip(*send_splits)], [sum(v) for v in zip(*recv_splits)])
        on_gpu = x.is_cuda
        cur = torch.cuda.current_stream(x.device) if on_gpu else None
        if on_gpu and self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=x.device)
        comm = self._comm_stream if on_gpu else None

        class _On:      # queue the enclosed work on the exchange stream (nothing to do for CPU ranks)
            def __enter__(s_):
                if on_gpu:
                    s_.ctx = torch.cuda.stream(comm)
                    s_.ctx.__enter__()
            def __exit__(s_, *a):
                if on_gpu:
                    s_.ctx.__exit__(*a)

        got, ev_disp = [], []
        if on_gpu:
            comm.wait_stream(cur)
        for c in range(c_n):
            order, _, local_ids, _ = plans[c]
            with _On():
                rows = x[cuts[c]:cuts[c + 1]].index_select(0, torch.div(order, k, rounding_mode="floor"))
                g_rows = self._all_to_all_v(rows, send_splits[c], recv_splits[c])
                g_ids = self._all_to_all_v(local_ids, send_splits[c], recv_splits[c])
                ev = comm.record_event() if on_gpu else None
            got.append((g_rows, g_ids, rows))
            ev_disp.append(ev)
        backs, ev_back, keep = [], [], []
        for c in range(c_n):
            g_rows, g_ids, _ = got[c]
            if on_gpu:
                cur.wait_event(ev_disp[c])
                g_rows.record_stream(cur)
                g_ids.record_stream(cur)
            y = self.expert_fn(g_rows, g_ids)
            if self.wire_dtype is not None and y.dtype != self.wire_dtype:
                y = y.to(self.wire_dtype)
            ev_y = cur.record_event() if on_gpu else None
            with _On():
                if on_gpu:
                    comm.wait_event(ev_y)
                    y.record_stream(comm)
                back = self._all_to_all_v(y, recv_splits[c], send_splits[c])
                ev_back.append(comm.record_event() if on_gpu else None)
            backs.append(back)
            keep.append(y)
        outs = []
        w32 = topk_weights.to(torch.float32)
        for c in range(c_n):
            if on_gpu:
                cur.wait_event(ev_back[c])
                backs[c].record_stream(cur)
            add = None if shared_out is None else shared_out.reshape(t, -1)[cuts[c]:cuts[c + 1]]
            outs.append(self.reduce_fn(backs[c], w32[cuts[c]:cuts[c + 1]].contiguous(), plans[c][3],
                                       out_dtype or xs.dtype, add))
        out = torch.cat(outs, dim=0)
        return out.reshape(*xs.shape[:-1], out.shape[-1])
