"""Expert-parallel MoE over the GPUs of one box: experts are sharded in contiguous ranges (E / world per rank),
tokens stay data-parallel, and two all-to-all exchanges per layer move token rows to the ranks that own their
experts and bring the expert outputs back (NCCL over NVLink through torch.distributed).

The reference has no expert parallelism (its only MoE collective is the tensor-parallel all-reduce at
hanzo-engine/src/moe/experts/mod.rs:260-263, hanzo-quant/src/distributed/mod.rs:360-411); this module is the
exchange step the sharded path needs, built around the same local kernels.

Per layer and rank (device work is the C ABI's hq_ep_pack / hq_ep_unpack_meta plus the local expert block):
  1. pack: every token is written ONCE into the slab of every rank that hosts at least one of its experts (as
     e4m3 codes + 1x128 scales for block-FP8 experts, else in the 16-bit wire dtype), together with its slots'
     local expert ids and router weights;
  2. one all-to-all of equal-sized slabs (capacity rows per peer: no counts, nothing read back by the host);
  3. the local expert block runs over the received rows with top_k slots per row (slots of other ranks are -1 and
     are skipped) and reduces each row's local experts with their router weights: one partial sum per row;
  4. the partial sums return by the mirrored all-to-all;
  5. the source rank adds the <= world partial sums of each token (and the shared expert's output).
Results equal the single-GPU result up to f32 summation order and the rounding of the partial sums to the wire
dtype.

`pack_fn`, `unpack_fn`, `expert_fn` and `reduce_fn` are injectable so the protocol can be exercised with CPU
ranks (gloo).
"""
from __future__ import annotations

import ctypes as C
from typing import Callable

import torch
import torch.distributed as dist

from . import _lib as L


def make_layout(world: int, top_k: int, experts_per_rank: int, capacity: int, hidden: int,
                wire_dtype: torch.dtype, fp8: bool) -> "L.HqEpLayout":
    """Slab geometry (hq_ep_layout_init: host arithmetic only, needs no GPU)."""
    lay = L.HqEpLayout()
    code = {torch.float16: L.DT_F16, torch.bfloat16: L.DT_BF16}.get(wire_dtype)
    if code is None:
        raise L.HqError("wire dtype must be float16 or bfloat16")
    L.check(L.lib().hq_ep_layout_init(C.byref(lay), world, top_k, experts_per_rank, capacity, hidden, code, int(fp8)),
            "hq_ep_layout_init")
    return lay


def _gpu_pack(lay, x, ids, weights, send):
    from .quant import _ptr, _stream, dt_code
    t = ids.shape[0]
    back_map = torch.empty((t, lay.world), dtype=torch.int32, device=x.device)
    L.check(L.lib().hq_ep_pack(C.byref(lay), _ptr(x), dt_code(x.dtype), _ptr(ids), _ptr(weights), t, _ptr(send),
                               _ptr(back_map), _stream()), "hq_ep_pack")
    return back_map


def _gpu_unpack(lay, recv):
    from .quant import _ptr, _stream
    rows = lay.world * lay.rows_per_peer
    ids = torch.empty((rows, lay.top_k), dtype=torch.int32, device=recv.device)
    w = torch.empty((rows, lay.top_k), dtype=torch.float32, device=recv.device)
    L.check(L.lib().hq_ep_unpack_meta(C.byref(lay), _ptr(recv), _ptr(ids), _ptr(w), _stream()), "hq_ep_unpack_meta")
    return ids, w


def _gpu_expert_fn(experts, wire_dtype, mx_act=False):
    def run(lay, recv, ids, weights):
        rows = lay.world * lay.rows_per_peer
        if lay.fp8:
            buf = recv.view(rows, lay.row_bytes)
            return experts.forward_fp8_act(None, weights, ids, out_dtype=wire_dtype, fp8_rows=(buf, lay.hidden))
        x = recv.view(wire_dtype).view(rows, lay.hidden)
        if mx_act:
            return experts.forward_mx_act(x, weights, ids, out_dtype=wire_dtype)
        return experts.forward(x, weights, ids, out_dtype=wire_dtype)
    return run


def _gpu_reduce_fn(y_rows, weights, row_map, out_dtype, addend):
    from .moe import moe_weighted_reduce
    return moe_weighted_reduce(y_rows, weights, out_dtype, row_map, addend)


# symmetric exchange buffers, shared by every layer with the same slab geometry (layers run one after the other and
# the barrier protocol makes the buffers safe to reuse from one call to the next)
_SYMM_CACHE: dict = {}


class ExpertParallelMoE:
    def __init__(self, n_experts_global: int, experts=None, *, top_k: int, hidden: int, capacity: int, group=None,
                 wire_dtype: torch.dtype = torch.bfloat16, fp8_act: bool = False, mx_act: bool = False,
                 pack_fn: Callable | None = None, unpack_fn: Callable | None = None,
                 expert_fn: Callable | None = None, reduce_fn: Callable | None = None, exchange: str = "nccl"):
        """capacity: the largest number of tokens a rank brings to one call; the same value on every rank (it fixes
        the slab size, so ranks may bring different token counts without telling each other).
        fp8_act: block-FP8 experts, rows cross the wire as e4m3 + 1x128 scales; mx_act: MXFP4 experts on the
        block-scaled MMA (rows cross as `wire_dtype` and are quantized to MXFP8 on the expert rank).
        exchange: "nccl" = two all_to_all_single calls; "p2p" = the receive buffers live in symmetric memory
        (torch.distributed._symmetric_memory) and every rank stores its slabs straight into its peers' buffers
        (hq_ep_push) followed by a flag barrier (hq_ep_barrier); GPU ranks of one NVLink domain only."""
        if exchange not in ("nccl", "p2p"):
            raise ValueError("exchange must be 'nccl' or 'p2p'")
        self.exchange = exchange
        self._symm = None
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if n_experts_global % self.world:
            raise ValueError(f"{n_experts_global} experts do not split over {self.world} ranks")
        self.n_experts = n_experts_global
        self.e_local = n_experts_global // self.world
        self.wire_dtype = wire_dtype
        self.layout = make_layout(self.world, top_k, self.e_local, capacity, hidden, wire_dtype, fp8_act)
        self.pack_fn = pack_fn or _gpu_pack
        self.unpack_fn = unpack_fn or _gpu_unpack
        self.expert_fn = expert_fn or _gpu_expert_fn(experts, wire_dtype, mx_act)
        self.reduce_fn = reduce_fn or _gpu_reduce_fn
        self._bufs = None
        self._side = None

    def local_expert_range(self):
        return self.rank * self.e_local, (self.rank + 1) * self.e_local

    def wire_bytes_per_direction(self) -> tuple[int, int]:
        """(dispatch, return) bytes this rank puts on the wire per call (slabs to the other ranks)."""
        lay = self.layout
        return ((self.world - 1) * lay.message_bytes,
                (self.world - 1) * lay.rows_per_peer * lay.hidden * 2)

    def _buffers(self, device):
        if self._bufs is None or self._bufs[0].device != device:
            lay = self.layout
            send = torch.zeros((lay.world, lay.rows_per_peer, lay.row_bytes), dtype=torch.uint8, device=device)
            recv = torch.zeros_like(send)
            back = torch.zeros((lay.world * lay.rows_per_peer, lay.hidden), dtype=self.wire_dtype, device=device)
            ones = torch.ones((lay.capacity, lay.world), dtype=torch.float32, device=device)
            self._bufs = (send, recv, back, ones)
        return self._bufs

    def _symm_buffers(self, device):
        """Receive buffers, flag array and their peer-pointer tables for the "p2p" exchange (collective: every rank
        of the group calls this at the same point, the first time it runs a layer)."""
        if self._symm is None:
            import torch.distributed._symmetric_memory as symm
            lay = self.layout
            grp = self.group if self.group is not None else dist.group.WORLD
            key = (id(grp), lay.world, lay.rows_per_peer, lay.row_bytes, lay.hidden, self.wire_dtype, str(device))
            if key in _SYMM_CACHE:
                self._symm = _SYMM_CACHE[key]
                return self._symm
            recv = symm.empty((lay.world, lay.rows_per_peer, lay.row_bytes), dtype=torch.uint8, device=device)
            back = symm.empty((lay.world * lay.rows_per_peer, lay.hidden), dtype=self.wire_dtype, device=device)
            flags = symm.empty((64,), dtype=torch.int32, device=device)
            recv.zero_()
            back.zero_()
            flags.zero_()
            handles = [symm.rendezvous(t, grp) for t in (recv, back, flags)]
            torch.cuda.synchronize(device)
            dist.barrier(grp)          # every rank's flags are zero before anyone signals
            self._symm = {
                "recv": recv, "back": back, "flags": flags, "handles": handles,
                "p_recv": C.c_void_p(handles[0].buffer_ptrs_dev), "p_back": C.c_void_p(handles[1].buffer_ptrs_dev),
                "p_flags": C.c_void_p(handles[2].buffer_ptrs_dev),
                "seq": torch.zeros(1, dtype=torch.int32, device=device),
                "status": torch.zeros(4, dtype=torch.int32, device=device),
            }
            _SYMM_CACHE[key] = self._symm
        return self._symm

    def exchange_status(self) -> list[int]:
        """Device status word of the "p2p" exchange ({code, block, thread, tag}; all zero = no wait ran out)."""
        if self._symm is None:
            return [0, 0, 0, 0]
        return [int(v) for v in self._symm["status"].cpu()]

    def _push(self, src: torch.Tensor, peers, row_bytes: int, always_from: int, back_map=None, n_tokens: int = 0,
              ids=None):
        """Rows of the local slabs -> the peers' buffers (only the rows somebody reads), then the flag barrier."""
        sm = self._symm
        lay = self.layout
        stream = C.c_void_p(torch.cuda.current_stream(src.device).cuda_stream)
        lib = L.lib()
        L.check(lib.hq_ep_push_rows(src.data_ptr(), peers, self.world, self.rank, lay.rows_per_peer, row_bytes,
                                    always_from, None if back_map is None else back_map.data_ptr(), n_tokens,
                                    None if ids is None else ids.data_ptr(), lay.top_k, stream), "hq_ep_push_rows")
        L.check(lib.hq_ep_barrier(sm["p_flags"], self.world, self.rank, sm["seq"].data_ptr(),
                                  sm["status"].data_ptr(), stream), "hq_ep_barrier")

    def forward(self, xs: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                shared_out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None,
                shared_fn: Callable | None = None, shared_event=None) -> torch.Tensor:
        """`shared_fn`, if given, computes the shared expert's output; on a GPU it is queued on a second stream
        behind the pack so that it runs beside the dispatch exchange.  A caller that has started the shared expert
        earlier on a stream of its own passes its result as `shared_out` with the CUDA event recorded behind it
        as `shared_event`; the final reduce waits for that event."""
        t, k = topk_ids.shape
        lay = self.layout
        if t > lay.capacity:
            raise L.HqError(f"{t} tokens exceed the capacity {lay.capacity} this exchange was built for")
        x = xs.reshape(t, -1).contiguous()
        send, recv, back, ones = self._buffers(x.device)
        ids = topk_ids if topk_ids.dtype == torch.int32 else topk_ids.to(torch.int32)
        back_map = self.pack_fn(lay, x, ids.contiguous(), topk_weights.to(torch.float32).contiguous(), send)
        ev_shared = None
        if shared_fn is not None:
            if x.is_cuda:
                cur = torch.cuda.current_stream(x.device)
                if self._side is None:
                    self._side = torch.cuda.Stream(device=x.device)
                self._side.wait_stream(cur)
                with torch.cuda.stream(self._side):
                    shared_out = shared_fn()
                    ev_shared = self._side.record_event()
            else:
                shared_out = shared_fn()
        p2p = self.exchange == "p2p" and self.world > 1 and x.is_cuda
        if p2p:
            sm = self._symm_buffers(x.device)
            recv, back = sm["recv"], sm["back"]
            self._push(send, sm["p_recv"], lay.row_bytes, lay.capacity, back_map=back_map, n_tokens=t)
        elif self.world > 1:
            dist.all_to_all_single(recv, send, group=self.group)
        else:
            recv = send
        ids_l, w_l = self.unpack_fn(lay, recv)
        y = self.expert_fn(lay, recv, ids_l, w_l)
        if p2p:
            self._push(y.contiguous(), sm["p_back"], lay.hidden * y.element_size(), lay.rows_per_peer, ids=ids_l)
        elif self.world > 1:
            dist.all_to_all_single(back, y.contiguous(), group=self.group)
        else:
            back = y
        if ev_shared is None and shared_event is not None and shared_out is not None:
            ev_shared = shared_event
        if ev_shared is not None:
            torch.cuda.current_stream(x.device).wait_event(ev_shared)
            shared_out.record_stream(torch.cuda.current_stream(x.device))
        out = self.reduce_fn(back, ones[:t], back_map, out_dtype or xs.dtype, shared_out)
        return out.reshape(*xs.shape[:-1], out.shape[-1])
