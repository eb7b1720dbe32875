"""Host-side mirror of the reference's MoE glue over the C ABI: `moe_router_topk`
(hanzo-engine/src/ops.rs:225-335), `MoEExperts.forward`
(hanzo-engine/src/moe/experts/mod.rs:241-266, backends.rs:560-605) and the gpt-oss
expert block (hanzo-engine/src/models/gpt_oss.rs:384-443)."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib as L
from .quant import (DispatchTables, QuantMethod, _ptr, _require_cuda, _stream, convert, dt_code,
                    moe_dispatch_build, mxfp8_quantize_rows, tensor_path_expected)


@dataclass
class MoeRouterTopKConfig:
    """Field for field the reference's config struct (hanzo-engine/src/ops.rs:225-233)."""
    top_k: int
    score_function: int = L.SCORE_SOFTMAX      # Raw / Softmax / Sigmoid
    selected_weight: int = L.WEIGHT_SCORE      # Score / Softmax / Sigmoid
    renormalize: bool = False
    norm_min: float = 0.0
    output_scale: float = 1.0
    logit_clip: tuple[float, float] | None = None


@dataclass
class TopKOutput:
    values: torch.Tensor    # f32 [T, k]
    indices: torch.Tensor   # int32 [T, k] (bit pattern of the reference's u32 ids)


def _router_args(e: int, config: MoeRouterTopKConfig, bias, scale) -> "L.HqRouterArgs":
    clip = config.logit_clip
    return L.HqRouterArgs(e, config.top_k, config.score_function, config.selected_weight, int(config.renormalize),
                          int(clip is not None), clip[0] if clip else 0.0, clip[1] if clip else 0.0,
                          config.norm_min, config.output_scale, 0 if bias is None else bias.data_ptr(),
                          0 if scale is None else scale.data_ptr())


def moe_router_topk(logits: torch.Tensor, config: MoeRouterTopKConfig, selection_bias: torch.Tensor | None = None,
                    expert_scale: torch.Tensor | None = None, n_group: int = 1, topk_group: int = 1,
                    group_score: str = "top2_sum") -> TopKOutput:
    """`n_group` > 1 adds the DeepSeek group-limited selection (hanzo-engine/src/models/deepseek3.rs:623-690):
    group_score "top2_sum" = noaux_tc, "max" = group_limited_greedy."""
    _require_cuda(logits, "logits")
    t, e = logits.shape
    logits = logits.contiguous()
    ids = torch.empty((t, config.top_k), dtype=torch.int32, device=logits.device)
    w = torch.empty((t, config.top_k), dtype=torch.float32, device=logits.device)
    bias = None if selection_bias is None else selection_bias.to(torch.float32).contiguous()
    scale = None if expert_scale is None else expert_scale.to(torch.float32).contiguous()
    args = _router_args(e, config, bias, scale)
    if n_group > 1:
        mode = {"top2_sum": 0, "max": 1}[group_score]
        L.check(L.lib().hq_router_topk_grouped(_ptr(logits), dt_code(logits.dtype), t, C.byref(args), n_group,
                                               topk_group, mode, _ptr(ids), _ptr(w), _stream()),
                "hq_router_topk_grouped")
    else:
        L.check(L.lib().hq_router_topk(_ptr(logits), dt_code(logits.dtype), t, C.byref(args), _ptr(ids), _ptr(w),
                                       _stream()), "hq_router_topk")
    return TopKOutput(w, ids)


def moe_router_forward(xs: torch.Tensor, router_weight: torch.Tensor, config: MoeRouterTopKConfig,
                       selection_bias: torch.Tensor | None = None, **group) -> TopKOutput:
    """Router logits + selection for hidden states: logits = xs . Wr^T in f32 (hanzo-engine/src/models/
    qwen3_moe.rs:397-410, deepseek3.rs:588-595), by this library's mat-vec for decode-sized calls (<= 8 rows) and a
    plain library GEMM beyond that, followed by moe_router_topk."""
    from .quant import gemv, should_use_gemv
    x = xs.reshape(-1, xs.shape[-1])
    if should_use_gemv(x, router_weight):
        logits = gemv(x, router_weight, None, out_dtype=torch.float32)
    else:
        logits = x.to(torch.float32) @ router_weight.to(torch.float32).t()
    return moe_router_topk(logits, config, selection_bias, None, **group)


def moe_weighted_reduce(y: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, row_map: torch.Tensor | None = None,
                        addend: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = sum_s w[t, s] * y[row(t, s)] (+ addend[t]); y [T*k, H] or [T, k, H]."""
    t, k = w.shape
    h = y.shape[-1]
    out = torch.empty((t, h), dtype=out_dtype, device=y.device)
    if addend is not None and addend.dtype != out_dtype:
        addend = addend.to(out_dtype)
    L.check(L.lib().hq_moe_weighted_reduce(_ptr(y.contiguous()), dt_code(y.dtype), _ptr(w.contiguous()),
                                           _ptr(row_map), _ptr(None if addend is None else addend.contiguous()),
                                           _ptr(out), dt_code(out_dtype), t, k, h, _stream()),
            "hq_moe_weighted_reduce")
    return out


def gated_act(gate: torch.Tensor, up: torch.Tensor | None, act: int, limit: float | None = None,
              alpha: float = 1.702, interleaved: bool = False) -> torch.Tensor:
    """fused_glu / gptoss_swiglu as a stand-alone op (hanzo-quant/kernels/ops/ops.cu:335-360, :845-858)."""
    gate = gate.contiguous()
    n = gate.numel() // 2 if interleaved else gate.numel()
    shape = gate.shape[:-1] if interleaved else gate.shape
    out = torch.empty(shape, dtype=gate.dtype, device=gate.device)
    a = L.HqActArgs(act, int(limit is not None), 0.0 if limit is None else limit, alpha)
    L.check(L.lib().hq_gated_act(_ptr(gate), _ptr(None if up is None else up.contiguous()), dt_code(gate.dtype), n,
                                 int(interleaved), C.byref(a), _ptr(out), _stream()), "hq_gated_act")
    return out


class MoEExperts:
    """Expert block: gate/up projection + gated activation + down projection + weighted sum over slots.

    gate_proj/up_proj [E, I, H] and down_proj [E, H, I] as separate banks (Qwen3, DeepSeek), or a single
    `gate_up_proj` [E, 2I, H] whose rows interleave gate/up (gpt-oss).  The intermediate stays expert-sorted
    between the two projections; one dispatch build serves both."""

    def __init__(self, down_proj: QuantMethod, gate_proj: QuantMethod | None = None, up_proj: QuantMethod | None = None,
                 gate_up_proj: QuantMethod | None = None, act: int = L.ACT_SWIGLU, limit: float | None = None,
                 alpha: float = 1.702, inter_dtype: torch.dtype = torch.float16):
        if (gate_up_proj is None) == (gate_proj is None):
            raise L.HqError("give either gate_proj+up_proj or gate_up_proj")
        self.gate, self.up, self.gate_up, self.down = gate_proj, up_proj, gate_up_proj, down_proj
        self.act = L.HqActArgs(act, int(limit is not None), 0.0 if limit is None else limit, alpha)
        self.inter_dtype = inter_dtype
        self.n_experts = down_proj.n_experts

    def forward(self, xs: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                shared_out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None,
                tables: DispatchTables | None = None, _skip_reduce: bool = False) -> torch.Tensor:
        _require_cuda(xs, "xs")
        lead = xs.shape[:-1]
        x = xs.reshape(-1, xs.shape[-1]).contiguous()
        t, k = topk_ids.shape
        tables = tables or moe_dispatch_build(topk_ids, self.n_experts)
        first = self.gate_up if self.gate_up is not None else self.gate
        if x.dtype != torch.float16 and tensor_path_expected(first, t * k, dense=False):
            # one cast per token instead of one conversion per (token, slot) in the kernel
            x = convert(x, torch.float16, first._status_buf(x.device))
        inter = first.n // 2 if self.gate_up is not None else first.n
        h = torch.empty((t * k, inter), dtype=self.inter_dtype, device=x.device)
        w0 = first._weight_struct()
        w1 = self.up._weight_struct() if self.up is not None else None
        status = first._status_buf(x.device)
        self._last_tables = tables
        ev0 = self._mark()
        L.check(L.lib().hq_moe_gather_forward(C.byref(w0), None if w1 is None else C.byref(w1), C.byref(self.act),
                                              _ptr(x), dt_code(x.dtype), L.ROWS_PER_TOKEN, t, k,
                                              _ptr(tables.expert_bounds), _ptr(tables.sorted_assign),
                                              _ptr(tables.sorted_token), _ptr(tables.workspace), _ptr(h),
                                              dt_code(h.dtype), L.ROWS_SORTED, _ptr(status), _stream()),
                "hq_moe_gather_forward(gate/up)")
        y = torch.empty((t * k, self.down.n), dtype=torch.float32, device=x.device)
        wd = self.down._weight_struct()
        L.check(L.lib().hq_moe_gather_forward(C.byref(wd), None, None, _ptr(h), dt_code(h.dtype), L.ROWS_SORTED, t, k,
                                              _ptr(tables.expert_bounds), _ptr(tables.sorted_assign),
                                              _ptr(tables.sorted_token), _ptr(tables.workspace), _ptr(y),
                                              dt_code(y.dtype), L.ROWS_SORTED, _ptr(status), _stream()),
                "hq_moe_gather_forward(down)")
        self._mark(ev0)
        if _skip_reduce:       # measurement aid: the two projections only, output left expert-sorted
            return y
        out = moe_weighted_reduce(y, topk_weights.to(torch.float32), out_dtype or xs.dtype, tables.inv_perm, shared_out)
        return out.reshape(*lead, self.down.n)

    def forward_fp8_act(self, xs: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                        shared_out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None,
                        tables: DispatchTables | None = None, _skip_reduce: bool = False,
                        fp8_rows: tuple | None = None) -> torch.Tensor:
        """The same block with block-scaled FP8 activations (block-FP8 experts with separate gate/up banks only):
        token rows are quantized 1x128 straight into expert-sorted order; one launch runs the gate and the up
        projection on the FP8 tensor-core MMA (weights and activations unconverted), applies the gated activation
        and quantizes the intermediate again; the down projection writes expert-sorted rows (16-bit when the
        output is 16-bit, f32 otherwise) and the weighted reduce un-permutes them.

        `fp8_rows` = (buffer uint8 [R, row_bytes], hidden): token rows that are FP8 already, codes followed by the
        f32 scales in each row (the layout hq_ep_pack puts on the wire); `xs` is then ignored.
        Slots whose id is outside [0, n_experts) are skipped."""
        if self.gate is None or self.gate.format != L.FMT_FP8_BLOCK:
            raise L.HqError("forward_fp8_act needs block-FP8 experts with separate gate and up banks")
        t, k = topk_ids.shape
        if fp8_rows is None:
            _require_cuda(xs, "xs")
            lead = xs.shape[:-1]
            x = xs.reshape(-1, xs.shape[-1]).contiguous()
            dev, hidden = x.device, x.shape[-1]
        else:
            buf, hidden = fp8_rows
            _require_cuda(buf, "fp8_rows")
            lead, dev = (t,), buf.device
        tables = tables or moe_dispatch_build(topk_ids, self.n_experts)
        lib = L.lib()
        status = self.gate._status_buf(dev)
        n_valid = tables.expert_bounds[self.n_experts:]
        xq = torch.empty((t * k, hidden), dtype=torch.uint8, device=dev)
        xsc = torch.empty((t * k, hidden // 128), dtype=torch.float32, device=dev)
        if fp8_rows is None:
            L.check(lib.hq_fp8_quant_rows_n(_ptr(x), dt_code(x.dtype), hidden, _ptr(tables.sorted_token),
                                            _ptr(n_valid), t * k, hidden, _ptr(xq), _ptr(xsc), _stream()),
                    "hq_fp8_quant_rows_n")
        else:
            L.check(lib.hq_fp8_gather_rows(buf.data_ptr(), buf.stride(0), buf.data_ptr() + hidden, buf.stride(0),
                                           _ptr(tables.sorted_token), _ptr(n_valid), t * k, hidden, _ptr(xq),
                                           _ptr(xsc), _stream()), "hq_fp8_gather_rows")
        inter = self.gate.n
        hq_ = torch.empty((t * k, inter), dtype=torch.uint8, device=dev)
        hs = torch.empty((t * k, inter // 128), dtype=torch.float32, device=dev)
        wg, wu = self.gate._weight_struct(), self.up._weight_struct()
        self._last_tables = tables
        ev0 = self._mark()
        L.check(lib.hq_moe_fp8_gate_up_forward(C.byref(wg), C.byref(wu), C.byref(self.act), _ptr(xq), _ptr(xsc), t, k,
                                               _ptr(tables.expert_bounds), _ptr(hq_), _ptr(hs), _ptr(status),
                                               _stream()), "hq_moe_fp8_gate_up_forward")
        out_dtype = out_dtype or (xs.dtype if fp8_rows is None else torch.bfloat16)
        y_dtype = out_dtype if out_dtype in (torch.float16, torch.bfloat16) else torch.float32
        y = torch.empty((t * k, self.down.n), dtype=y_dtype, device=dev)
        wd = self.down._weight_struct()
        L.check(lib.hq_moe_fp8_gather_forward(C.byref(wd), _ptr(hq_), _ptr(hs), t, k, _ptr(tables.expert_bounds),
                                              _ptr(tables.sorted_assign), None, _ptr(y),
                                              dt_code(y.dtype), self.down.n, L.ROWS_SORTED, _ptr(status), _stream()),
                "hq_moe_fp8_gather_forward(down)")
        self._mark(ev0)
        if _skip_reduce:
            return y
        out = moe_weighted_reduce(y, topk_weights.to(torch.float32), out_dtype, tables.inv_perm, shared_out)
        return out.reshape(*lead, self.down.n)

    def forward_mx_act(self, xs: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                       shared_out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None,
                       tables: DispatchTables | None = None, _skip_reduce: bool = False) -> torch.Tensor:
        """The block with MXFP8 activations for MXFP4 experts on the block-scaled tensor-core MMA: token rows are
        quantized (e4m3 + one e8m0 scale per 32 elements) straight into expert-sorted order; the gate/up launch
        multiplies them with the e2m1 nibbles as stored, adds the bias, applies the gated activation and quantizes
        the intermediate the same way; the down projection writes expert-sorted rows for the weighted reduce.
        An interleaved gate_up bank (gpt-oss) takes one launch; separate gate and up banks take two plain
        launches, the gated activation and the row quantizer.  Slots with ids outside [0, n_experts) are skipped."""
        first = self.gate_up if self.gate_up is not None else self.gate
        banks = [first, self.down] + ([self.up] if self.up is not None else [])
        if any(b.format != L.FMT_MXFP4 or not b.mx_supported() for b in banks):
            raise L.HqError("forward_mx_act needs MXFP4 experts with K % 64 == 0")
        _require_cuda(xs, "xs")
        lead = xs.shape[:-1]
        x = xs.reshape(-1, xs.shape[-1]).contiguous()
        dev, hidden = x.device, x.shape[-1]
        t, k = topk_ids.shape
        tables = tables or moe_dispatch_build(topk_ids, self.n_experts)
        lib = L.lib()
        status = first._status_buf(dev)
        n_valid = tables.expert_bounds[self.n_experts:]
        xq, xsc = mxfp8_quantize_rows(x, tables.sorted_token, n_valid)
        self._last_tables = tables
        ev0 = self._mark()
        inter = first.n // 2 if self.gate_up is not None else first.n
        if inter % 32 != 0:
            raise L.HqError("forward_mx_act: the intermediate width must be a multiple of 32")
        if self.gate_up is not None:
            hq_ = torch.empty((t * k, inter), dtype=torch.uint8, device=dev)
            hs = torch.empty((t * k, inter // 32), dtype=torch.uint8, device=dev)
            w0 = first._weight_struct()
            L.check(lib.hq_moe_mx_gather_forward(C.byref(w0), C.byref(self.act), _ptr(xq), _ptr(xsc), t, k,
                                                 _ptr(tables.expert_bounds), None, None, 0, 0, L.ROWS_SORTED,
                                                 _ptr(hq_), _ptr(hs), _ptr(status), _stream()),
                    "hq_moe_mx_gather_forward(gate_up)")
        else:
            gu = []
            for bank in (self.gate, self.up):
                o = torch.empty((t * k, inter), dtype=torch.float32, device=dev)
                wb = bank._weight_struct()
                L.check(lib.hq_moe_mx_gather_forward(C.byref(wb), None, _ptr(xq), _ptr(xsc), t, k,
                                                     _ptr(tables.expert_bounds), None, _ptr(o), dt_code(o.dtype), inter,
                                                     L.ROWS_SORTED, None, None, _ptr(status), _stream()),
                        "hq_moe_mx_gather_forward(gate/up)")
                gu.append(o)
            hmid = gated_act(gu[0], gu[1], self.act.act, self.act.limit if self.act.has_limit else None,
                             self.act.alpha)
            hq_, hs = mxfp8_quantize_rows(hmid, None, n_valid)
        out_dtype = out_dtype or xs.dtype
        y_dtype = out_dtype if out_dtype in (torch.float16, torch.bfloat16) else torch.float32
        y = torch.empty((t * k, self.down.n), dtype=y_dtype, device=dev)
        wd = self.down._weight_struct()
        L.check(lib.hq_moe_mx_gather_forward(C.byref(wd), None, _ptr(hq_), _ptr(hs), t, k, _ptr(tables.expert_bounds),
                                             None, _ptr(y), dt_code(y.dtype), self.down.n, L.ROWS_SORTED, None, None,
                                             _ptr(status), _stream()), "hq_moe_mx_gather_forward(down)")
        self._mark(ev0)
        if _skip_reduce:
            return y
        out = moe_weighted_reduce(y, topk_weights.to(torch.float32), out_dtype, tables.inv_perm, shared_out)
        return out.reshape(*lead, self.down.n)

    def forward_fp8_dense(self, xs: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        """A one-expert block applied to every token (DeepSeek's shared expert,
        hanzo-engine/src/models/deepseek3.rs:783-786) on the FP8 path: 1x128 row quantizer, the fused gate/up
        launch over one expert holding all rows, and the dense FP8 down projection.  No routing tables."""
        _require_cuda(xs, "xs")
        if self.gate is None or self.gate.format != L.FMT_FP8_BLOCK or self.n_experts != 1:
            raise L.HqError("forward_fp8_dense needs a one-expert block-FP8 bank with separate gate and up")
        lead = xs.shape[:-1]
        x = xs.reshape(-1, xs.shape[-1]).contiguous()
        t, hidden = x.shape
        dev = x.device
        lib = L.lib()
        status = self.gate._status_buf(dev)
        bounds = getattr(self, "_dense_bounds", None)
        if bounds is None or bounds[1] != t or bounds[0].device != dev:
            bounds = (torch.tensor([0, t], dtype=torch.int32, device=dev), t)
            self._dense_bounds = bounds
        xq = torch.empty((t, hidden), dtype=torch.uint8, device=dev)
        xsc = torch.empty((t, hidden // 128), dtype=torch.float32, device=dev)
        L.check(lib.hq_fp8_quant_rows(_ptr(x), dt_code(x.dtype), hidden, None, t, hidden, _ptr(xq), _ptr(xsc),
                                      _stream()), "hq_fp8_quant_rows")
        inter = self.gate.n
        hq_ = torch.empty((t, inter), dtype=torch.uint8, device=dev)
        hs = torch.empty((t, inter // 128), dtype=torch.float32, device=dev)
        wg, wu, wd = self.gate._weight_struct(), self.up._weight_struct(), self.down._weight_struct()
        L.check(lib.hq_moe_fp8_gate_up_forward(C.byref(wg), C.byref(wu), C.byref(self.act), _ptr(xq), _ptr(xsc), t, 1,
                                               _ptr(bounds[0]), _ptr(hq_), _ptr(hs), _ptr(status), _stream()),
                "hq_moe_fp8_gate_up_forward(shared)")
        out_dtype = out_dtype or xs.dtype
        y = torch.empty((t, self.down.n), dtype=out_dtype, device=dev)
        L.check(lib.hq_fp8_linear_forward(C.byref(wd), _ptr(hq_), _ptr(hs), t, _ptr(y), dt_code(out_dtype), self.down.n,
                                          _ptr(status), _stream()), "hq_fp8_linear_forward(shared)")
        return y.reshape(*lead, self.down.n)

    def _mark(self, start=None):
        """Measurement hook: with `gemm_events` set to a list, every forward appends a (start, end) CUDA event
        pair around its two expert-GEMM launches.  While the stream is being captured into a CUDA graph the
        events are created as external event nodes, so they can be read after every replay of the graph."""
        evs = getattr(self, "gemm_events", None)
        if evs is None:
            return None
        if torch.cuda.is_current_stream_capturing():
            ev = torch.cuda.Event(enable_timing=True, external=True)
        else:
            ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        if start is not None:
            evs.append((start, ev))
        return ev

    def forward_layer(self, xs: torch.Tensor, logits: torch.Tensor, config: MoeRouterTopKConfig,
                      selection_bias: torch.Tensor | None = None, expert_scale: torch.Tensor | None = None,
                      shared_out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        """Router, dispatch, both projections and the weighted sum in one library call (hq_moe_layer_forward): the
        same kernels as moe_router_topk + forward, launched back to back without host work in between.  The
        scratch is kept by the object and grown when a call needs more."""
        _require_cuda(xs, "xs")
        lead = xs.shape[:-1]
        x = xs.reshape(-1, xs.shape[-1]).contiguous()
        t = x.shape[0]
        logits = logits.reshape(t, -1).contiguous()
        out_dtype = out_dtype or xs.dtype
        bias = None if selection_bias is None else selection_bias.to(torch.float32).contiguous()
        scale = None if expert_scale is None else expert_scale.to(torch.float32).contiguous()
        first = self.gate_up if self.gate_up is not None else self.gate
        w0, wd = first._weight_struct(), self.down._weight_struct()
        w1 = self.up._weight_struct() if self.up is not None else None
        layer = L.HqMoeLayer(C.pointer(w0), C.pointer(w1) if w1 is not None else None, C.pointer(wd), self.act,
                             _router_args(self.n_experts, config, bias, scale))
        lib = L.lib()
        need = int(lib.hq_moe_layer_workspace_bytes(C.byref(layer), t, dt_code(x.dtype)))
        if need == 0 and t > 0:
            raise L.HqError("hq_moe_layer_workspace_bytes: the layer description is inconsistent")
        ws = getattr(self, "_layer_ws", None)
        if ws is None or ws.numel() < need or ws.device != x.device:
            ws = torch.empty(max(need, 256), dtype=torch.uint8, device=x.device)
            self._layer_ws = ws
        out = torch.empty((t, self.down.n), dtype=out_dtype, device=x.device)
        add = None
        if shared_out is not None:
            add = shared_out.reshape(t, -1)
            add = add.to(out_dtype).contiguous() if add.dtype != out_dtype else add.contiguous()
        L.check(lib.hq_moe_layer_forward(C.byref(layer), _ptr(logits), dt_code(logits.dtype), _ptr(x), dt_code(x.dtype),
                                         t, _ptr(add), _ptr(out), dt_code(out_dtype), _ptr(ws), ws.numel(),
                                         _ptr(first._status_buf(x.device)), _stream()), "hq_moe_layer_forward")
        return out.reshape(*lead, self.down.n)
