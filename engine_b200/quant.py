"""Host-side mirror of hanzo-quant's `QuantMethod` API over the C ABI.

Same names and argument meaning as the reference trait
(hanzo-quant/src/lib.rs:1004-1108): `forward`, `forward_raw`, `gather_forward`,
`gather_forward_raw`, `dequantize_w`, `quantized_act_type`, implemented by
`GgufMatMul` (hanzo-quant/src/gguf/mod.rs:31-399), `BlockwiseFP8Linear`
(blockwise_fp8/mod.rs:24-198) and `MXFP4Layer` (mxfp4/mod.rs:29-174).  torch is
used only for device memory and the stream; every computation is a call into
libhanzoquant_b200.so.  The reference is Rust; with no Rust toolchain available
this Python layer is the tested host binding of the same C entry points.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib as L

_DT = {torch.float32: L.DT_F32, torch.float16: L.DT_F16, torch.bfloat16: L.DT_BF16}


def dt_code(dtype: torch.dtype) -> int:
    try:
        return _DT[dtype]
    except KeyError:
        raise L.HqError(f"unsupported dtype {dtype}: expected f32, f16 or bf16") from None


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: torch.Tensor | None) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise L.HqError(f"{name} must be a CUDA tensor: this library has no CPU path")


@dataclass
class DispatchTables:
    """Output of `moe_dispatch_build` (hanzo-quant/src/gguf/cuda.rs:538-578): expert-sorted views of
    the flat assignment list t*k+s."""
    n_tokens: int
    top_k: int
    n_experts: int
    expert_bounds: torch.Tensor   # int32 [E+1]
    sorted_assign: torch.Tensor   # int32 [T*k] flat assignment index
    sorted_token: torch.Tensor    # int32 [T*k] token index
    inv_perm: torch.Tensor        # int32 [T*k] flat index -> sorted position
    workspace: torch.Tensor       # int32 words (tile lists)


def moe_dispatch_build(ids: torch.Tensor, n_experts: int) -> DispatchTables:
    _require_cuda(ids, "ids")
    t, k = ids.shape
    ids = ids.contiguous()
    if ids.dtype not in (torch.int32, torch.uint32):
        ids = ids.to(torch.int32)
    dev = ids.device
    ws_bytes = L.lib().hq_moe_dispatch_workspace_bytes(t, k, n_experts)
    bounds = torch.empty(n_experts + 1, dtype=torch.int32, device=dev)
    sa = torch.empty(t * k, dtype=torch.int32, device=dev)
    st = torch.empty(t * k, dtype=torch.int32, device=dev)
    inv = torch.empty(t * k, dtype=torch.int32, device=dev)
    ws = torch.empty(ws_bytes // 4, dtype=torch.int32, device=dev)
    L.check(L.lib().hq_moe_dispatch_build(_ptr(ids), t, k, n_experts, _ptr(bounds), _ptr(sa), _ptr(st), _ptr(inv),
                                          _ptr(ws), ws_bytes, _stream()), "hq_moe_dispatch_build")
    return DispatchTables(t, k, n_experts, bounds, sa, st, inv, ws)


def convert(x: torch.Tensor, dtype: torch.dtype, status: torch.Tensor | None = None) -> torch.Tensor:
    """Elementwise cast through the library's own kernel (hq_convert_status).  Casting to f16 clamps finite values
    beyond +-65504 and leaves HQ_DEV_F16_RANGE in `status` (the layer's device status word)."""
    if x.dtype == dtype:
        return x
    x = x.contiguous()
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    L.check(L.lib().hq_convert_status(_ptr(x), dt_code(x.dtype), _ptr(out), dt_code(dtype), x.numel(), _ptr(status),
                                      _stream()), "hq_convert_status")
    return out


def tensor_path_expected(layer, n_rows_total: int, dense: bool) -> bool:
    """Mirror of the C-side rule that sends a call to the tensor-core grouped GEMM (prefill-sized row counts,
    K % 64 == 0; Q8_0 from four times the configured row thresholds, because its decode kernel streams at HBM
    speed).  Used only to decide whether to hand activations over as f16, which that kernel copies into its
    operand tiles without a conversion pass."""
    if layer.k % 64:
        return False
    if layer.format == L.FMT_FP8_BLOCK and (layer.n % 128 or layer.k % 128):
        return False
    lib = L.lib()
    mult = 4 if layer.format == L.FMT_Q8_0 else 1
    if dense:
        return n_rows_total >= mult * lib.hq_config_get(L.CFG_DENSE_TENSOR_MIN_ROWS)
    return n_rows_total >= mult * lib.hq_config_get(L.CFG_MOE_TENSOR_MIN_ROWS) * layer.n_experts


class QuantMethod:
    """Base of the quantized layers; weights are [N, K] (dense) or [E, N, K] (expert bank)."""

    format: int
    n_experts: int
    n: int
    k: int

    def __init__(self):
        self._status = None
        self._ws = {}
        self._ws_need = {}
        self._w_cached = None

    # -- plumbing -------------------------------------------------------------------
    # QuantizedSerde (hanzo-quant/src/lib.rs:911-945): layer types the reference does not serialise say so
    def name(self) -> str:
        return type(self).__name__

    def isq_serde_supported(self) -> bool:
        return False

    def serialize(self) -> bytes:
        raise L.HqError(f"{self.name()} has no UQFF form")

    def _weight_struct(self) -> L.HqWeight:
        raise NotImplementedError

    def _status_buf(self, dev) -> torch.Tensor:
        if self._status is None or self._status.device != dev:
            self._status = torch.zeros(4, dtype=torch.int32, device=dev)
        return self._status

    def device_status(self) -> list[int]:
        """Reads the device status word (synchronises the current stream); [0] != 0 means a kernel gave up on
        a bounded wait."""
        if self._status is None:
            return [0, 0, 0, 0]
        out = (C.c_int32 * 4)()
        L.check(L.lib().hq_status_read(_ptr(self._status), C.byref(out), _stream()), "hq_status_read")
        return list(out)

    # -- QuantMethod API ------------------------------------------------------------------
    def quantized_act_type(self):
        """Activation dtype the layer computes in; None = use the input's (lib.rs:1065)."""
        return None

    def forward(self, a: torch.Tensor) -> torch.Tensor:
        """y = a . W^T (+ b); leading dims are flattened to rows (lib.rs:1014-1021)."""
        return self.forward_raw(a)

    def forward_raw(self, a: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        _require_cuda(a, "a")
        if self.n_experts != 1:
            raise L.HqError("forward on an expert bank: use gather_forward")
        if a.shape[-1] != self.k:
            raise L.HqError(f"shape mismatch: input has {a.shape[-1]} features, weight expects {self.k}")
        lead = a.shape[:-1]
        x = a.reshape(-1, self.k)
        if x.stride(-1) != 1:
            x = x.contiguous()
        m = x.shape[0]
        out_dtype = out_dtype or a.dtype
        if x.dtype != torch.float16 and tensor_path_expected(self, m, dense=True):
            # the tensor-core kernel multiplies in f16 either way (values beyond +-65504 are clamped and flagged)
            x = convert(x if x.is_contiguous() else x.contiguous(), torch.float16, self._status_buf(a.device))
        y = torch.empty((m, self.n), dtype=out_dtype, device=a.device)
        # the weight descriptor never changes after construction: built once (a decode call is a few microseconds
        # of GPU time, so host work per call matters)
        w = self._w_cached
        if w is None:
            w = self._w_cached = self._weight_struct()
        stream = torch.cuda.current_stream(a.device).cuda_stream
        ws, ws_bytes = self._linear_workspace(w, m, a.device, stream)
        rc = L.lib().hq_linear_forward_ws(C.byref(w), x.data_ptr(), dt_code(x.dtype), x.stride(0) if m > 1 else self.k,
                                          y.data_ptr(), dt_code(out_dtype), self.n, m, ws, ws_bytes,
                                          self._status_buf(a.device).data_ptr(), stream)
        if rc != 0:
            L.check(rc, "hq_linear_forward_ws")
        return y.reshape(*lead, self.n)

    def _linear_workspace(self, w, m: int, device, stream: int):
        """Scratch for hq_linear_forward_ws, owned by the layer like the reference's Q8_1 activation buffer
        (fast_mmvq.rs:107-148): zero-filled once, grown when a call asks for more, one per CUDA stream."""
        need = self._ws_need.get(m)
        if need is None:
            need = self._ws_need[m] = int(L.lib().hq_linear_workspace_bytes(C.byref(w), m))
        if need == 0:
            return None, 0
        key = (device.index, stream)
        buf = self._ws.get(key)
        if buf is None or buf.numel() < need:
            buf = torch.zeros(need, dtype=torch.uint8, device=device)
            self._ws[key] = buf
        return buf.data_ptr(), buf.numel()

    def gather_forward(self, a: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
        """Per-assignment projection out of the bank (lib.rs:1032-1040): a is [T, K], [T, 1, K] (one row per
        token) or [T, k, K] (one row per slot); indices [T, k]; returns [T, k, N] in a's dtype."""
        return self.gather_forward_raw(a, indices)

    def gather_forward_raw(self, a: torch.Tensor, indices: torch.Tensor, out_dtype: torch.dtype | None = None,
                           tables: DispatchTables | None = None) -> torch.Tensor:
        _require_cuda(a, "a")
        t, k = indices.shape
        if a.dim() == 2:
            layout = L.ROWS_PER_TOKEN
        elif a.shape[1] == 1 and not self._3d_input_is_per_slot():
            layout = L.ROWS_PER_TOKEN
        else:
            layout = L.ROWS_PER_SLOT
            if a.shape[1] != k:
                raise L.HqError(f"per-slot input has {a.shape[1]} slots, indices have {k}")
        if a.shape[0] != t or a.shape[-1] != self.k:
            raise L.HqError("gather_forward: input / indices / weight shapes disagree")
        x = a.contiguous()
        if x.dtype != torch.float16 and tensor_path_expected(self, t * k, dense=False):
            x = convert(x, torch.float16, self._status_buf(a.device))
        tables = tables or moe_dispatch_build(indices, self.n_experts)
        out_dtype = out_dtype or a.dtype
        out = torch.empty((t, k, self.n), dtype=out_dtype, device=a.device)
        w = self._weight_struct()
        L.check(L.lib().hq_moe_gather_forward(C.byref(w), None, None, _ptr(x), dt_code(x.dtype), layout, t, k,
                                              _ptr(tables.expert_bounds), _ptr(tables.sorted_assign),
                                              _ptr(tables.sorted_token), _ptr(tables.workspace), _ptr(out),
                                              dt_code(out_dtype), L.ROWS_PER_SLOT,
                                              _ptr(self._status_buf(a.device)), _stream()),
                "hq_moe_gather_forward")
        return out

    def _3d_input_is_per_slot(self) -> bool:
        return False

    def dequantize_w(self) -> torch.Tensor:
        """f32 weights [N, K] / [E, N, K], computed on the device by pushing the identity through the layer's
        own kernels (every product is exact, each sum has one non-zero term)."""
        dev = self._device()
        eye = torch.eye(self.k, dtype=torch.float16, device=dev)
        outs = []
        lib = L.lib()
        old = lib.hq_config_get(L.CFG_DENSE_TENSOR_MIN_ROWS)
        lib.hq_config_set(L.CFG_DENSE_TENSOR_MIN_ROWS, 1 << 40)   # the decode kernel is the exact one
        try:
            for e in range(self.n_experts):
                layer = self._expert_view(e)
                outs.append(layer.forward_raw(eye, torch.float32).t().contiguous())
        finally:
            lib.hq_config_set(L.CFG_DENSE_TENSOR_MIN_ROWS, old)
        return outs[0] if self.n_experts == 1 else torch.stack(outs)

    def _device(self):
        raise NotImplementedError

    def _expert_view(self, e: int) -> "QuantMethod":
        raise NotImplementedError


GGML_Q8_0, GGML_Q4_K, GGML_Q6_K = "Q8_0", "Q4_K", "Q6_K"
_GGML = {GGML_Q8_0: (L.FMT_Q8_0, 32, 34), GGML_Q4_K: (L.FMT_Q4_K, 256, 144), GGML_Q6_K: (L.FMT_Q6_K, 256, 210),
         "Q5_K": (L.FMT_Q5_K, 256, 176), "Q4_0": (L.FMT_Q4_0, 32, 18), "Q5_0": (L.FMT_Q5_0, 32, 22),
         "Q4_1": (L.FMT_Q4_1, 32, 20), "Q5_1": (L.FMT_Q5_1, 32, 24), "Q2_K": (L.FMT_Q2_K, 256, 84),
         "Q3_K": (L.FMT_Q3_K, 256, 110)}


class GgufMatMul(QuantMethod):
    """GGUF block-quantized linear / expert bank (hanzo-quant/src/gguf/mod.rs:31-399); `data` holds the raw
    GGUF block bytes exactly as a .gguf file stores them: uint8 [N, K/blk*bytes] or [E, N, ...]."""

    def __init__(self, data: torch.Tensor, qtype: str, k: int, bias: torch.Tensor | None = None):
        super().__init__()
        if qtype not in _GGML:
            raise L.HqError(f"GGML type {qtype} is not on this path ({', '.join(_GGML)} are)")
        _require_cuda(data, "data")
        self.format, blk, nbytes = _GGML[qtype]
        self.qtype = qtype
        if k % 256:
            raise L.HqError(f"K = {k} must be a multiple of 256")
        row_bytes = k // blk * nbytes
        if data.dtype != torch.uint8 or data.shape[-1] != row_bytes:
            raise L.HqError(f"expected uint8 rows of {row_bytes} bytes")
        self.data = data.contiguous()
        self.n_experts = data.shape[0] if data.dim() == 3 else 1
        self.n = data.shape[-2]
        self.k = k
        self.bias = bias

    def _weight_struct(self):
        return L.HqWeight(self.format, self.n_experts, self.n, self.k, self.data.data_ptr(), 0,
                          0 if self.bias is None else self.bias.data_ptr(),
                          0 if self.bias is None else dt_code(self.bias.dtype), 0)

    def _device(self):
        return self.data.device

    def _expert_view(self, e):
        if self.n_experts == 1:
            return self
        return GgufMatMul(self.data[e], self.qtype, self.k)

    # QuantizedSerde (hanzo-quant/src/lib.rs:911-945, gguf/mod.rs:427-674): the layer as a UQFF byte string
    def name(self) -> str:
        return "gguf"

    def isq_serde_supported(self) -> bool:
        return True

    def serialize(self) -> bytes:
        return self.serialize_with_bias(self.bias)

    def serialize_with_bias(self, bias: torch.Tensor | None) -> bytes:
        from . import uqff
        return uqff.serialize_gguf(self.data, self.qtype, self.k, bias)

    @classmethod
    def deserialize(cls, data, device) -> "GgufMatMul":
        return cls.deserialize_ext_bias(data, device)[0]

    @classmethod
    def deserialize_ext_bias(cls, data, device):
        """Returns (layer, bias): the bias is part of the layer and handed out as well, as in the reference."""
        from . import uqff
        raw, qtype, k, bias = uqff.deserialize_gguf(data)
        bias = None if bias is None else bias.to(device)
        return cls(raw.to(device), qtype, k, bias), bias


class BlockwiseFP8Linear(QuantMethod):
    """e4m3 weight with a 128x128 f32 `weight_scale_inv` grid (hanzo-quant/src/blockwise_fp8/mod.rs:24-198).
    weight uint8/float8 [N, K] or [E, N, K]; scale f32 [ceil(N/128), ceil(K/128)] (+ leading E)."""

    def __init__(self, weight: torch.Tensor, weight_scale_inv: torch.Tensor, bias: torch.Tensor | None = None,
                 weight_block_size=(128, 128)):
        super().__init__()
        _require_cuda(weight, "weight")
        if tuple(weight_block_size) != (128, 128):
            raise L.HqError("only 128x128 weight blocks are supported")
        if weight.dtype != torch.uint8:
            weight = weight.view(torch.uint8)
        self.format = L.FMT_FP8_BLOCK
        self.weight = weight.contiguous()
        self.scale = weight_scale_inv.to(torch.float32).contiguous()
        self.n_experts = weight.shape[0] if weight.dim() == 3 else 1
        self.n, self.k = weight.shape[-2], weight.shape[-1]
        want = (-(-self.n // 128), -(-self.k // 128))
        if tuple(self.scale.shape[-2:]) != want:
            raise L.HqError(f"scale grid {tuple(self.scale.shape)} does not match {want}")
        self.bias = bias
        # tables for the tensor-core path, derived once from the scale grid
        self.tile_scale = torch.empty(self.scale.shape[:-1], dtype=torch.float32, device=weight.device)
        self.rel_scale = torch.empty_like(self.scale)
        L.check(L.lib().hq_fp8_scale_prepare(_ptr(self.scale), self.n_experts, self.n, self.k, _ptr(self.tile_scale),
                                             _ptr(self.rel_scale), _stream()), "hq_fp8_scale_prepare")

    def _weight_struct(self):
        return L.HqWeight(self.format, self.n_experts, self.n, self.k, self.weight.data_ptr(), self.scale.data_ptr(),
                          0 if self.bias is None else self.bias.data_ptr(),
                          0 if self.bias is None else dt_code(self.bias.dtype), 0, self.tile_scale.data_ptr(),
                          self.rel_scale.data_ptr())

    def _device(self):
        return self.weight.device

    def _expert_view(self, e):
        return self if self.n_experts == 1 else BlockwiseFP8Linear(self.weight[e], self.scale[e])


    def forward_fp8_rows(self, codes: torch.Tensor, scales: torch.Tensor, out_dtype: torch.dtype = torch.float16):
        """Dense layer over rows that are already FP8 (codes [M, K], scales [M, K/128]): the FP8 tensor-core path
        with block-scaled activations."""
        if self.n_experts != 1:
            raise L.HqError("forward_fp8_rows on an expert bank")
        m = codes.shape[0]
        y = torch.empty((m, self.n), dtype=out_dtype, device=codes.device)
        w = self._weight_struct()
        L.check(L.lib().hq_fp8_linear_forward(C.byref(w), _ptr(codes.contiguous()), _ptr(scales.contiguous()), m,
                                              _ptr(y), dt_code(out_dtype), self.n,
                                              _ptr(self._status_buf(codes.device)), _stream()), "hq_fp8_linear_forward")
        return y


class MXFP4Layer(QuantMethod):
    """MXFP4 expert bank / linear (hanzo-quant/src/mxfp4/mod.rs:29-174): blocks uint8 [E, N, K/2] (low nibble =
    even element), scales uint8 [E, N, K/32] (e8m0), optional bias [E, N].  Any 3-D input to gather_forward is
    taken as one row per slot with top_k = dim 1 (mxfp4/ops.rs:349-355)."""

    def __init__(self, blocks: torch.Tensor, scales: torch.Tensor, bias: torch.Tensor | None = None):
        super().__init__()
        _require_cuda(blocks, "blocks")
        self.format = L.FMT_MXFP4
        # the bytes live in a buffer with 64 spare bytes behind them: the packed 4-bit tensor map of the
        # block-scaled path reads whole 128-element groups and may run past the last row's end
        store = torch.empty(blocks.numel() + 64, dtype=torch.uint8, device=blocks.device)
        store[:blocks.numel()].copy_(blocks.reshape(-1))
        store[blocks.numel():].zero_()
        self._store = store
        self.blocks = store[:blocks.numel()].view(blocks.shape)
        self.scales = scales.contiguous()
        self.n_experts = blocks.shape[0] if blocks.dim() == 3 else 1
        self.n, self.k = blocks.shape[-2], blocks.shape[-1] * 2
        if self.k % 32 or tuple(scales.shape[-2:]) != (self.n, self.k // 32):
            raise L.HqError("MXFP4: K must be a multiple of 32 and scales [.., N, K/32]")
        self.bias = None if bias is None else bias.contiguous()

    def _weight_struct(self):
        return L.HqWeight(self.format, self.n_experts, self.n, self.k, self.blocks.data_ptr(),
                          self.scales.data_ptr(), 0 if self.bias is None else self.bias.data_ptr(),
                          0 if self.bias is None else dt_code(self.bias.dtype), 0)

    def _3d_input_is_per_slot(self):
        return True

    def _device(self):
        return self.blocks.device

    def _expert_view(self, e):
        return self if self.n_experts == 1 else MXFP4Layer(self.blocks[e], self.scales[e])

    # QuantizedSerde (hanzo-quant/src/lib.rs:911-945, mxfp4/mod.rs:742-826)
    def name(self) -> str:
        return "mxfp4-layer"

    def isq_serde_supported(self) -> bool:
        return True

    def serialize(self) -> bytes:
        return self.serialize_with_bias(self.bias)

    def serialize_with_bias(self, bias: torch.Tensor | None) -> bytes:
        from . import uqff
        return uqff.serialize_mxfp4(self.blocks, self.scales, bias)

    @classmethod
    def deserialize(cls, data, device) -> "MXFP4Layer":
        return cls.deserialize_ext_bias(data, device)[0]

    @classmethod
    def deserialize_ext_bias(cls, data, device):
        from . import uqff
        blocks, scales, bias = uqff.deserialize_mxfp4(data)
        bias = None if bias is None else bias.to(device)
        return cls(blocks.to(device), scales.to(device), bias), bias

    def mx_supported(self) -> bool:
        """Shapes the block-scaled tensor-core path takes (K a multiple of 64, at least 128)."""
        return self.k % 64 == 0 and self.k >= 128

    def forward_mx_rows(self, codes: torch.Tensor, scales: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16):
        """Dense layer over rows that are MXFP8 already (mxfp8_quantize_rows): block-scaled MMA, nibbles and
        activation codes unconverted."""
        if self.n_experts != 1:
            raise L.HqError("forward_mx_rows is the dense call; expert banks go through MoEExperts.forward_mx_act")
        m = codes.shape[0]
        y = torch.empty((m, self.n), dtype=out_dtype, device=codes.device)
        w = self._weight_struct()
        L.check(L.lib().hq_mx_linear_forward(C.byref(w), _ptr(codes), _ptr(scales), m, _ptr(y), dt_code(out_dtype),
                                             self.n, _ptr(self._status_buf(codes.device)), _stream()),
                "hq_mx_linear_forward")
        return y


# ---- fused dense decode set (hanzo-quant/src/lib.rs:1116-1204, gemv/mod.rs) --------------------------

def try_fused_quantized_gate_up(xs: torch.Tensor, gate: QuantMethod, up: QuantMethod, act: int = L.ACT_SWIGLU,
                                limit: float | None = None, alpha: float = 1.702,
                                out_dtype: torch.dtype | None = None) -> torch.Tensor | None:
    """act(xs . Wgate^T) * (xs . Wup^T) in one launch (hanzo-quant/src/lib.rs:1116-1160).  Returns None where the
    reference's function would (biases, mismatched layers, expert banks), so callers keep their unfused route."""
    if getattr(gate, "bias", None) is not None or getattr(up, "bias", None) is not None:
        return None
    if gate.format != up.format or (gate.n, gate.k) != (up.n, up.k) or gate.n_experts != 1 or up.n_experts != 1:
        return None
    if xs.shape[-1] != gate.k or xs.dtype not in _DT:
        return None
    _require_cuda(xs, "xs")
    lead = xs.shape[:-1]
    x = xs.reshape(-1, gate.k)
    if x.stride(-1) != 1:
        x = x.contiguous()
    m = x.shape[0]
    if m == 0:
        return None
    if x.dtype != torch.float16 and tensor_path_expected(gate, m, dense=True):
        x = convert(x.contiguous(), torch.float16, gate._status_buf(xs.device))
    out_dtype = out_dtype or xs.dtype
    y = torch.empty((m, gate.n), dtype=out_dtype, device=xs.device)
    a = L.HqActArgs(act, int(limit is not None), 0.0 if limit is None else limit, alpha)
    wg, wu = gate._weight_struct(), up._weight_struct()
    L.check(L.lib().hq_linear_glu_forward(C.byref(wg), C.byref(wu), C.byref(a), _ptr(x), dt_code(x.dtype),
                                          x.stride(0) if m > 1 else gate.k, _ptr(y), dt_code(out_dtype), gate.n, m,
                                          _ptr(gate._status_buf(xs.device)), _stream()), "hq_linear_glu_forward")
    return y.reshape(*lead, gate.n)


def try_fused_quantized_qkv(xs: torch.Tensor, q: QuantMethod, k: QuantMethod, v: QuantMethod,
                            out_dtype: torch.dtype | None = None):
    """The three attention projections of one activation in one call (hanzo-quant/src/lib.rs:1162-1204)."""
    layers = (q, k, v)
    if any(getattr(l, "bias", None) is not None for l in layers) or any(l.n_experts != 1 for l in layers):
        return None
    if len({l.format for l in layers}) != 1 or any(l.k != xs.shape[-1] for l in layers) or xs.dtype not in _DT:
        return None
    _require_cuda(xs, "xs")
    lead = xs.shape[:-1]
    x = xs.reshape(-1, q.k).contiguous()
    m = x.shape[0]
    if m == 0:
        return None
    if x.dtype != torch.float16 and tensor_path_expected(q, m, dense=True):
        x = convert(x, torch.float16, q._status_buf(xs.device))
    out_dtype = out_dtype or xs.dtype
    outs = [torch.empty((m, l.n), dtype=out_dtype, device=xs.device) for l in layers]
    ws = [l._weight_struct() for l in layers]
    L.check(L.lib().hq_linear_qkv_forward(C.byref(ws[0]), C.byref(ws[1]), C.byref(ws[2]), _ptr(x), dt_code(x.dtype),
                                          q.k, _ptr(outs[0]), _ptr(outs[1]), _ptr(outs[2]), dt_code(out_dtype), m,
                                          _ptr(q._status_buf(xs.device)), _stream()), "hq_linear_qkv_forward")
    return tuple(o.reshape(*lead, o.shape[-1]) for o in outs)


MAX_GEMV_BATCH_SIZE = 8


def should_use_gemv(x: torch.Tensor, w: torch.Tensor) -> bool:
    """hanzo-quant/src/gemv/mod.rs:65-110: CUDA tensors, 1..8 rows, K a multiple of 8."""
    if not (x.is_cuda and w.is_cuda) or w.dim() != 2 or x.shape[-1] != w.shape[1] or w.shape[1] % 8:
        return False
    rows = 1
    for d in x.shape[:-1]:
        rows *= d
    return 1 <= rows <= MAX_GEMV_BATCH_SIZE


def gemv(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
         out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """Unquantized decode mat-vec y = x . w^T (+ bias), w [N, K] f16 / bf16 / f32 (hanzo-quant/src/gemv/mod.rs:120-185)."""
    _require_cuda(x, "x")
    if not should_use_gemv(x, w):
        raise L.HqError(f"GEMV batch size exceeds maximum {MAX_GEMV_BATCH_SIZE} or shapes disagree")
    lead = x.shape[:-1]
    k = w.shape[1]
    xr = x.reshape(-1, k).contiguous()
    m = xr.shape[0]
    w = w.contiguous()
    out_dtype = out_dtype or x.dtype
    y = torch.empty((m, w.shape[0]), dtype=out_dtype, device=x.device)
    L.check(L.lib().hq_dense_gemv(_ptr(w), dt_code(w.dtype), w.shape[0], k, _ptr(bias),
                                  0 if bias is None else dt_code(bias.dtype), _ptr(xr), dt_code(xr.dtype), k, _ptr(y),
                                  dt_code(out_dtype), w.shape[0], m, _stream()), "hq_dense_gemv")
    return y.reshape(*lead, w.shape[0])


# ---- FP8 quantizers (hanzo-quant/src/vector_fp8/ops.rs, blockwise_fp8/ops.rs) --------------------

def fp8_vector_quantize(x: torch.Tensor):
    """1x128 groups along the flattened tensor -> (codes uint8 like x, scales f32 [numel/128])."""
    _require_cuda(x, "x")
    x = x.contiguous()
    n = x.numel()
    codes = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    scales = torch.empty(n // 128, dtype=torch.float32, device=x.device)
    L.check(L.lib().hq_fp8_vector_quant(_ptr(x), dt_code(x.dtype), n, _ptr(codes), _ptr(scales), _stream()),
            "hq_fp8_vector_quant")
    return codes, scales


def fp8_vector_dequantize(codes: torch.Tensor, scales: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    out = torch.empty(codes.shape, dtype=out_dtype, device=codes.device)
    L.check(L.lib().hq_fp8_vector_dequant(_ptr(codes.contiguous()), _ptr(scales), codes.numel(), _ptr(out),
                                          dt_code(out_dtype), _stream()), "hq_fp8_vector_dequant")
    return out


def fp8_quantize_rows(x: torch.Tensor, row_map: torch.Tensor | None = None):
    """The 1x128 quantizer over rows x[row_map[r]] (row_map None = identity): codes uint8 [R, K] and scales f32
    [R, K/128].  With `sorted_token` as the row map this produces the expert-sorted rows the FP8 expert GEMM reads."""
    _require_cuda(x, "x")
    x = x.contiguous()
    k = x.shape[-1]
    rows = x.shape[0] if row_map is None else row_map.numel()
    codes = torch.empty((rows, k), dtype=torch.uint8, device=x.device)
    scales = torch.empty((rows, k // 128), dtype=torch.float32, device=x.device)
    L.check(L.lib().hq_fp8_quant_rows(_ptr(x), dt_code(x.dtype), k, _ptr(row_map), rows, k, _ptr(codes), _ptr(scales),
                                      _stream()), "hq_fp8_quant_rows")
    return codes, scales


def mxfp8_quantize_rows(x: torch.Tensor, row_map: torch.Tensor | None = None, n_valid: torch.Tensor | None = None):
    """MXFP8 quantizer over rows x[row_map[r]]: e4m3 codes uint8 [R, K] and e8m0 scales uint8 [R, K/32] (shared
    exponent floor(log2 amax) - 8 per 32 elements).  Rows at or past *n_valid (a device int32) are left unwritten."""
    _require_cuda(x, "x")
    x = x.contiguous()
    k = x.shape[-1]
    rows = x.shape[0] if row_map is None else row_map.numel()
    codes = torch.empty((rows, k), dtype=torch.uint8, device=x.device)
    scales = torch.empty((rows, k // 32), dtype=torch.uint8, device=x.device)
    L.check(L.lib().hq_mxfp8_quant_rows(_ptr(x), dt_code(x.dtype), k, _ptr(row_map), _ptr(n_valid), rows, k,
                                        _ptr(codes), _ptr(scales), _stream()), "hq_mxfp8_quant_rows")
    return codes, scales


def fp8_gated_quantize_rows(gate_up: torch.Tensor, act: "L.HqActArgs"):
    """{gate | up} [R, 2W] -> act(gate) * up -> 1x128 quantizer: codes [R, W], scales [R, W/128]."""
    _require_cuda(gate_up, "gate_up")
    gate_up = gate_up.contiguous()
    rows, w2 = gate_up.shape
    codes = torch.empty((rows, w2 // 2), dtype=torch.uint8, device=gate_up.device)
    scales = torch.empty((rows, w2 // 256), dtype=torch.float32, device=gate_up.device)
    L.check(L.lib().hq_fp8_gated_quant_rows(_ptr(gate_up), dt_code(gate_up.dtype), rows, w2 // 2, C.byref(act),
                                            _ptr(codes), _ptr(scales), _stream()), "hq_fp8_gated_quant_rows")
    return codes, scales


def fp8_blockwise_quantize(w: torch.Tensor, weight_block_size=(128, 128)):
    _require_cuda(w, "w")
    w = w.contiguous()
    rows, cols = w.shape
    by, bx = weight_block_size
    codes = torch.empty((rows, cols), dtype=torch.uint8, device=w.device)
    scales = torch.empty((-(-rows // by), -(-cols // bx)), dtype=torch.float32, device=w.device)
    L.check(L.lib().hq_fp8_block_quant(_ptr(w), dt_code(w.dtype), rows, cols, by, bx, _ptr(codes), _ptr(scales),
                                       _stream()), "hq_fp8_block_quant")
    return codes, scales


def fp8_blockwise_dequantize(codes: torch.Tensor, scales: torch.Tensor, weight_block_size, out_dtype):
    rows, cols = codes.shape
    by, bx = weight_block_size
    out = torch.empty((rows, cols), dtype=out_dtype, device=codes.device)
    L.check(L.lib().hq_fp8_block_dequant(_ptr(codes.contiguous()), _ptr(scales.contiguous()), rows, cols, by, bx,
                                         _ptr(out), dt_code(out_dtype), _stream()), "hq_fp8_block_dequant")
    return out
