"""ctypes binding of libhanzoquant_b200.so -- the same C ABI a Rust/cgo host
would bind (include/hanzoquant_b200.h).  Loading fails loudly: there is no
Python or CPU fallback behind these calls."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libhanzoquant_b200.so")

# codes (mirror include/hanzoquant_b200.h)
FMT_Q8_0, FMT_Q4_K, FMT_FP8_BLOCK, FMT_MXFP4, FMT_Q6_K, FMT_Q5_K, FMT_Q4_0, FMT_Q5_0 = 0, 1, 2, 3, 4, 5, 6, 7
FMT_Q4_1, FMT_Q5_1, FMT_Q2_K, FMT_Q3_K = 8, 9, 10, 11
DT_F32, DT_F16, DT_BF16 = 0, 1, 2
SCORE_RAW, SCORE_SOFTMAX, SCORE_SIGMOID = 0, 1, 2
WEIGHT_SCORE, WEIGHT_SOFTMAX, WEIGHT_SIGMOID = 0, 1, 2
ACT_NONE, ACT_SWIGLU, ACT_GPTOSS = 0, 1, 2
DEV_OK, DEV_WAIT_TIMEOUT, DEV_BAD_INDEX, DEV_SCALE_RANGE, DEV_F16_RANGE = 0, 1, 2, 3, 4
ROWS_PER_TOKEN, ROWS_PER_SLOT, ROWS_SORTED = 0, 1, 2
CFG_MOE_TENSOR_MIN_ROWS, CFG_DENSE_TENSOR_MIN_ROWS, CFG_SPIN_LIMIT, CFG_TEST_SKIP_PRODUCER = 0, 1, 2, 3
CFG_FP8_LOAD_BURST, CFG_FP8_L2_PREFETCH = 4, 5


class HqWeight(C.Structure):
    _fields_ = [("format", C.c_int32), ("n_experts", C.c_int32), ("n", C.c_int64), ("k", C.c_int64),
                ("data", C.c_void_p), ("scales", C.c_void_p), ("bias", C.c_void_p),
                ("bias_dtype", C.c_int32), ("reserved", C.c_int32),
                ("fp8_tile_scale", C.c_void_p), ("fp8_rel_scale", C.c_void_p)]


class HqRouterArgs(C.Structure):
    _fields_ = [("n_experts", C.c_int32), ("top_k", C.c_int32), ("score_mode", C.c_int32),
                ("weight_mode", C.c_int32), ("renormalize", C.c_int32), ("clamp_logits", C.c_int32),
                ("clamp_min", C.c_float), ("clamp_max", C.c_float), ("norm_min", C.c_float),
                ("output_scale", C.c_float), ("selection_bias", C.c_void_p), ("expert_scale", C.c_void_p)]


class HqActArgs(C.Structure):
    _fields_ = [("act", C.c_int32), ("has_limit", C.c_int32), ("limit", C.c_float), ("alpha", C.c_float)]


class HqEpLayout(C.Structure):
    _fields_ = [("world", C.c_int32), ("top_k", C.c_int32), ("experts_per_rank", C.c_int32), ("capacity", C.c_int32),
                ("pad_rows", C.c_int32), ("rows_per_peer", C.c_int32), ("fp8", C.c_int32), ("wire_dtype", C.c_int32),
                ("hidden", C.c_int64), ("row_bytes", C.c_int64), ("message_bytes", C.c_int64)]


class HqMoeLayer(C.Structure):
    _fields_ = [("gate", C.POINTER(HqWeight)), ("up", C.POINTER(HqWeight)), ("down", C.POINTER(HqWeight)),
                ("act", HqActArgs), ("router", HqRouterArgs)]


_P, _I32, _I64 = C.c_void_p, C.c_int32, C.c_int64

# every symbol include/hanzoquant_b200.h declares: name -> (restype, argtypes)
SIGNATURES = {
    "hq_abi_version": (_I32, []),
    "hq_error_string": (C.c_char_p, [_I32]),
    "hq_status_read": (_I32, [_P, C.POINTER(_I32 * 4), _P]),
    "hq_linear_forward": (_I32, [C.POINTER(HqWeight), _P, _I32, _I64, _P, _I32, _I64, _I64, _P, _P]),
    "hq_fp8_quant_rows": (_I32, [_P, _I32, _I64, _P, _I64, _I64, _P, _P, _P]),
    "hq_fp8_quant_rows_n": (_I32, [_P, _I32, _I64, _P, _P, _I64, _I64, _P, _P, _P]),
    "hq_fp8_gather_rows": (_I32, [_P, _I64, _P, _I64, _P, _P, _I64, _I64, _P, _P, _P]),
    "hq_ep_push": (_I32, [_P, _P, _I32, _I32, _I64, _P]),
    "hq_ep_push_rows": (_I32, [_P, _P, _I32, _I32, _I32, _I64, _I32, _P, _I32, _P, _I32, _P]),
    "hq_ep_barrier": (_I32, [_P, _I32, _I32, _P, _P, _P]),
    "hq_mxfp8_quant_rows": (_I32, [_P, _I32, _I64, _P, _P, _I64, _I64, _P, _P, _P]),
    "hq_mx_linear_forward": (_I32, [C.POINTER(HqWeight), _P, _P, _I64, _P, _I32, _I64, _P, _P]),
    "hq_moe_mx_gather_forward": (_I32, [C.POINTER(HqWeight), C.POINTER(HqActArgs), _P, _P, _I64, _I32, _P, _P, _P, _I32,
                                        _I64, _I32, _P, _P, _P, _P]),
    "hq_ep_layout_init": (_I32, [C.POINTER(HqEpLayout), _I32, _I32, _I32, _I32, _I64, _I32, _I32]),
    "hq_ep_pack": (_I32, [C.POINTER(HqEpLayout), _P, _I32, _P, _P, _I64, _P, _P, _P]),
    "hq_ep_unpack_meta": (_I32, [C.POINTER(HqEpLayout), _P, _P, _P, _P]),
    "hq_fp8_gated_quant_rows": (_I32, [_P, _I32, _I64, _I64, C.POINTER(HqActArgs), _P, _P, _P]),
    "hq_fp8_linear_forward": (_I32, [C.POINTER(HqWeight), _P, _P, _I64, _P, _I32, _I64, _P, _P]),
    "hq_moe_fp8_gather_forward": (_I32, [C.POINTER(HqWeight), _P, _P, _I64, _I32, _P, _P, _P, _P, _I32, _I64, _I32,
                                         _P, _P]),
    "hq_moe_fp8_gate_up_forward": (_I32, [C.POINTER(HqWeight), C.POINTER(HqWeight), C.POINTER(HqActArgs), _P, _P, _I64,
                                          _I32, _P, _P, _P, _P, _P]),
    "hq_moe_layer_workspace_bytes": (_I64, [C.POINTER(HqMoeLayer), _I64, _I32]),
    "hq_moe_layer_forward": (_I32, [C.POINTER(HqMoeLayer), _P, _I32, _P, _I32, _I64, _P, _P, _I32, _P, _I64, _P, _P]),
    "hq_linear_workspace_bytes": (_I64, [C.POINTER(HqWeight), _I64]),
    "hq_linear_forward_ws": (_I32, [C.POINTER(HqWeight), _P, _I32, _I64, _P, _I32, _I64, _I64, _P, _I64, _P, _P]),
    "hq_linear_glu_forward": (_I32, [C.POINTER(HqWeight), C.POINTER(HqWeight), C.POINTER(HqActArgs), _P, _I32, _I64, _P,
                                     _I32, _I64, _I64, _P, _P]),
    "hq_linear_qkv_forward": (_I32, [C.POINTER(HqWeight), C.POINTER(HqWeight), C.POINTER(HqWeight), _P, _I32, _I64, _P,
                                     _P, _P, _I32, _I64, _P, _P]),
    "hq_dense_gemv": (_I32, [_P, _I32, _I64, _I64, _P, _I32, _P, _I32, _I64, _P, _I32, _I64, _I64, _P]),
    "hq_router_topk": (_I32, [_P, _I32, _I64, C.POINTER(HqRouterArgs), _P, _P, _P]),
    "hq_router_topk_grouped": (_I32, [_P, _I32, _I64, C.POINTER(HqRouterArgs), _I32, _I32, _I32, _P, _P, _P]),
    "hq_moe_dispatch_workspace_bytes": (_I64, [_I64, _I32, _I32]),
    "hq_moe_dispatch_build": (_I32, [_P, _I64, _I32, _I32, _P, _P, _P, _P, _P, _I64, _P]),
    "hq_moe_dispatch_build_noalloc": (_I32, [_P, _I64, _I32, _I32, _P, _P, _P, _P, _P]),
    "hq_moe_gather_forward": (_I32, [C.POINTER(HqWeight), C.POINTER(HqWeight), C.POINTER(HqActArgs), _P, _I32,
                                     _I32, _I64, _I32, _P, _P, _P, _P, _P, _I32, _I32, _P, _P]),
    "hq_moe_weighted_reduce": (_I32, [_P, _I32, _P, _P, _P, _P, _I32, _I64, _I32, _I64, _P]),
    "hq_fp8_vector_quant": (_I32, [_P, _I32, _I64, _P, _P, _P]),
    "hq_fp8_vector_dequant": (_I32, [_P, _P, _I64, _P, _I32, _P]),
    "hq_fp8_block_quant": (_I32, [_P, _I32, _I64, _I64, _I32, _I32, _P, _P, _P]),
    "hq_fp8_block_dequant": (_I32, [_P, _P, _I64, _I64, _I32, _I32, _P, _I32, _P]),
    "hq_fp8_scale_prepare": (_I32, [_P, _I32, _I64, _I64, _P, _P, _P]),
    "hq_config_set": (_I32, [_I32, _I64]),
    "hq_config_get": (_I64, [_I32]),
    "hq_convert": (_I32, [_P, _I32, _P, _I32, _I64, _P]),
    "hq_convert_status": (_I32, [_P, _I32, _P, _I32, _I64, _P, _P]),
    "hq_probe_tensor_peak": (_I32, [_I32, _I32, _I32, _P, C.POINTER(C.c_double), _P]),
    "hq_gated_act": (_I32, [_P, _P, _I32, _I64, _I32, C.POINTER(HqActArgs), _P, _P]),
}

_lib = None


class HqError(RuntimeError):
    pass


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise HqError(f"{LIB_PATH} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` "
                          "(there is no fallback path)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise HqError(f"{what}: {lib().hq_error_string(rc).decode()} ({rc})")
