"""B200-native quantized-linear and sparse-MoE expert path behind hanzo-quant's
QuantMethod API.  Importing the package does not need a GPU; every operation
does, and fails loudly without libhanzoquant_b200.so."""
from . import _lib, uqff
from ._lib import HqError
from .moe import (MoEExperts, MoeRouterTopKConfig, TopKOutput, gated_act, moe_router_forward, moe_router_topk,
                  moe_weighted_reduce)
from .quant import (BlockwiseFP8Linear, DispatchTables, GgufMatMul, MXFP4Layer, QuantMethod, fp8_blockwise_dequantize,
                    fp8_blockwise_quantize, fp8_gated_quantize_rows, fp8_quantize_rows, fp8_vector_dequantize,
                    fp8_vector_quantize, gemv, moe_dispatch_build, mxfp8_quantize_rows, should_use_gemv, try_fused_quantized_gate_up,
                    try_fused_quantized_qkv)

__all__ = [n for n in dir() if not n.startswith("_")]
