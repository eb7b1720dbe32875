"""UQFF: the reference's byte format for quantized layers ("ISQ artifacts"), for the two layer types of this path
that the reference serialises -- `GgufMatMul` (hanzo-quant/src/gguf/mod.rs:401-674) and `MXFP4Layer`
(hanzo-quant/src/mxfp4/mod.rs:729-826); `BlockwiseFP8Linear` reports `isq_serde_supported() == false` there
(blockwise_fp8/mod.rs:401-408) and does so here.  Host-side byte shuffling only: the payload of a GGUF layer is its raw
block bytes, exactly what the kernels read.

Layouts (all integers little endian):

  GGUF layer    u32 version | u8 0 (QuantizedSerdeType::Gguf) | u32 payload bytes | u8 has_bias | u32 ggml type id |
                u32 n_dims | u32 dims[n_dims] (the logical weight shape, [N, K] or [E, N, K]) | payload |
                [bias tensor]
  MXFP4 layer   u32 version | u8 6 (QuantizedSerdeType::Mxfp4) | u8 has_bias | blocks tensor | scales tensor |
                [bias tensor]
  tensor        u32 data bytes | u32 dtype code | u32 n_dims | u32 dims[n_dims] | data   (utils/uqff.rs:88-162)

The version word is 0x00MMmmpp (major, minor, patch; utils/uqff.rs:14-39): a file is accepted when its major equals
this build's and its minor is not newer.

No fixture of the format exists in the reference's tree, so these functions are checked against byte strings built by
hand from the layout above, not against files the reference wrote."""
from __future__ import annotations

import struct

import numpy as np
import torch

UQFF_VERSION_MAJOR, UQFF_VERSION_MINOR, UQFF_VERSION_PATCH = 0, 2, 0
UQFF_VERSION = (UQFF_VERSION_MAJOR << 16) | (UQFF_VERSION_MINOR << 8) | UQFF_VERSION_PATCH
UQFF_QUANT_TYPE_OFFSET = 4                       # the serde type byte follows the version word

SERDE_GGUF, SERDE_UNQUANT, SERDE_HQQ, SERDE_FP8, SERDE_AFQ, SERDE_F8Q8, SERDE_MXFP4 = range(7)   # lib.rs:885-893

# ggml type ids of the weight types this library runs (gguf/mod.rs:455-470)
GGML_TYPE_ID = {"Q4_0": 2, "Q4_1": 3, "Q5_0": 6, "Q5_1": 7, "Q8_0": 8, "Q2_K": 10, "Q3_K": 11, "Q4_K": 12, "Q5_K": 13,
                "Q6_K": 14}
_GGML_NAME = {v: k for k, v in GGML_TYPE_ID.items()}
# weights per block, bytes per block
_GGML_BLOCK = {"Q4_0": (32, 18), "Q4_1": (32, 20), "Q5_0": (32, 22), "Q5_1": (32, 24), "Q8_0": (32, 34),
               "Q2_K": (256, 84), "Q3_K": (256, 110), "Q4_K": (256, 144), "Q5_K": (256, 176), "Q6_K": (256, 210)}

# tensor dtype codes (utils/uqff.rs:45-63)
_DTYPE_CODE = {torch.uint8: 0, torch.int32: 2, torch.int64: 3, torch.float16: 4, torch.bfloat16: 5, torch.float32: 6,
               torch.float64: 7, torch.int16: 8}
_CODE_DTYPE = {v: k for k, v in _DTYPE_CODE.items()}


class UqffError(ValueError):
    pass


def version_is_compatible(version: int) -> None:
    """utils/uqff.rs:25-39: same major, minor not newer than this build's."""
    major, minor, patch = version >> 16, (version >> 8) & 0xFF, version & 0xFF
    if major != UQFF_VERSION_MAJOR:
        raise UqffError(f"major version of the artifact ({major}) does not match this build ({UQFF_VERSION_MAJOR})")
    if minor > UQFF_VERSION_MINOR:
        raise UqffError(f"artifact version {major}.{minor}.{patch} is newer than this build supports "
                        f"({UQFF_VERSION_MAJOR}.{UQFF_VERSION_MINOR}.{UQFF_VERSION_PATCH})")


def _raw_bytes(t: torch.Tensor) -> bytes:
    return t.detach().contiguous().cpu().reshape(-1).view(torch.uint8).numpy().tobytes()


def write_tensor(buf: bytearray, t: torch.Tensor) -> None:
    """serialize_tensor, utils/uqff.rs:104-162."""
    if t.dtype not in _DTYPE_CODE:
        raise UqffError(f"dtype {t.dtype} cannot be serialised")
    data = _raw_bytes(t)
    if len(data) > 0xFFFFFFFF:
        raise UqffError("tensor data too large for the format (u32 length)")
    buf += struct.pack("<III", len(data), _DTYPE_CODE[t.dtype], t.dim())
    buf += struct.pack(f"<{t.dim()}I", *t.shape)
    buf += data


def read_tensor(data: bytes | memoryview, pos: int):
    """deserialize_tensor, utils/uqff.rs:164-201.  Returns (CPU tensor, position behind it)."""
    try:
        nbytes, code, ndim = struct.unpack_from("<III", data, pos)
        dims = struct.unpack_from(f"<{ndim}I", data, pos + 12)
    except struct.error as e:
        raise UqffError("truncated tensor header") from e
    pos += 12 + 4 * ndim
    if code not in _CODE_DTYPE:
        raise UqffError(f"unknown dtype for quantized tensor {code}")
    dtype = _CODE_DTYPE[code]
    if pos + nbytes > len(data):
        raise UqffError("truncated tensor data")
    want = int(np.prod(dims, dtype=np.int64)) * torch.empty((), dtype=dtype).element_size()
    if want != nbytes:
        raise UqffError(f"tensor of shape {dims} and dtype {dtype} needs {want} bytes, the record holds {nbytes}")
    raw = torch.frombuffer(bytearray(data[pos:pos + nbytes]), dtype=torch.uint8) if nbytes else \
        torch.empty(0, dtype=torch.uint8)
    return raw.view(dtype).reshape(dims), pos + nbytes


def serde_type(data: bytes | memoryview) -> int:
    """The QuantizedSerdeType byte of an artifact (what the reference's loader dispatches on)."""
    if len(data) <= UQFF_QUANT_TYPE_OFFSET:
        raise UqffError("truncated artifact")
    return data[UQFF_QUANT_TYPE_OFFSET]


def _header(data, expected: int) -> int:
    if len(data) < 5:
        raise UqffError("truncated artifact")
    version_is_compatible(struct.unpack_from("<I", data, 0)[0])
    if data[4] != expected:
        raise UqffError(f"ISQ type ({data[4]}) doesn't match expected type {expected}")
    return 5


# ---- GgufMatMul ----------------------------------------------------------------------------------------------------

def serialize_gguf(raw: torch.Tensor, qtype: str, k: int, bias: torch.Tensor | None = None) -> bytes:
    """raw: uint8 block bytes [N, row_bytes] or [E, N, row_bytes] (gguf/mod.rs:437-526)."""
    if qtype not in GGML_TYPE_ID:
        raise UqffError(f"GGML type {qtype} has no id here")
    per, nbytes = _GGML_BLOCK[qtype]
    if raw.dtype != torch.uint8 or raw.shape[-1] != k // per * nbytes:
        raise UqffError("block bytes do not match the type and K")
    payload = _raw_bytes(raw)
    if len(payload) > 0xFFFFFFFF:
        raise UqffError("weight too large for the format (u32 length)")
    shape = tuple(raw.shape[:-1]) + (k,)
    buf = bytearray()
    buf += struct.pack("<IBIBII", UQFF_VERSION, SERDE_GGUF, len(payload), 1 if bias is not None else 0,
                       GGML_TYPE_ID[qtype], len(shape))
    buf += struct.pack(f"<{len(shape)}I", *shape)
    buf += payload
    if bias is not None:
        write_tensor(buf, bias)
    return bytes(buf)


def deserialize_gguf(data: bytes | memoryview):
    """Returns (raw uint8 [.., N, row_bytes] on the CPU, type name, K, bias or None) (gguf/mod.rs:528-674)."""
    pos = _header(data, SERDE_GGUF)
    try:
        nbytes, has_bias, type_id, ndim = struct.unpack_from("<IBII", data, pos)
        dims = struct.unpack_from(f"<{ndim}I", data, pos + 13)
    except struct.error as e:
        raise UqffError("truncated GGUF layer header") from e
    pos += 13 + 4 * ndim
    if type_id not in _GGML_NAME:
        raise UqffError(f"ggml type id {type_id} is not on this path ({', '.join(GGML_TYPE_ID)} are)")
    qtype = _GGML_NAME[type_id]
    per, bb = _GGML_BLOCK[qtype]
    if ndim < 2 or dims[-1] % per:
        raise UqffError(f"weight shape {dims} does not fit blocks of {per}")
    k = dims[-1]
    row_bytes = k // per * bb
    if int(np.prod(dims[:-1], dtype=np.int64)) * row_bytes != nbytes or pos + nbytes > len(data):
        raise UqffError("payload length does not match the weight shape")
    raw = torch.frombuffer(bytearray(data[pos:pos + nbytes]), dtype=torch.uint8).reshape(tuple(dims[:-1]) + (row_bytes,))
    pos += nbytes
    bias = None
    if has_bias:
        bias, pos = read_tensor(data, pos)
    return raw, qtype, k, bias


# ---- MXFP4Layer ----------------------------------------------------------------------------------------------------

def serialize_mxfp4(blocks: torch.Tensor, scales: torch.Tensor, bias: torch.Tensor | None = None) -> bytes:
    """mxfp4/mod.rs:752-768."""
    if blocks.dtype != torch.uint8 or scales.dtype != torch.uint8:
        raise UqffError("MXFP4 blocks and scales are uint8 tensors")
    buf = bytearray(struct.pack("<IBB", UQFF_VERSION, SERDE_MXFP4, 1 if bias is not None else 0))
    write_tensor(buf, blocks)
    write_tensor(buf, scales)
    if bias is not None:
        write_tensor(buf, bias)
    return bytes(buf)


def deserialize_mxfp4(data: bytes | memoryview):
    """Returns (blocks, scales, bias or None) on the CPU (mxfp4/mod.rs:782-826)."""
    pos = _header(data, SERDE_MXFP4)
    if len(data) < pos + 1:
        raise UqffError("truncated MXFP4 layer header")
    has_bias = data[pos] != 0
    pos += 1
    blocks, pos = read_tensor(data, pos)
    scales, pos = read_tensor(data, pos)
    bias = None
    if has_bias:
        bias, pos = read_tensor(data, pos)
    return blocks, scales, bias
