"""Reader for .gguf files: tensor directory + raw block bytes, enough to put `ffn_{gate,up,down}_exps` expert banks
and dense quantized matrices on the device as the layers of this package, without the Rust loader
(the reference reads the same files through hanzo-ml's gguf_file and wraps the tensors in `GgufMatMul`,
hanzo-quant/src/gguf/mod.rs:401-425; expert banks hanzo-engine/src/models/quantized_qwen3_moe.rs:58-77).

File layout (GGUF v2 / v3, little endian): magic "GGUF", version u32, tensor count u64, metadata count u64; the
metadata key/value pairs; per tensor: name, n_dims u32, dims u64[n_dims] (innermost first), ggml type u32, offset
u64; padding to `general.alignment` (default 32); tensor data.  Quantized tensors are arrays of fixed-size blocks
in row-major order, which is exactly the byte layout the kernels consume: nothing is converted here.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass

import numpy as np

GGUF_MAGIC = 0x46554747
# ggml type id -> (name, elements per block, bytes per block)
GGML_TYPES = {
    0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 6: ("Q5_0", 32, 22),
    7: ("Q5_1", 32, 24), 8: ("Q8_0", 32, 34), 9: ("Q8_1", 32, 36), 10: ("Q2_K", 256, 84), 11: ("Q3_K", 256, 110),
    12: ("Q4_K", 256, 144), 13: ("Q5_K", 256, 176), 14: ("Q6_K", 256, 210), 15: ("Q8_K", 256, 292),
    30: ("BF16", 1, 2),
}
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}


class GgufError(ValueError):
    pass


@dataclass
class GgufTensor:
    name: str
    shape: tuple          # outermost first (numpy order); the last axis is the quantized row
    ggml_type: int
    offset: int           # from the start of the data section
    n_bytes: int

    @property
    def type_name(self) -> str:
        return GGML_TYPES[self.ggml_type][0]

    @property
    def row_bytes(self) -> int:
        _, per, nbytes = GGML_TYPES[self.ggml_type]
        return self.shape[-1] // per * nbytes


class GgufFile:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self._pos = 0
        magic, self.version = self._unpack("<II")
        if magic != GGUF_MAGIC:
            raise GgufError(f"{path}: not a GGUF file")
        if self.version not in (2, 3):
            raise GgufError(f"{path}: GGUF version {self.version} is not supported (2 and 3 are)")
        n_tensors, n_kv = self._unpack("<QQ")
        self.metadata = {}
        for _ in range(n_kv):
            key = self._string()
            (vtype,) = self._unpack("<I")
            self.metadata[key] = self._value(vtype)
        self.tensors = {}
        for _ in range(n_tensors):
            name = self._string()
            (n_dims,) = self._unpack("<I")
            dims = self._unpack("<" + "Q" * n_dims)
            ggml_type, offset = self._unpack("<IQ")
            if ggml_type not in GGML_TYPES:
                raise GgufError(f"{name}: unknown ggml type {ggml_type}")
            _, per, nbytes = GGML_TYPES[ggml_type]
            if dims[0] % per:
                raise GgufError(f"{name}: row of {dims[0]} elements is not a whole number of {per}-element blocks")
            n_elems = int(np.prod(dims, dtype=np.int64))
            self.tensors[name] = GgufTensor(name, tuple(int(d) for d in reversed(dims)), ggml_type, int(offset),
                                            n_elems // per * nbytes)
        align = int(self.metadata.get("general.alignment", 32))
        self.data_start = (self._pos + align - 1) // align * align

    # -- parsing helpers ----------------------------------------------------------------------------------
    def _unpack(self, fmt):
        size = struct.calcsize(fmt)
        out = struct.unpack_from(fmt, self._mm, self._pos)
        self._pos += size
        return out

    def _string(self) -> str:
        (n,) = self._unpack("<Q")
        s = self._mm[self._pos:self._pos + n].decode("utf-8", errors="replace")
        self._pos += n
        return s

    def _value(self, vtype):
        if vtype in _SCALARS:
            return self._unpack(_SCALARS[vtype])[0]
        if vtype == 8:
            return self._string()
        if vtype == 9:
            etype, count = self._unpack("<IQ")
            return [self._value(etype) for _ in range(count)]
        raise GgufError(f"unknown metadata value type {vtype}")

    # -- tensors -------------------------------------------------------------------------------------------
    def raw(self, name: str) -> np.ndarray:
        """The tensor's bytes as uint8 [..., row_bytes] (a view of the mapped file)."""
        t = self.tensors[name]
        start = self.data_start + t.offset
        flat = np.frombuffer(self._mm, dtype=np.uint8, count=t.n_bytes, offset=start)
        return flat.reshape(*t.shape[:-1], t.row_bytes)

    def quant_method(self, name: str, device, bias_name: str | None = None):
        """A 2-D tensor as a dense layer, a 3-D tensor ([E, N, K]) as an expert bank: `GgufMatMul` over the file's
        own block bytes."""
        import torch
        from .quant import GgufMatMul
        t = self.tensors[name]
        if t.type_name not in ("Q8_0", "Q4_K", "Q6_K", "Q5_K", "Q4_0", "Q5_0", "Q4_1", "Q5_1", "Q2_K", "Q3_K"):
            raise GgufError(f"{name}: GGML type {t.type_name} is not on this path "
                            "(Q8_0, Q4_0, Q4_1, Q5_0, Q5_1 and Q2_K .. Q6_K are)")
        if len(t.shape) not in (2, 3):
            raise GgufError(f"{name}: expected a matrix or an expert bank, got shape {t.shape}")
        data = torch.from_numpy(np.array(self.raw(name), copy=True)).to(device)
        bias = None
        if bias_name is not None and bias_name in self.tensors:
            b = self.tensors[bias_name]
            arr = np.frombuffer(self._mm, dtype={"F32": np.float32, "F16": np.float16}[b.type_name],
                                count=int(np.prod(b.shape)), offset=self.data_start + b.offset)
            bias = torch.from_numpy(arr.reshape(b.shape).copy()).to(device)
        return GgufMatMul(data, t.type_name, t.shape[-1], bias)

    def moe_experts(self, layer: int, device, prefix: str = "blk"):
        """`blk.{layer}.ffn_{gate,up,down}_exps.weight` as a MoEExperts block."""
        from .moe import MoEExperts
        names = [f"{prefix}.{layer}.ffn_{p}_exps.weight" for p in ("gate", "up", "down")]
        for n in names:
            if n not in self.tensors:
                raise GgufError(f"{self.path}: no tensor {n}")
        gate, up, down = (self.quant_method(n, device) for n in names)
        return MoEExperts(down, gate, up)

    def close(self):
        self._mm.close()
        self._f.close()
