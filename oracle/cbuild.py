"""Builds and loads the C restatement of the oracle (oracle/hq_oracle.c) -- test infrastructure, see that file."""
import ctypes as C
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "libhq_oracle.so")
SRC = os.path.join(HERE, "hq_oracle.c")


def build(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(SRC):
        # -march is left at the baseline ISA so the library built on one machine runs on another
        cmd = ["gcc", "-O3", "-fopenmp", "-fPIC", "-shared", "-mavx2", "-mfma", "-o", LIB, SRC, "-lm"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("gcc failed:\n" + res.stderr)
    return LIB


_lib = None


def lib():
    global _lib
    if _lib is None:
        h = C.CDLL(build())
        P, I32, I64 = C.c_void_p, C.c_int32, C.c_int64
        h.oracle_linear.argtypes = [I32, P, P, P, P, P, I64, I64, I64, I32]
        h.oracle_linear.restype = None
        h.oracle_gather.argtypes = [I32, P, P, P, P, P, I64, I64, I32, P, P, P, I32]
        h.oracle_gather.restype = None
        h.oracle_max_threads.restype = I32
        _lib = h
    return _lib


FMT = {"Q8_0": 0, "Q4_K": 1, "FP8": 2, "MXFP4": 3, "Q6_K": 4, "Q5_K": 5, "Q4_0": 6, "Q5_0": 7, "Q4_1": 8, "Q5_1": 9,
       "Q2_K": 10, "Q3_K": 11}


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def linear(fmt: str, w, scales, bias, x, threads: int = 0):
    """x f32 [M, K], w uint8 [N, row_bytes] -> f32 [M, N]."""
    import numpy as np
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w)
    m, k = x.shape
    n = w.shape[0]
    y = np.empty((m, n), np.float32)
    sc = None if scales is None else np.ascontiguousarray(scales)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    lib().oracle_linear(FMT[fmt], _p(w), _p(sc), _p(b), _p(x), _p(y), n, k, m, threads)
    return y


def gather(fmt: str, w, scales, bias, x, n_experts, bounds, xrows, orows, n_out_rows, threads: int = 0):
    """Expert-grouped projection: w uint8 [E, N, row_bytes]; x f32 [rows, K]; returns f32 [n_out_rows, N]."""
    import numpy as np
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w)
    k = x.shape[1]
    n = w.shape[1]
    out = np.zeros((n_out_rows, n), np.float32)
    sc = None if scales is None else np.ascontiguousarray(scales)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    bounds = np.ascontiguousarray(bounds, dtype=np.int32)
    xrows = np.ascontiguousarray(xrows, dtype=np.int32)
    orows = np.ascontiguousarray(orows, dtype=np.int32)
    lib().oracle_gather(FMT[fmt], _p(w), _p(sc), _p(b), _p(x), _p(out), n, k, n_experts, _p(bounds), _p(xrows),
                        _p(orows), threads)
    return out
