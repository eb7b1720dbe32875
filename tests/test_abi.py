"""CPU-side checks of the boundary: the library builds, loads, exports every symbol the header declares, and
rejects bad arguments on the host before any launch (no GPU needed)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as g
    g.build()
    from engine_b200 import _lib as L
    return L.lib()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "hanzoquant_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hq_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    from engine_b200 import _lib as L
    names = declared_symbols()
    assert len(names) >= 14
    for n in names:
        assert hasattr(lib, n), n
        assert n in L.SIGNATURES, f"{n} has no ctypes signature"
    assert lib.hq_abi_version() == 3
    assert lib.hq_error_string(-2).decode() == "unsupported size"


def test_every_reference_named_symbol_is_exported(lib):
    text = open(os.path.join(ROOT, "include", "hanzoquant_compat.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"#define[^\n]*(\\\n[^\n]*)*", "", text)          # macro bodies declare nothing by themselves
    names = set(re.findall(r"\b((?:launch_|moe_router_topk_|gptoss_swiglu_|fused_glu_|mxfp4_get_)[a-z0-9_]+)\s*\(", text))
    names |= set(re.findall(r"HQ_COMPAT_[A-Z0-9_]+\((\w+)\);", text))
    assert len(names) >= 50, sorted(names)
    for n in sorted(names):
        assert hasattr(lib, n), n


def test_host_side_argument_errors(lib):
    from engine_b200 import _lib as L
    w = L.HqWeight(L.FMT_Q8_0, 1, 64, 100, 16, 0, 0, 0, 0)           # K % 256 != 0
    assert lib.hq_linear_forward(C.byref(w), 16, L.DT_BF16, 100, 16, L.DT_F32, 64, 1, None, None) == -2
    w = L.HqWeight(99, 1, 64, 256, 16, 0, 0, 0, 0)                     # no such format
    assert lib.hq_linear_forward(C.byref(w), 16, L.DT_BF16, 256, 16, L.DT_F32, 64, 1, None, None) == -4
    w = L.HqWeight(L.FMT_Q8_0, 1, 64, 256, 0, 0, 0, 0, 0)
    assert lib.hq_linear_forward(C.byref(w), 16, L.DT_BF16, 256, 16, L.DT_F32, 64, 1, None, None) == -1
    w = L.HqWeight(L.FMT_Q8_0, 1, 64, 256, 16, 0, 0, 0, 0)
    assert lib.hq_linear_forward(C.byref(w), 8, L.DT_BF16, 256, 16, L.DT_F32, 64, 1, None, None) == -3
    assert lib.hq_linear_forward(C.byref(w), 16, L.DT_BF16, 256, 16, L.DT_F32, 64, 0, None, None) == 0  # m = 0
    w = L.HqWeight(L.FMT_FP8_BLOCK, 1, 128, 256, 16, 0, 0, 0, 0)     # FP8 needs scales
    assert lib.hq_linear_forward(C.byref(w), 16, L.DT_BF16, 256, 16, L.DT_F32, 128, 1, None, None) == -1
    a = L.HqRouterArgs(2048, 8, 1, 0, 1, 0, 0, 0, 0, 1.0, 0, 0)
    assert lib.hq_router_topk(16, L.DT_F32, 4, C.byref(a), 16, 16, None) == -2
    assert lib.hq_moe_dispatch_workspace_bytes(4096, 8, 128) > 0
    assert lib.hq_moe_dispatch_build(16, 4, 8, 128, 16, 16, 16, 16, 16, 8, None) == -6
    assert lib.hq_fp8_vector_quant(16, L.DT_F32, 100, 16, 16, None) == -2


def test_package_has_no_cpu_fallback():
    import torch
    import engine_b200 as hq
    with pytest.raises(hq.HqError):
        hq.GgufMatMul(torch.zeros((4, 272), dtype=torch.uint8), "Q8_0", 256)
    with pytest.raises(hq.HqError):
        hq.moe_router_topk(torch.zeros((2, 8)), hq.MoeRouterTopKConfig(2))
    # the product never imports the oracle
    for dirpath, _, files in os.walk(os.path.join(ROOT, "engine_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                assert "oracle" not in open(os.path.join(dirpath, f)).read(), f


def test_split_k_scratch_plan_is_host_arithmetic(lib):
    # the scratch a dense decode call asks for: nothing while the activations of the whole K stay staged, else
    # 1024 bytes of arrival counters + 512 bytes per (16-row item, K slice) with two to eight slices
    from engine_b200 import _lib as L

    def need(fmt, n, k, m):
        w = L.HqWeight(fmt, 1, n, k, 16, 0, 0, 0, 0)
        return lib.hq_linear_workspace_bytes(C.byref(w), m)

    assert need(L.FMT_Q8_0, 4096, 4096, 1) == 0
    assert need(L.FMT_Q8_0, 128256, 4096, 8) == 0
    for n in (1000, 4096):
        for m in (1, 4, 8):
            b = need(L.FMT_Q8_0, n, 14336, m)
            items = (n + 15) // 16
            assert b > 1024 and (b - 1024) % (items * 512) == 0, (n, m, b)
            assert 2 <= (b - 1024) // (items * 512) <= 8
            assert b == need(L.FMT_Q8_0, n, 14336, m)
    # more than eight rows are served as several row groups of one launch: one item per (row group, 16 rows)
    b = need(L.FMT_Q8_0, 4096, 14336, 11)
    assert b > 1024 and (b - 1024) % (2 * 256 * 512) == 0
    assert need(L.FMT_Q4_K, 4096, 14336, 4) > 1024
    bad = L.HqWeight(L.FMT_Q8_0, 1, 64, 100, 16, 0, 0, 0, 0)
    assert lib.hq_linear_workspace_bytes(C.byref(bad), 1) == 0
