"""The C++ host layer (include/hanzoquant_b200.hpp): compiles against the C ABI without a GPU; on a GPU its test
program reproduces the reference's known-answer tests through `QuantMethod` / `moe_router_topk`."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "host_mirror_test.cpp")
OUT_DIR = os.path.join(ROOT, "tests", "cpp", "_build")
EXE = os.path.join(OUT_DIR, "host_mirror_test")


def build_exe():
    import __graft_entry__ as g
    g.build()
    os.makedirs(OUT_DIR, exist_ok=True)
    libdir = os.path.join(ROOT, "engine_b200")
    cmd = ["nvcc", "-std=c++17", "-O1", "-x", "cu", "-gencode", "arch=compute_100a,code=sm_100a",
           "-I", os.path.join(ROOT, "include"), SRC, "-o", EXE, "-L", libdir, "-lhanzoquant_b200",
           "-Xlinker", f"-rpath={libdir}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return EXE


def test_cpp_host_layer_compiles_and_links():
    build_exe()
    assert os.path.exists(EXE)


@pytest.mark.gpu
def test_cpp_host_layer_known_answers():
    exe = build_exe()
    res = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "host mirror ok" in res.stdout
