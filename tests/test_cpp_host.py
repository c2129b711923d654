"""The C++ host shim (include/prichs_moe.hpp): it compiles against the C ABI everywhere, and on a GPU its own
test program (tests/cpp/test_moe_layer.cpp, modelled on the reference's GPU MoE test) passes."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "test_moe_layer")


def _compile(capi):
    lib_dir = os.path.dirname(capi.LIB_PATH)
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "cpp", "test_moe_layer.cpp"), "-o", EXE, "-L", lib_dir, "-lprichs_moe",
           f"-Wl,-rpath,{lib_dir}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    assert "warning" not in res.stderr, res.stderr


def test_cpp_shim_compiles_and_links(capi):
    _compile(capi)
    assert os.path.exists(EXE)


@pytest.mark.gpu
def test_cpp_moe_layer_program(capi):
    _compile(capi)
    res = subprocess.run([EXE], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "CPP_OK" in res.stdout
