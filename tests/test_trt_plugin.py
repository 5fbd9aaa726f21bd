"""The TensorRT plugin source (gtr_b200/csrc/gla_plugin_b200.cu) without TensorRT: compiled against a stand-in
NvInfer.h (tests/trt_stub) and driven on the CPU through creator -> plugin -> build / runtime capabilities.
What needs TensorRT itself (engine build, trtexec timing) is unavailable on this image."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_plugin_source_compiles_and_honours_the_reference_contract(tmp_path):
    from gtr_b200 import build
    lib = build.build()
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    stub, inc = os.path.join(ROOT, "tests", "trt_stub"), os.path.join(ROOT, "include")
    obj, exe = str(tmp_path / "plugin.o"), str(tmp_path / "driver")
    subprocess.run(["g++", "-std=c++17", "-x", "c++", "-I", stub, "-I", inc, "-I", cuda_inc, "-c",
                    os.path.join(ROOT, "gtr_b200", "csrc", "gla_plugin_b200.cu"), "-o", obj], check=True)
    subprocess.run(["g++", "-std=c++17", "-I", stub, "-I", inc, os.path.join(stub, "plugin_driver.cpp"), obj, lib,
                    f"-Wl,-rpath,{os.path.dirname(lib)}", "-o", exe], check=True)
    run = subprocess.run([exe], capture_output=True, text=True)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "0 failure(s)" in run.stdout and "FAIL" not in run.stdout


def test_plugin_source_is_empty_without_tensorrt_headers(tmp_path):
    """Without NvInfer.h on the include path the file must still compile (to nothing)."""
    obj = str(tmp_path / "empty.o")
    subprocess.run(["g++", "-std=c++17", "-x", "c++", "-I", os.path.join(ROOT, "include"), "-c",
                    os.path.join(ROOT, "gtr_b200", "csrc", "gla_plugin_b200.cu"), "-o", obj], check=True)
    syms = subprocess.run(["nm", obj], capture_output=True, text=True).stdout
    assert "gla_b200_trt_plugin_creator" not in syms
