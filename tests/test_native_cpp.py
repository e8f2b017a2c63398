"""Builds and runs the C++ unit tests (and micro-benchmark) of the dynamic-embedding library."""
import os
import shutil
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
CPU = os.path.join(os.path.dirname(HERE), "torchrec_b200", "csrc", "cpu")


@pytest.mark.skipif(shutil.which("g++") is None, reason="no C++ compiler")
def test_native_library_cpp_suite(tmp_path):
    exe = str(tmp_path / "test_tde")
    cmd = ["g++", "-std=c++17", "-O2", "-pthread", f"-I{CPU}", os.path.join(CPU, "tests", "test_tde.cpp"), os.path.join(CPU, "tde_id_transformer.cpp"),
           os.path.join(CPU, "tde_io.cpp"), "-ldl", "-o", exe]
    build = subprocess.run(cmd, capture_output=True, text=True)
    assert build.returncode == 0, build.stderr
    run = subprocess.run([exe, "--bench"], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "all native checks passed" in run.stdout and "BENCH id_transformer" in run.stdout


@pytest.mark.skipif(shutil.which("g++") is None, reason="no C++ compiler")
def test_serving_runtime_cpp_suite(tmp_path):
    """The batching queue of the serving runtime, driven from C++ (merging, result routing, limits, producer / consumer threads)."""
    import sysconfig

    import torch
    from torch.utils import cpp_extension

    exe = str(tmp_path / "test_inference_runtime")
    lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    inc = [p for p in cpp_extension.include_paths() if "cuda" not in os.path.basename(p.rstrip("/"))] + [sysconfig.get_paths()["include"]]
    cmd = (["g++", "-std=c++17", "-O1", "-pthread", "-D_GLIBCXX_USE_CXX11_ABI=1"] + [f"-I{p}" for p in inc]
           + [os.path.join(CPU, "tests", "test_inference_runtime.cpp"), f"-L{lib}", "-ltorch", "-ltorch_cpu", "-lc10", f"-Wl,-rpath,{lib}", "-o", exe])
    build = subprocess.run(cmd, capture_output=True, text=True)
    assert build.returncode == 0, build.stderr[-3000:]
    run = subprocess.run([exe, "--bench"], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "all serving-runtime checks passed" in run.stdout and "BENCH batching_queue" in run.stdout
