"""The C++ mirror of the reference's operator interface compiles against the C ABI and keeps the reference's error
behaviour on the host (no GPU needed: every checked path returns before a launch)."""
import os
import shutil
import subprocess

import pytest

from helpers import ROOT, pkg


@pytest.mark.skipif(shutil.which("nvcc") is None, reason="needs the CUDA toolkit headers")
def test_host_mirror_compiles_and_rejects_bad_arguments(tmp_path):
    pkg().build()
    libdir = os.path.join(ROOT, "ninfer-3080-iq3_s_b200")
    exe = str(tmp_path / "host_mirror_check")
    subprocess.run(["nvcc", "-std=c++17", "-x", "cu", "-I", os.path.join(libdir, "host"), os.path.join(ROOT, "tests", "cpp", "host_mirror_check.cpp"),
                    "-o", exe, "-L", libdir, "-lkvarn_b200", "-Xlinker", "-rpath", "-Xlinker", libdir], check=True)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "host mirror: ok" in r.stdout


@pytest.mark.skipif(shutil.which("nvcc") is None, reason="needs the CUDA toolkit headers")
def test_engine_shim_compiles_and_refuses_what_the_reference_refuses(tmp_path):
    pkg().build()
    libdir = os.path.join(ROOT, "ninfer-3080-iq3_s_b200")
    exe = str(tmp_path / "engine_shim_check")
    subprocess.run(["nvcc", "-std=c++17", "-x", "cu", "-I", os.path.join(libdir, "host"), os.path.join(ROOT, "tests", "cpp", "engine_shim_check.cpp"),
                    "-o", exe, "-L", libdir, "-lkvarn_b200", "-Xlinker", "-rpath", "-Xlinker", libdir], check=True)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "engine shim: ok" in r.stdout


@pytest.mark.gpu
@pytest.mark.skipif(shutil.which("nvcc") is None, reason="needs nvcc on the GPU machine")
def test_engine_shim_on_the_gpu_equals_the_c_abi(tmp_path):
    """The engine-shaped launchers (Tensor / PagedKV*LayerView values, op-owned stage) against the C ABI called
    directly on a second, identical cache: prompt chunk, verify step, append + cached decode, bit for bit."""
    libdir = os.path.join(ROOT, "ninfer-3080-iq3_s_b200")
    pkg().capi.load()  # fails loudly if the library is missing
    exe = str(tmp_path / "engine_shim_gpu")
    subprocess.run(["nvcc", "-std=c++17", "-x", "cu", "-I", os.path.join(libdir, "host"), os.path.join(ROOT, "tests", "cpp", "engine_shim_gpu.cpp"),
                    "-o", exe, "-L", libdir, "-lkvarn_b200", "-Xlinker", "-rpath", "-Xlinker", libdir], check=True)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "engine shim on the GPU: ok" in r.stdout
