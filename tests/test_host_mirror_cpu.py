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
