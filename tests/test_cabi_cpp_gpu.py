"""The C ABI from C++: a host program with no torch in it (tests/cabi/host_driver.cpp) is compiled
against include/nvfp4_b200.h, linked with the shipped library and run; its cases mirror the
reference's Catch2 tests of the same launchers."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "blackwell_diffusion_rtx6000_5090_i2v_b200")


def _build(tmp_path):
    nvcc = next((c for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc"))
                 if c and os.path.exists(c)), None)
    if nvcc is None:
        pytest.skip("nvcc not found")
    exe = os.path.join(str(tmp_path), "host_driver")
    cmd = [nvcc, "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "cabi", "host_driver.cpp"), "-o", exe,
           "-L", PKG, "-lnvfp4_b200", "-Xlinker", "-rpath", "-Xlinker", PKG]
    if os.path.exists("/usr/bin/g++"):
        cmd[1:1] = ["-ccbin", "/usr/bin/g++"]
    subprocess.run(cmd, check=True)
    return exe


def test_host_driver_compiles_and_links(tmp_path):
    """No GPU needed: the header is valid C++ and every symbol the driver uses resolves."""
    assert os.path.exists(_build(tmp_path))


@pytest.mark.gpu
def test_host_driver_runs(tmp_path):
    exe = _build(tmp_path)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    print(r.stdout)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "0 failure(s)" in r.stdout and "FAIL" not in r.stdout
