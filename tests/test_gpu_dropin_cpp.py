"""The C++ drop-in: tests/cpp/dropin_test.cu is an ordinary Thrust program (device_vector,
thrust::device, thrust::cuda::par.on(stream), user functors, zip / transform / counting iterators)
compiled by nvcc with include/thrust_b200/thrust_overlay.cuh force-included.  It checks every
hot-path algorithm against a host computation and that the overlay, not the stock CUB path, served
all the calls."""
import os
import shutil
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_thrust_program_runs_on_overlay(tb, tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.isfile(nvcc):
        pytest.skip("nvcc is not available on this machine")
    exe = str(tmp_path / "dropin_test")
    cmd = [nvcc, "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "--extended-lambda", "-I" + os.path.join(ROOT, "include"),
           "-include", "thrust_b200/thrust_overlay.cuh", "-DTHRUST_B200_OVERLAY_EXPECTED", os.path.join(ROOT, "tests", "cpp", "dropin_test.cu"), "-o", exe]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout + r.stderr
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "all checks passed" in r.stdout, r.stdout + r.stderr
    assert "overlay served 44 calls" in r.stdout
