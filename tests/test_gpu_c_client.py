"""The C ABI used from plain C: tests/c_abi_client.c is compiled against include/dd_b200.h and the
CUDA runtime, linked with libdd_b200.so, and run (reorder, activation, bias add, reduction, a
refused call).  No Python, torch or ctypes on that path."""
import os
import shutil
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_c_client(tmp_path):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not found")
    lib_dir = os.path.join(ROOT, "deep_diamond_b200")
    exe = str(tmp_path / "c_abi_client")
    build = subprocess.run([nvcc, "-x", "c", os.path.join(ROOT, "tests", "c_abi_client.c"), "-o", exe,
                            "-L" + lib_dir, "-ldd_b200", "-Xlinker", "-rpath," + lib_dir, "-lm"],
                           capture_output=True, text=True)
    assert build.returncode == 0, build.stdout + build.stderr
    run = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "reorder: ok (transform/tile" in run.stdout
    assert "relu + bias: ok (optensor/flat-bcast)" in run.stdout
    assert "reduce: ok (reduce/" in run.stdout
    assert "shape mismatch -> DD_STATUS_BAD_PARAM" in run.stdout
