"""A compiled C caller on the GPU: tests/abi/gpu_abi.c links libqk_kernels.so, runs the
float64 device product and the resident factorized layer and compares them with its own C
loops (whose arithmetic the CPU suite checks against the oracle).  Sorts after the other test
files, so that a run which stops at the first failure has already run them."""

import os
import shutil
import subprocess

import pytest

from conftest import ROOT
from quantibbler_b200 import _build, _lib

pytestmark = pytest.mark.gpu


def test_c_program_runs_the_device_entry_points(tmp_path):
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    _lib.lib()                      # the library the other tests loaded; never rebuilt here
    lib_dir = os.path.dirname(_build.LIB_PATH)
    exe = tmp_path / "gpu_abi"
    res = subprocess.run(
        [gcc, "-std=c99", "-Wall", "-Wextra", "-I", os.path.join(ROOT, "include"),
         os.path.join(ROOT, "tests", "abi", "gpu_abi.c"), "-L", lib_dir, "-lqk_kernels", "-lm",
         f"-Wl,-rpath,{lib_dir}", "-o", str(exe)], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "gpu ABI ok" in run.stdout
