"""The lean RESCALE form of the tensor-core epilogue, checked on the host: the arithmetic lives in
__host__ __device__ functions (reference_model_b200/csrc/rescale_math.cuh), so nvcc builds the very code the kernels
run for the CPU and a small program compares it with apply_scale_32 (reference_model/src/quant_util.h:45-84)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _nvcc():
    for cand in ("/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    return None


@pytest.mark.skipif(_nvcc() is None, reason="needs nvcc to build the host side of the device header")
def test_lean_rescale_form_equals_apply_scale_32(tmp_path):
    exe = str(tmp_path / "rescale_rec_check")
    src = os.path.join(ROOT, "tests", "native", "rescale_rec_check.cu")
    build = subprocess.run([_nvcc(), "-O2", "-std=c++17", "-Wno-deprecated-gpu-targets", "-o", exe, src],
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert build.returncode == 0, build.stdout
    run = subprocess.run([exe, "400000"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert run.returncode == 0, run.stdout
    assert "mismatches=0" in run.stdout and "checked=" in run.stdout, run.stdout


@pytest.mark.skipif(_nvcc() is None, reason="needs nvcc to build the host side of the device header")
def test_invariant_division_equals_the_operator(tmp_path):
    """fastdiv_make / fastdiv_apply (the kernels' tile-number decode) against the / operator."""
    exe = str(tmp_path / "fastdiv_check")
    src = os.path.join(ROOT, "tests", "native", "fastdiv_check.cu")
    build = subprocess.run([_nvcc(), "-O2", "-std=c++17", "-Wno-deprecated-gpu-targets", "-o", exe, src],
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert build.returncode == 0, build.stdout
    run = subprocess.run([exe], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert run.returncode == 0 and "mismatches=0" in run.stdout, run.stdout
