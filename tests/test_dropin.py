"""The drop-in boundary on C++ callers: include/cudalm_b200_shims.hpp gives CUDALM's own
names and signatures over the C ABI.

* CPU: the shim header and a C++ caller of it compile.
* GPU: CUDALM's own kernel test (tests/cuda/test_int4_gemv_bf16.cpp: vectorised shapes,
  the zero group that must give exact zeros, misaligned pointers), compiled with the shim
  header in place of CUDALM's kernel and linked with this library, exits 0.  It is built
  where the CUDALM tree is present (oracle/Makefile -> oracle/_ref/) and travels as a
  binary.  The row-equals-single-call check of CUDALM's batch test
  (tests/cuda/test_qwen35_batch_kernels.cpp:88-134) is run by tests/dropin/batch_rows_via_shims.cpp.
"""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INCLUDE = os.path.join(ROOT, "include")
LIB_DIR = os.path.join(ROOT, "cudalm_agent_b200", "lib")
CALLER = os.path.join(ROOT, "tests", "dropin", "batch_rows_via_shims.cpp")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _nvcc():
    cand = os.path.join(CUDA, "bin", "nvcc")
    return cand if os.path.exists(cand) else shutil.which("nvcc")


def test_shim_header_and_caller_compile(tmp_path):
    cxx = shutil.which("g++")
    if cxx is None or not os.path.isdir(os.path.join(CUDA, "include")):
        pytest.skip("no host compiler or CUDA headers here")
    tu = tmp_path / "only_shims.cpp"
    tu.write_text('#include "cudalm_b200_shims.hpp"\nint main() { return 0; }\n')
    for src in (str(tu), CALLER):
        res = subprocess.run([cxx, "-std=c++17", "-Wall", "-Wextra", "-Werror", "-fsyntax-only",
                              f"-I{INCLUDE}", f"-I{CUDA}/include", src], capture_output=True, text=True)
        assert res.returncode == 0, res.stderr


@pytest.mark.gpu
def test_reference_kernel_test_passes_through_the_shims():
    exe = os.path.join(ROOT, "oracle", "_ref", "test_int4_gemv_bf16_dropin")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/test_int4_gemv_bf16_dropin was not built (needs the CUDALM tree: make -C oracle)")
    res = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "test_int4_gemv_bf16" in res.stdout + res.stderr


@pytest.mark.gpu
def test_batch_rows_equal_single_calls_through_the_shims(tmp_path):
    nvcc = _nvcc()
    assert nvcc, "nvcc is needed to build the C++ caller"
    exe = tmp_path / "batch_rows_via_shims"
    res = subprocess.run([nvcc, "-std=c++17", "-O2", "-Wno-deprecated-gpu-targets", f"-I{INCLUDE}", CALLER,
                          f"-L{LIB_DIR}", "-lcudalm_b200", "-Xlinker", "-rpath", "-Xlinker", LIB_DIR,
                          "-o", str(exe)], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "PASS" in run.stdout
