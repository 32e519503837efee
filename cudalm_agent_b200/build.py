"""Builds the native library in-tree with nvcc for sm_100a.

    python -m cudalm_agent_b200.build

produces ``cudalm_agent_b200/lib/libcudalm_b200.so``.  The library is
self-contained (static CUDA runtime) and exports only the C ABI declared in
``include/cudalm_b200.h``.
"""
from __future__ import annotations

import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libcudalm_b200.so")

SOURCES = ["runtime.cu", "w4a16_linear.cu", "w4a16_tc.cu", "w4a16_direct.cu", "quantize.cu", "lm_head.cu", "sample.cu",
           "weights_v2.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-shared", "-cudart", "static",
]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(os.path.dirname(PKG), "include", "cudalm_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compiles the library if it is missing or older than its sources: one object
    per source file, compiled in parallel, then one link step."""
    if not force and not _stale():
        return LIB_PATH
    from concurrent.futures import ThreadPoolExecutor

    os.makedirs(LIB_DIR, exist_ok=True)
    obj_dir = os.path.join(LIB_DIR, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    srcs = [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h", ".hpp"))]
    headers.append(os.path.join(os.path.dirname(PKG), "include", "cudalm_b200.h"))
    newest_header = max(os.path.getmtime(h) for h in headers)
    compile_flags = [f for f in NVCC_FLAGS if f not in ("-shared",)]

    def compile_one(src: str):
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        if (not force and os.path.exists(obj)
                and os.path.getmtime(obj) > max(os.path.getmtime(src), newest_header)):
            return obj, 0, ""
        cmd = [_nvcc(), *compile_flags, "-c"]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        cmd += ["-o", obj, src]
        res = subprocess.run(cmd, capture_output=True, text=True)
        return obj, res.returncode, res.stdout + res.stderr

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(compile_one, srcs))
    for _, rc, out in results:
        if verbose or rc != 0:
            sys.stderr.write(out)
    if any(rc != 0 for _, rc, _ in results):
        raise RuntimeError("nvcc failed building libcudalm_b200.so")
    link = [_nvcc(), *NVCC_FLAGS, "-o", LIB_PATH, *[o for o, _, _ in results]]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed linking libcudalm_b200.so")
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force=True, verbose="-v" in sys.argv))
