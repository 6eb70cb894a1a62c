"""Builds ``libvolta_b200.so`` in-tree with nvcc for sm_100a (the only target).

    python volta_b200/build.py [--force] [--verbose]

(run as a script: importing the ``volta_b200`` package itself needs the built library)

The library is plain CUDA C++ behind a C ABI (``include/volta_b200.h``); it does not link
against torch or Python.  Objects are compiled in parallel and linked with nvcc.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libvolta_b200.so")

SOURCES = ["api.cu", "multi_tensor.cu", "muon.cu", "ns_gemm_f32.cu", "ns_gemm_tc.cu", "exchange_fence.cu", "comm.cpp"]

# No --use_fast_math: the Adam/SGD kernels promise bit parity with IEEE f32 arithmetic,
# which needs precise division/sqrt and no flush-to-zero (nvcc's defaults, spelled out).
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-prec-div=true", "-prec-sqrt=true", "-ftz=false",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _deps_mtime() -> float:
    latest = 0.0
    for root in (CSRC, os.path.join(HERE, "..", "include")):
        for dirpath, _, files in os.walk(root):
            for f in files:
                latest = max(latest, os.path.getmtime(os.path.join(dirpath, f)))
    return max(latest, os.path.getmtime(__file__))


def _compile(src: str, verbose: bool) -> str:
    obj = os.path.join(OBJ_DIR, os.path.splitext(src)[0] + ".o")
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
    if src.endswith(".cpp"):
        cmd = [_nvcc(), "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-c", os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    log = os.path.join(OBJ_DIR, os.path.splitext(src)[0] + ".log")
    with open(log, "w") as fh:
        fh.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    if verbose:
        sys.stderr.write(r.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile and link the library if it is missing or older than its sources."""
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _deps_mtime():
        return LIB
    os.makedirs(OBJ_DIR, exist_ok=True)
    with cf.ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), SOURCES))
    tmp = LIB + f".tmp{os.getpid()}"
    cmd = [_nvcc(), "-shared", "-o", tmp, *objs, "-lcudart", "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, LIB)
    return LIB


CPP_TEST_SRC = os.path.join(HERE, "..", "tests", "cpp", "test_optimizers.cpp")
CPP_TEST_BIN = os.path.join(HERE, "..", "tests", "cpp", "test_optimizers.bin")


def build_cpp_tests(force: bool = False) -> str:
    """Compiles the C++ replay of the reference's optimizer tests against the C++ host mirror
    (include/volta_b200.hpp) and links it to the library."""
    src, out = os.path.abspath(CPP_TEST_SRC), os.path.abspath(CPP_TEST_BIN)
    hdr = os.path.join(HERE, "..", "include", "volta_b200.hpp")
    newest = max(os.path.getmtime(src), os.path.getmtime(hdr), os.path.getmtime(LIB))
    if not force and os.path.exists(out) and os.path.getmtime(out) >= newest:
        return out
    cuda_lib = os.path.join(os.path.dirname(os.path.dirname(os.path.realpath(_nvcc()))), "lib64") \
        if os.path.sep in _nvcc() else "/usr/local/cuda/lib64"
    cmd = ["g++", "-std=c++17", "-O2", "-I", os.path.join(HERE, "..", "include"), src, "-o", out,
           "-L", HERE, "-lvolta_b200", "-Wl,-rpath,$ORIGIN/../../volta_b200", "-L", cuda_lib,
           f"-Wl,-rpath,{cuda_lib}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"g++ failed on the C++ tests:\n{r.stdout}\n{r.stderr}")
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print(build_cpp_tests(force="--force" in sys.argv))
