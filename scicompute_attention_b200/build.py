"""In-tree build of the native libraries (no JIT cache: the built .so files sit next to the package
so that they travel with the source tree).

  libsca_b200.so      hand-written sm_100a CUDA behind the C ABI of include/sca_b200.h
  libsci_attention.so C++ host layer (public sca:: API, dispatcher, KV cache) on top of it

`python -m scicompute_attention_b200.build` builds both; `--force` rebuilds everything.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(ROOT, "build", "obj")
INCLUDE = os.path.join(ROOT, "include")
KERNEL_LIB = os.path.join(PKG, "libsca_b200.so")
HOST_LIB = os.path.join(PKG, "libsci_attention.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall", "--expt-relaxed-constexpr",
    "-I", INCLUDE, "-I", os.path.join(CSRC, "kernels"),
]
CXX_FLAGS = ["-O2", "-std=c++20", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wextra",
             "-I", INCLUDE, "-I", os.path.join(INCLUDE, "sci_infra"), "-I", os.path.join(CSRC, "host")]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")
    return exe


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps if os.path.exists(d))


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)


def _headers() -> list[str]:
    out = glob.glob(os.path.join(INCLUDE, "**", "*.h*"), recursive=True)
    out += glob.glob(os.path.join(CSRC, "**", "*.cuh"), recursive=True)
    out += glob.glob(os.path.join(CSRC, "**", "*.hpp"), recursive=True)
    out += glob.glob(os.path.join(CSRC, "**", "*.inc"), recursive=True)
    return out


def build_kernels(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    sources = sorted(glob.glob(os.path.join(CSRC, "kernels", "*.cu")))
    hdrs = _headers()
    nvcc = _nvcc()
    jobs = []
    objs = []
    for src in sources:
        obj = os.path.join(OBJ, os.path.basename(src) + ".o")
        objs.append(obj)
        if force or not _newer(obj, [src] + hdrs):
            jobs.append([nvcc] + NVCC_FLAGS + ["-c", src, "-o", obj])
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            list(pool.map(_run, jobs))
    if jobs or not os.path.exists(KERNEL_LIB):
        _run([nvcc, "-shared", "-o", KERNEL_LIB] + objs + ["-cudart", "static", "-ldl"])
    if verbose:
        print("built", KERNEL_LIB)
    return KERNEL_LIB


def build_host(force: bool = False, verbose: bool = False) -> str | None:
    sources = sorted(glob.glob(os.path.join(CSRC, "host", "*.cpp")))
    if not sources:
        return None
    os.makedirs(OBJ, exist_ok=True)
    hdrs = _headers()
    cxx = shutil.which("g++") or "g++"
    cuda_inc = os.path.join(os.path.dirname(os.path.dirname(_nvcc())), "include")
    jobs, objs = [], []
    for src in sources:
        obj = os.path.join(OBJ, "host_" + os.path.basename(src) + ".o")
        objs.append(obj)
        if force or not _newer(obj, [src] + hdrs):
            jobs.append([cxx] + CXX_FLAGS + ["-I", cuda_inc, "-c", src, "-o", obj])
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            list(pool.map(_run, jobs))
    if jobs or not os.path.exists(HOST_LIB) or not _newer(HOST_LIB, [KERNEL_LIB]):
        cuda_lib = os.path.join(os.path.dirname(os.path.dirname(_nvcc())), "lib64")
        _run([cxx, "-shared", "-o", HOST_LIB] + objs +
             ["-L", PKG, "-l:libsca_b200.so", "-L", cuda_lib, "-lcudart_static", "-lrt", "-ldl", "-lpthread",
              "-Wl,-rpath,$ORIGIN"])
    if verbose:
        print("built", HOST_LIB)
    return HOST_LIB


def build_cpp_tests(force: bool = False, verbose: bool = False) -> str | None:
    """tests/cpp/api_tests.cpp -> tests/cpp/api_tests (links the host library and, as the checker, the oracle)."""
    src = os.path.join(ROOT, "tests", "cpp", "api_tests.cpp")
    oracle_so = os.path.join(ROOT, "oracle", "liboracle.so")
    if not os.path.exists(src) or not os.path.exists(HOST_LIB):
        return None
    if not os.path.exists(oracle_so):
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "-s"], check=True)
    exe = os.path.join(ROOT, "tests", "cpp", "api_tests")
    deps = [src, os.path.join(ROOT, "tests", "cpp", "mini_test.hpp"), HOST_LIB, oracle_so] + _headers()
    if force or not _newer(exe, deps):
        cxx = shutil.which("g++") or "g++"
        cuda = os.path.dirname(os.path.dirname(_nvcc()))
        _run([cxx, "-O1", "-std=c++20", "-Wall", "-I", INCLUDE, "-I", os.path.join(INCLUDE, "sci_infra"),
              "-I", os.path.join(ROOT, "tests", "cpp"), "-I", os.path.join(cuda, "include"), src, "-o", exe,
              "-L", PKG, "-l:libsci_attention.so", "-l:libsca_b200.so", "-L", os.path.join(ROOT, "oracle"),
              "-l:liboracle.so", "-L", os.path.join(cuda, "lib64"), "-lcudart_static", "-lrt", "-ldl", "-lpthread",
              "-Wl,-rpath,$ORIGIN/../../scicompute_attention_b200", "-Wl,-rpath,$ORIGIN/../../oracle"])
    if verbose:
        print("built", exe)
    return exe


def build_examples(force: bool = False, verbose: bool = False) -> str | None:
    """examples/*.cpp -> examples/<name> (public C++ API only; bench_attention also uses CUDA events)."""
    if not os.path.exists(HOST_LIB):
        return None
    cxx = shutil.which("g++") or "g++"
    cuda = os.path.dirname(os.path.dirname(_nvcc()))
    last = None
    for src in sorted(glob.glob(os.path.join(ROOT, "examples", "*.cpp"))):
        exe = os.path.splitext(src)[0]
        if force or not _newer(exe, [src, HOST_LIB] + _headers()):
            _run([cxx, "-O2", "-std=c++20", "-Wall", "-I", INCLUDE, "-I", os.path.join(INCLUDE, "sci_infra"),
                  "-I", os.path.join(cuda, "include"), src, "-o", exe, "-L", PKG, "-l:libsci_attention.so",
                  "-l:libsca_b200.so", "-L", os.path.join(cuda, "lib64"), "-lcudart_static", "-lrt", "-ldl", "-lpthread",
                  "-Wl,-rpath,$ORIGIN/../scicompute_attention_b200"])
        if verbose:
            print("built", exe)
        last = exe
    return last


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force, verbose)
    build_host(force, verbose)
    build_cpp_tests(force, verbose)
    build_examples(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
