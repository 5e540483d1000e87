"""Builds the drop-in proof: the reference's own sources, UNMODIFIED and compiled where they lie, on top of this
repository's libraries. Two families of executables land in tests/dropin/_built/ (git-ignored; they travel with
the source tree like the other built files):

  api_<test>   a test source of the reference (tests/unit, tests/kv, tests/kernel) compiled against THIS
               repository's public headers (include/scicompute_attention) and linked to libsci_attention.so:
               the outer seam - callers of the reference's C++ API switch libraries without touching their code.
  ref_<test>   the same test source compiled against the REFERENCE's headers and linked to
               libsci_attention_refhost.so = the reference's unmodified host layer (src/api, src/runtime,
               src/backends/*_backend.cpp, src/kv_cache/*.cpp) + tests/dropin/ref_launch_bindings.cpp (the launch
               functions forwarded to libsca_b200.so): the inner seam - the reference keeps its own dispatcher,
               backends and KV cache and only swaps its CUDA translation units for the C ABI.

The reference's own callers - examples/example_attention.cpp, examples/rollout_engine_stub.cpp and the benchmark
harness benchmarks/benchmark_attention.cu (both families), benchmarks/benchmark_naive.cu (ref family only: it calls
the naive launch functions below the public API) - are built the same way, unmodified, as api_<name> / ref_<name>.

Both use tests/dropin/gtest/gtest.h in place of GoogleTest. The reference checkout is found through the
SCA_REFERENCE_ROOT environment variable (or a `reference` directory beside the repository); without one the
build is skipped and the tests that need the executables skip as well, unless the executables are already there.

    python tests/dropin/build_dropin.py [--force]
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(HERE, "_built")
PKG = os.path.join(ROOT, "scicompute_attention_b200")
INCLUDE = os.path.join(ROOT, "include")
INFRA = os.path.join(INCLUDE, "sci_infra")
REFHOST_LIB = os.path.join(OUT, "libsci_attention_refhost.so")

# src/CMakeLists.txt of the reference: SCI_ATTENTION_HOST_SOURCES (the three *_stub.cpp of its CPU-only build are
# what the bindings replace)
REF_HOST_SOURCES = [
    "api/status.cpp", "api/api_validate.cpp", "api/attention_api.cpp",
    "kv_cache/kv_cache.cpp", "kv_cache/block_manager.cpp", "kv_cache/paged_kv_cache.cpp",
    "runtime/capability.cpp", "runtime/workspace.cpp", "runtime/dispatcher.cpp", "runtime/backend_lookup.cpp",
    "runtime/scratch_pool.cpp",
    "backends/naive/naive_backend.cpp", "backends/tiled/tiled_backend.cpp", "backends/flash/flash_backend.cpp",
    "backends/decode/decode_backend.cpp", "backends/paged/paged_backend.cpp",
]
REF_TESTS = [
    "unit/test_capability.cpp", "unit/test_config.cpp", "unit/test_dispatch.cpp", "unit/test_status.cpp",
    "unit/test_tile_smem_calc.cpp",
    "kv/test_block_manager.cpp", "kv/test_kv_cache.cpp", "kv/test_paged_kv.cpp",
    "kernel/test_flash_correctness.cu", "kernel/test_decode_correctness.cu", "kernel/test_paged_correctness.cu",
    "kernel/test_naive_correctness.cu", "kernel/test_tiled_correctness.cu", "kernel/test_numerics.cu",
]


# the reference's callers outside its test tree: (path below the reference root, families)
REF_CALLERS = [
    ("examples/example_attention.cpp", ("api", "ref")),
    ("examples/rollout_engine_stub.cpp", ("api", "ref")),
    ("benchmarks/benchmark_attention.cu", ("api", "ref")),
    ("benchmarks/benchmark_naive.cu", ("ref",)),
]


def reference_root() -> str | None:
    for cand in (os.environ.get("SCA_REFERENCE_ROOT"), os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "src")) and os.path.isdir(os.path.join(cand, "tests")):
            return cand
    return None


def test_name(rel: str) -> str:
    return os.path.splitext(os.path.basename(rel))[0]


def executables() -> dict[str, str]:
    """name -> path of every executable this script produces (whether or not it exists yet)."""
    out = {}
    for rel in REF_TESTS:
        for family in ("api", "ref"):
            out[f"{family}_{test_name(rel)}"] = os.path.join(OUT, f"{family}_{test_name(rel)}")
    for rel, families in REF_CALLERS:
        for family in families:
            out[f"{family}_{test_name(rel)}"] = os.path.join(OUT, f"{family}_{test_name(rel)}")
    return out


def _cuda_home() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return os.path.dirname(os.path.dirname(nvcc))


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> bool:
    ref = reference_root()
    if ref is None:
        if verbose:
            print("build_dropin: no reference checkout (set SCA_REFERENCE_ROOT); skipped")
        return False
    kernel_lib = os.path.join(PKG, "libsca_b200.so")
    host_lib = os.path.join(PKG, "libsci_attention.so")
    for lib in (kernel_lib, host_lib):
        if not os.path.exists(lib):
            raise RuntimeError(f"{lib} is missing: run python -m scicompute_attention_b200.build first")
    os.makedirs(OUT, exist_ok=True)
    cxx = shutil.which("g++") or "g++"
    cuda = _cuda_home()
    headers = glob.glob(os.path.join(INCLUDE, "**", "*.h*"), recursive=True) + [os.path.join(HERE, "gtest", "gtest.h")]
    common = [cxx, "-std=c++20", "-O1", "-fPIC", "-w"]
    rpath = ["-Wl,-rpath,$ORIGIN", "-Wl,-rpath,$ORIGIN/../../../scicompute_attention_b200"]

    # ---- the reference's host layer on the C ABI -------------------------------------------------------------
    host_srcs = [os.path.join(ref, "src", s) for s in REF_HOST_SOURCES]
    own_srcs = [os.path.join(HERE, "ref_launch_bindings.cpp"), os.path.join(HERE, "probe_layout_check.cpp"),
                os.path.join(PKG, "csrc", "host", "sci_infra.cpp")]
    if force or _stale(REFHOST_LIB, host_srcs + own_srcs + headers + [kernel_lib]):
        ref_inc = ["-I", INFRA, "-I", os.path.join(ref, "include"), "-I", os.path.join(ref, "src"),
                   "-I", INCLUDE, "-I", os.path.join(cuda, "include")]
        objs, jobs = [], []
        for src in host_srcs + own_srcs:
            obj = os.path.join(OUT, "obj_" + os.path.basename(src) + ".o")
            objs.append(obj)
            jobs.append(common + ref_inc + ["-c", src, "-o", obj])
        with cf.ThreadPoolExecutor(max_workers=8) as pool:
            list(pool.map(_run, jobs))
        _run([cxx, "-shared", "-o", REFHOST_LIB] + objs +
             ["-L", PKG, "-l:libsca_b200.so", "-L", os.path.join(cuda, "lib64"), "-lcudart_static", "-lrt", "-ldl",
              "-lpthread"] + rpath)
        for obj in objs:
            os.remove(obj)
        if verbose:
            print("built", REFHOST_LIB)

    # ---- the reference's tests, twice ------------------------------------------------------------------------
    jobs = []
    for rel in REF_TESTS:
        src = os.path.join(ref, "tests", rel)
        name = test_name(rel)
        test_inc = ["-I", HERE, "-I", os.path.join(ref, "tests"), "-DGTEST_SHIM_MAIN",
                    f'-DSCA_PROJECT_ROOT="{ref}"', "-x", "c++", src, "-x", "none"]
        api_exe = os.path.join(OUT, "api_" + name)
        if force or _stale(api_exe, [src, host_lib] + headers):
            jobs.append(common + ["-I", INCLUDE, "-I", INFRA] + test_inc +
                        ["-o", api_exe, "-L", PKG, "-l:libsci_attention.so", "-l:libsca_b200.so"] + rpath)
        ref_exe = os.path.join(OUT, "ref_" + name)
        if force or _stale(ref_exe, [src, REFHOST_LIB] + headers):
            jobs.append(common + ["-I", os.path.join(ref, "include"), "-I", INFRA] + test_inc +
                        ["-o", ref_exe, "-L", OUT, "-l:libsci_attention_refhost.so", "-L", PKG, "-l:libsca_b200.so"] + rpath)
    # ---- the reference's examples and benchmark harness ------------------------------------------------------
    cudart = ["-L", os.path.join(cuda, "lib64"), "-lcudart_static", "-lrt", "-ldl", "-lpthread"]
    for rel, families in REF_CALLERS:
        src = os.path.join(ref, rel)
        name = test_name(rel)
        caller_inc = ["-I", ref, "-I", os.path.join(ref, "benchmarks"), "-I", os.path.join(ref, "tests"),
                      "-I", os.path.join(cuda, "include"), f'-DSCA_PROJECT_ROOT="{ref}"', "-x", "c++", src, "-x", "none"]
        if "api" in families:
            exe = os.path.join(OUT, "api_" + name)
            if force or _stale(exe, [src, host_lib] + headers):
                jobs.append(common + ["-I", INCLUDE, "-I", INFRA] + caller_inc +
                            ["-o", exe, "-L", PKG, "-l:libsci_attention.so", "-l:libsca_b200.so"] + cudart + rpath)
        if "ref" in families:
            exe = os.path.join(OUT, "ref_" + name)
            if force or _stale(exe, [src, REFHOST_LIB] + headers):
                jobs.append(common + ["-I", os.path.join(ref, "include"), "-I", os.path.join(ref, "src"), "-I", INFRA] +
                            caller_inc + ["-o", exe, "-L", OUT, "-l:libsci_attention_refhost.so", "-L", PKG,
                                          "-l:libsca_b200.so"] + cudart + rpath)
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=8) as pool:
            list(pool.map(_run, jobs))
    if verbose:
        print(f"build_dropin: {len(jobs)} executables rebuilt in {OUT}")
    return True


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
