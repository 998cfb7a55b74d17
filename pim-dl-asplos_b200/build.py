"""Builds libpimdl_b200.so (CUDA kernels + C ABI) for sm_100a, in-tree, with nvcc.

The library links the CUDA runtime statically and resolves the one driver entry point it
needs (tensor-map encoding) at run time, so it loads on machines without a GPU driver -
which is what lets CPU-only checks verify that every declared symbol is exported.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libpimdl_b200.so")
HOST_LIB = os.path.join(HERE, "libpimdl_host.so")
TEST_AMM = os.path.join(HERE, "bin", "test_amm")
TUNER = os.path.join(HERE, "bin", "tuner")
TEST_LAYER = os.path.join(HERE, "bin", "test_transformer_layer")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared", "-cudart", "static"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built on this machine")
    return exe


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def cuda_sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def build_cuda(force: bool = False, verbose: bool = False) -> str:
    """One object per .cu (compiled in parallel, rebuilt only when it or a header changed), then one link."""
    srcs = cuda_sources()
    hdrs = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + \
        [os.path.join(HERE, "..", "include", "lutamm.h")]
    objdir = os.path.join(CSRC, "build")
    os.makedirs(objdir, exist_ok=True)
    compile_flags = [f for f in NVCC_FLAGS if f not in ("-shared", "-cudart", "static")]
    jobs, objs = [], []
    for src in srcs:
        obj = os.path.join(objdir, os.path.splitext(os.path.basename(src))[0] + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + hdrs):
            cmd = [_nvcc()] + compile_flags + (["-Xptxas", "-v"] if verbose else []) + ["-c", "-o", obj, src]
            jobs.append((src, subprocess.Popen(cmd)))
    failed = [src for src, p in jobs if p.wait() != 0]
    if failed:
        raise RuntimeError("nvcc failed for " + ", ".join(os.path.basename(f) for f in failed))
    if jobs or _stale(LIB, objs):
        subprocess.run([_nvcc(), "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a",
                        "-o", LIB] + objs, check=True)
    return LIB


def host_sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "host", "*.cpp")))


def build_host(force: bool = False) -> None:
    """C++ host layer above the C ABI (parser, amm_host shim, test_amm driver, tuner)."""
    hdir = os.path.join(CSRC, "host")
    if not os.path.isdir(hdir):
        return
    os.makedirs(os.path.join(HERE, "bin"), exist_ok=True)
    lib_srcs = [s for s in host_sources() if os.path.basename(s) not in ("test_amm.cpp", "auto_tuner.cpp", "test_transformer_layer.cpp")]
    deps = host_sources() + glob.glob(os.path.join(hdir, "*.h")) + [os.path.join(HERE, "..", "include", "lutamm.h")]
    common = ["g++", "-std=c++17", "-O2", "-Wall", "-fPIC", "-I", hdir, "-I", os.path.join(HERE, "..", "include")]
    rpath = ["-Wl,-rpath,$ORIGIN", "-Wl,-rpath,$ORIGIN/.."]
    if lib_srcs and (force or _stale(HOST_LIB, deps + [LIB])):
        subprocess.run(common + ["-shared", "-o", HOST_LIB] + lib_srcs + ["-L", HERE, "-lpimdl_b200"] + rpath, check=True)
    for exe, src in ((TEST_AMM, "test_amm.cpp"), (TUNER, "auto_tuner.cpp"), (TEST_LAYER, "test_transformer_layer.cpp")):
        sp = os.path.join(hdir, src)
        if os.path.exists(sp) and (force or _stale(exe, deps + [LIB])):
            subprocess.run(common + ["-o", exe, sp, "-L", HERE, "-lpimdl_host", "-lpimdl_b200", "-lpthread"] + rpath,
                           check=True)


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cuda(force, verbose)
    build_host(force)


if __name__ == "__main__":
    import sys
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB)
