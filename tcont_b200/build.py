"""Builds the engine's shared libraries in-tree with nvcc for sm_100a.

    tcont_b200/libtcontb.so   C ABI (include/tcontb.h): planner + CUDA kernels
    tcont_b200/libtcont.so    C++ surface of include/tcont.hpp on top of the C ABI

Objects go to tcont_b200/_build/.  A source is recompiled when it is newer than its object.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "_build")
LIB_C = os.path.join(PKG, "libtcontb.so")
LIB_CPP = os.path.join(PKG, "libtcont.so")

CORE_SOURCES = ["planner.cpp", "api.cpp", "simt_contract.cu", "dmma_f64.cu", "dmma_tma_f64.cu", "transpose.cu", "umma_tf32.cu", "splitk_reduce.cu", "no_alloc.cu", "peaks.cu"]
SHIM_SOURCES = ["tcont_shim.cpp"]
HEADERS = ["planner.hpp", "kernels.hpp", "tile_common.cuh", os.path.join(ROOT, "include", "tcontb.h"), os.path.join(ROOT, "include", "tcont.hpp"),
           os.path.join(ROOT, "include", "tcont_b200", "tcont_api.hpp")]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "-I" + os.path.join(ROOT, "include")]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the engine has CUDA kernels only and cannot be built without it")
    return exe


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def _compile(src: str, verbose: bool) -> str:
    path = os.path.join(CSRC, src)
    obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
    hdrs = [h if os.path.isabs(h) else os.path.join(CSRC, h) for h in HEADERS]
    if _stale(obj, [path] + hdrs):
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", path, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr)
    return obj


def build(verbose: bool = False) -> None:
    os.makedirs(OBJ, exist_ok=True)
    core = [s for s in CORE_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    shim = [s for s in SHIM_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose), core + shim))
    core_objs, shim_objs = objs[:len(core)], objs[len(core):]
    if _stale(LIB_C, core_objs):
        subprocess.run([_nvcc()] + NVCC_FLAGS[:2] + ["-shared", "-o", LIB_C] + core_objs + ["-cudart", "static"], check=True)
    if shim_objs and _stale(LIB_CPP, shim_objs + [LIB_C]):
        subprocess.run([_nvcc()] + NVCC_FLAGS[:2] + ["-shared", "-o", LIB_CPP] + shim_objs +
                       ["-L" + PKG, "-ltcontb", "-Xlinker", "-rpath=$ORIGIN", "-cudart", "static"], check=True)


if __name__ == "__main__":
    import sys
    build(verbose="-v" in sys.argv)
    print("built", LIB_C, LIB_CPP if os.path.exists(LIB_CPP) else "")
