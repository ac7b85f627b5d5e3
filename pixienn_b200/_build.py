"""Builds ``pixienn_b200/lib/libpxe.so`` from ``csrc/`` with nvcc for sm_100a.

The library is built in-tree so that it travels with the source tree; there is no JIT step and
no fallback: importing :mod:`pixienn_b200.capi` without the built library raises.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(LIBDIR, "obj")
LIB = os.path.join(LIBDIR, "libpxe.so")
# The same sources with every global-memory access of every kernel checked against the caller's allocations
# (include/pxe_debug.h); slow, for tests on small shapes.
CHECKED_OBJDIR = os.path.join(LIBDIR, "obj_checked")
CHECKED_LIB = os.path.join(LIBDIR, "libpxe_checked.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

CU_SOURCES = ["pxe_api.cu", "pxe_epilogue.cu", "pxe_pool.cu", "pxe_move.cu", "pxe_heads.cu", "pxe_compat.cu", "pxe_nms_gpu.cu", "pxe_nhwc.cu", "pxe_stem.cu", "pxe_backward.cu", "pxe_loss.cu", "pxe_bn_train.cu"]
CXX_SOURCES = ["pxe_nms.cpp", "pxe_plan.cpp"]
HEADERS = [os.path.join(CSRC, "pxe_common.cuh"), os.path.join(INCLUDE, "pxe.h"),
           os.path.join(INCLUDE, "pxe_compat.hpp"), os.path.join(INCLUDE, "pxe_plan.h"),
           os.path.join(INCLUDE, "pxe_debug.h")]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "-I", INCLUDE, "-I", CSRC]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def _digest(paths, extra) -> str:
    h = hashlib.sha256()
    for p in paths:
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS + extra).encode())
    return h.hexdigest()


def _compile(src: str, verbose: bool, checked: bool = False) -> str:
    path = os.path.join(CSRC, src)
    extra = ["-DPXE_BOUNDS_CHECK"] if checked else []
    obj = os.path.join(CHECKED_OBJDIR if checked else OBJDIR, os.path.splitext(src)[0] + ".o")
    stamp = obj + ".sha"
    want = _digest([path] + HEADERS, extra)
    if os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == want:
        return obj
    if src.endswith(".cu"):
        cmd = [_nvcc()] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", path, "-o", obj]
    else:
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-I", INCLUDE] + extra + ["-c", path, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose and res.stderr:
        sys.stderr.write(res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"compiling {src} failed:\n{res.stdout}\n{res.stderr}")
    with open(stamp, "w") as f:
        f.write(want)
    return obj


def build(verbose: bool = False, force: bool = False, checked: bool = False) -> str:
    """Compile whatever changed and link the shared library (``checked``: the bounds-checked one).  Returns its path."""
    objdir, lib = (CHECKED_OBJDIR, CHECKED_LIB) if checked else (OBJDIR, LIB)
    os.makedirs(objdir, exist_ok=True)
    if force:
        for f in os.listdir(objdir):
            os.remove(os.path.join(objdir, f))
    srcs = CU_SOURCES + CXX_SOURCES
    with cf.ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 2)) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose, checked), srcs))
    newest = max(os.path.getmtime(o) for o in objs)
    if not os.path.exists(lib) or os.path.getmtime(lib) < newest:
        cmd = [_nvcc(), "-shared", "-o", lib] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"linking {os.path.basename(lib)} failed:\n{res.stdout}\n{res.stderr}")
    return lib


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv, checked="--checked" in sys.argv))
