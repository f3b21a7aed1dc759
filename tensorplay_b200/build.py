"""Compiles the CUDA sources under csrc/ into tensorplay_b200/libtpb200.so for sm_100a.

nvcc cross-compiles without a GPU, so this runs on any machine with the CUDA 12.9 toolkit.
The shared library exports exactly the C ABI declared in include/tpb200.h.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from concurrent.futures import ThreadPoolExecutor

_PKG = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_PKG, "csrc")
_ROOT = os.path.dirname(_PKG)
LIB_PATH = os.path.join(_PKG, "libtpb200.so")
# The same sources with -DTPB200_CHECKED: every global access range-checked (see include/tpb200.h).
# Relocatable device code, because the range table and the violation record are shared by all files.
LIB_PATH_CHECKED = os.path.join(_PKG, "libtpb200_checked.so")
# The same sources with -DTPB200_TRACE: phase stamps (%globaltimer) in the sampled-threshold top-k kernel
# and in the whole-tensor exchange, read by tensorplay_b200/trace.py.  A development build.
LIB_PATH_TRACE = os.path.join(_PKG, "libtpb200_trace.so")

SOURCES = ["api_common.cu", "reduce.cu", "topk.cu", "softmax.cu", "median.cu", "comm.cu", "copy.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build libtpb200.so")
    return exe


def _stale(lib: str = LIB_PATH) -> bool:
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    deps = [os.path.join(_CSRC, f) for f in os.listdir(_CSRC)]
    deps.append(os.path.join(_ROOT, "include", "tpb200.h"))
    return any(os.path.getmtime(d) > t for d in deps if os.path.isfile(d))


def build_library(force: bool = False, verbose: bool = False, checked: bool = False, trace: bool = False) -> str:
    """Build libtpb200.so (or, with checked=True, libtpb200_checked.so; with trace=True,
    libtpb200_trace.so) if it is missing or older than its sources; returns its path."""
    lib = LIB_PATH_CHECKED if checked else (LIB_PATH_TRACE if trace else LIB_PATH)
    if not force and not _stale(lib):
        return lib
    nvcc = _nvcc()
    # separately compiled device functions do not see their callers' launch bounds: one register cap for all
    # (40: the tightest launch bound in the sources, 512 threads x 3 CTAs per SM)
    extra = ["-DTPB200_CHECKED", "-rdc=true", "-maxrregcount=40"] if checked else (["-DTPB200_TRACE"] if trace else [])
    objdir = os.path.join(_PKG, "build_checked" if checked else ("build_trace" if trace else "build"))
    os.makedirs(objdir, exist_ok=True)
    srcs = [s for s in SOURCES if os.path.exists(os.path.join(_CSRC, s))]

    def compile_one(src: str) -> str:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", os.path.join(_CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=len(srcs)) as ex:
        objs = list(ex.map(compile_one, srcs))
    cmd = [nvcc, "-shared", "-o", lib, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return lib


if __name__ == "__main__":
    import sys

    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv, checked="--checked" in sys.argv,
                        trace="--trace" in sys.argv))
