"""Build ``libpackboost_b200.so`` (sm_100a only) in-tree with nvcc.

Run as ``python -m packboost_b200.build``.  The library is a plain C-ABI shared
object (no Python or torch dependency); ``packboost_b200.backends`` loads it
with ctypes.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_NAME = "libpackboost_b200.so"
LIB_PATH = os.path.join(HERE, LIB_NAME)

SOURCES = ["api.cu", "hist.cu", "score.cu", "frontier.cu", "pack.cu", "predict.cu", "metrics.cu", "comm.cu"]
# The scorer, and the histogram kernel whose flush computes the per-era gains, must round every
# product and sum separately (no fused multiply-add) to keep the float32 operation order of the
# algorithm they implement.
EXTRA = {"score.cu": ["-fmad=false"], "hist.cu": ["-fmad=false"]}

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set CUDA_HOME")
    return cand


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


DEBUG_LIB_PATH = os.path.join(HERE, "libpackboost_b200_dbg.so")


def build(force: bool = False, verbose: bool = False, debug_bounds: bool = False) -> str:
    """``debug_bounds``: build the variant with the kernels' index checks compiled in
    (``-DPB_DEBUG_BOUNDS``, see ``pb_debug_flags`` in the header) as ``libpackboost_b200_dbg.so``
    beside the regular library (``PACKBOOST_DEBUG_LIB=1`` makes ``packboost_b200.backends`` load it)."""
    nvcc = _nvcc()
    objdir = os.path.join(HERE, "build_dbg" if debug_bounds else "build")
    lib_path = DEBUG_LIB_PATH if debug_bounds else LIB_PATH
    os.makedirs(objdir, exist_ok=True)
    headers = [os.path.join(CSRC, "common.cuh"), os.path.join(CSRC, "des_math.cuh"),
               os.path.join(HERE, "..", "include", "packboost_b200.h")]
    objs = []
    log_lines = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(objdir, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _stale(o, [s] + headers):
            cmd = [nvcc, "-c", s, "-o", o] + ARCH + COMMON + EXTRA.get(src, []) + (["-DPB_DEBUG_BOUNDS"] if debug_bounds else [])
            res = subprocess.run(cmd, capture_output=True, text=True)
            log_lines.append("$ " + " ".join(cmd))
            log_lines.append(res.stderr)
            if res.returncode != 0:
                sys.stderr.write(res.stdout + res.stderr)
                raise RuntimeError(f"nvcc failed on {src}")
    if force or _stale(lib_path, objs):
        cmd = [nvcc, "-shared", "-o", lib_path] + objs + ARCH + ["-ldl"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link failed")
    if log_lines:
        with open(os.path.join(objdir, "ptxas.log"), "w") as fh:
            fh.write("\n".join(log_lines))
        if verbose:
            print("\n".join(log_lines))
    return lib_path


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, debug_bounds="--debug-bounds" in sys.argv))
