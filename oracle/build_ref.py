"""Compile the reference's own C++/OpenMP split finder into ``oracle/_ref/``.

TEST INFRASTRUCTURE ONLY (see ``packboost_oracle.py``).  The two source files are compiled
where they lie in the reference checkout; nothing of them is copied into this repository and
the output directory is git-ignored:

    python oracle/build_ref.py /path/to/reference

    g++ -O3 -std=c++17 -fopenmp -fPIC -shared $(python -m pybind11 --includes) \
        <ref>/packboost/backends/cpu/frontier_cpu.cpp <ref>/packboost/backends/bindings.cpp \
        -o oracle/_ref/_backend<EXT_SUFFIX>

(the reference's own ``setup_native.py`` does the same through setuptools; without
``PACKBOOST_ENABLE_CUDA`` the module registers the CPU functions only,
``packboost/backends/bindings.cpp:11-24``).
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
SOURCES = ("packboost/backends/cpu/frontier_cpu.cpp", "packboost/backends/bindings.cpp")


def output_path() -> str:
    return os.path.join(OUT_DIR, "_backend" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))


def build(ref_root: str, force: bool = False) -> str | None:
    """Returns the path of the built module, or ``None`` when the sources are not there."""
    srcs = [os.path.join(ref_root, s) for s in SOURCES]
    if not all(os.path.exists(s) for s in srcs):
        return None
    out = output_path()
    if not force and os.path.exists(out) and all(os.path.getmtime(out) >= os.path.getmtime(s) for s in srcs):
        return out
    import pybind11
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else (shutil.which("g++") or "g++")
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = [cxx, "-O3", "-std=c++17", "-fopenmp", "-fPIC", "-shared", "-I" + pybind11.get_include(),
           "-I" + sysconfig.get_paths()["include"], *srcs, "-o", out]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("compiling the reference's C++ split finder failed")
    return out


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python oracle/build_ref.py /path/to/reference")
    print(build(sys.argv[1], force=True))
