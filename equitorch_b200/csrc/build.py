"""Compile the CUDA sources of this directory into ``equitorch_b200/lib/libeqt_b200.so``.

    python -m equitorch_b200.csrc.build [--force] [--verbose]

Only sm_100a code is generated (``-gencode arch=compute_100a,code=sm_100a``).  The shared
library sits inside the package so that it travels with the source tree; nothing is
installed into site-packages.  ``nvcc`` cross-compiles without a GPU.
"""
from __future__ import annotations

import argparse
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
LIB_DIR = os.path.join(PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libeqt_b200.so")

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-O3",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or add the CUDA toolkit to PATH")


def sources():
    return sorted(glob.glob(os.path.join(HERE, "*.cu")))


def _stale() -> bool:
    if not os.path.exists(LIB_PATH) or not os.path.exists(os.path.join(HERE, "generated", "tp_specs.inc")) \
            or not os.path.exists(os.path.join(HERE, "generated", "sh_specs.inc")):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = sources() + glob.glob(os.path.join(HERE, "*.cuh")) + glob.glob(os.path.join(HERE, "*.inc")) + glob.glob(os.path.join(HERE, "*.py")) \
        + glob.glob(os.path.join(os.path.dirname(PKG), "include", "*.h"))
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Build if sources are newer than the library; returns the library path."""
    if not force and not _stale():
        return LIB_PATH
    from .gen_sh_specs import generate as generate_sh
    from .gen_tp_specs import generate
    generate()
    generate_sh()
    os.makedirs(LIB_DIR, exist_ok=True)
    obj_dir = os.path.join(LIB_DIR, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = _nvcc()
    objs, procs = [], []
    for src in sources():
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", src, "-o", obj] + (["-Xptxas", "-v"] if verbose else [])
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for src, proc in procs:
        log, _ = proc.communicate()
        if verbose or proc.returncode:
            sys.stderr.write(log)
        if proc.returncode:
            raise RuntimeError(f"nvcc failed on {src}")
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB_PATH + ".tmp", *objs,
            "-Xcompiler", "-fPIC"]
    subprocess.check_call(link)
    os.replace(LIB_PATH + ".tmp", LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
