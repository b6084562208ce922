"""Builds libkda_b200.so in-tree with nvcc for sm_100a.  `python -m kda_b200.build` or `build()`."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libkda_b200.so")
DEBUG_LIB = os.path.join(PKG, "libkda_b200_debug.so")      # development checks (csrc/debug/): loaded by tests only
OBJ = os.path.join(PKG, "csrc", "_obj")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-I", os.path.join(ROOT, "include"), "-I", CSRC,
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the kda_b200 kernels cannot be built")
    return exe


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def debug_sources() -> list[str]:
    d = os.path.join(CSRC, "debug")
    return sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith(".cu"))


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False, phase_clocks: bool = False) -> str:
    """Compiles every .cu under csrc/ and links libkda_b200.so next to the package (and the development checks under
    csrc/debug/ into libkda_b200_debug.so, which only tests load).  Returns the product library's path.

    phase_clocks compiles the development-only per-phase clock marks into the kernels (always with force)."""
    nvcc = _nvcc()
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(ROOT, "include", "kda_b200.h"))
    objs, dbg_objs = [], []
    procs = []
    for src in sources() + debug_sources():
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        (dbg_objs if os.path.dirname(src).endswith("debug") else objs).append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + (["-DKDA_PHASE_CLOCKS"] if phase_clocks else [])
            cmd += ["-c", src, "-o", obj]
            if verbose:
                print(" ".join(cmd), flush=True)
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(out)
        elif ptxas_info or verbose:
            sys.stdout.write(out)
    if failed:
        raise RuntimeError("nvcc failed")
    for lib, lib_objs in ((LIB, objs), (DEBUG_LIB, dbg_objs)):
        if force or _stale(lib, lib_objs):
            cmd = [nvcc, "-shared", "-o", lib] + lib_objs + ["-lcudart"]
            if verbose:
                print(" ".join(cmd), flush=True)
            subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    clocks = "--clocks" in sys.argv
    print(build(force="--force" in sys.argv or clocks, verbose=True, ptxas_info="--ptxas" in sys.argv, phase_clocks=clocks))
