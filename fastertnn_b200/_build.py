"""Builds libtnns_b200.so in-tree: nvcc (sm_100a only) for the CUDA translation units,
gcc for the C host shim, one shared library as the result.

Run as ``python -m fastertnn_b200._build`` or call :func:`build`.  The library is rebuilt
only when a source or header is newer than it.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
INCLUDE = ROOT / "include"
OBJ = PKG / "build"
LIB = PKG / "libtnns_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]
GCC_FLAGS = ["-O2", "-std=c11", "-fPIC", "-Wall", "-Wextra"]


def _find(tool: str, fallback: str) -> str:
    return shutil.which(tool) or fallback


def sources():
    cu = sorted(CSRC.glob("*.cu"))
    c = sorted(CSRC.glob("*.c"))
    return cu, c


def _stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*")) + list(INCLUDE.glob("*.h")) + [Path(__file__)]
    return any(p.stat().st_mtime > t for p in deps)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile every CUDA translation unit for sm_100a and link the shared library."""
    if not force and not _stale():
        return LIB
    nvcc = _find("nvcc", "/usr/local/cuda/bin/nvcc")
    gcc = _find("gcc", "gcc")
    OBJ.mkdir(exist_ok=True)
    cu, c = sources()
    objs = []
    procs = []
    for src in cu:
        obj = OBJ / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, f"-I{INCLUDE}", f"-I{CSRC}", "-c", str(src), "-o", str(obj)]
        if ptxas_info:
            cmd[1:1] = ["-Xptxas", "-v"]
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for src in c:
        obj = OBJ / (src.stem + ".o")
        cmd = [gcc, *GCC_FLAGS, f"-I{INCLUDE}", "-c", str(src), "-o", str(obj)]
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for cmd, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0 or ptxas_info:
            sys.stderr.write(" ".join(cmd) + "\n" + out)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("compilation of libtnns_b200 failed")
    tmp = LIB.with_suffix(".so.tmp")
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(tmp), *map(str, objs)]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(link) + "\n" + r.stdout)
        raise RuntimeError("link of libtnns_b200 failed")
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv)
    print(LIB)
