"""Compile the engine for sm_100a, in tree.

    python distributed-kge-poplar_b200/build.py [--force] [--verbose]

Produces, next to this file:
  libkge_b200.so              the C ABI of include/kge_b200.h (CUDA runtime only)
  libpoplar_kge<ext-suffix>   the pybind11 module with the reference's `Engine` class
A target is rebuilt when any source or header is newer than it.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
INCLUDE = HERE.parent / "include"
NVCC = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]

LIB = HERE / "libkge_b200.so"
MODULE = HERE / ("libpoplar_kge" + sysconfig.get_config_var("EXT_SUFFIX"))


def _newer_than(target: Path, sources) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > stamp for s in sources)


def _run(cmd, verbose: bool) -> None:
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    proc = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if proc.returncode != 0 or verbose:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(str(c) for c in cmd)}")


def build(force: bool = False, verbose: bool = False) -> None:
    headers = list(CSRC.glob("*.hpp")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    lib_sources = sorted(CSRC.glob("*.cu"))
    common = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-Wall,-Wextra", *ARCH]
    if verbose:
        common += ["-Xptxas", "-v"]
    if force or _newer_than(LIB, lib_sources + headers + [Path(__file__)]):
        objects = []
        for src in lib_sources:
            obj = HERE / "build" / (src.stem + ".o")
            obj.parent.mkdir(exist_ok=True)
            if force or _newer_than(obj, [src, *headers, Path(__file__)]):
                _run([NVCC, *common, "-c", src, "-o", obj], verbose)
            objects.append(obj)
        _run([NVCC, "-shared", *ARCH, "-o", LIB, *objects, "-cudart", "shared"], verbose)
    binding = CSRC / "pybind_module.cpp"
    if binding.exists() and (force or _newer_than(MODULE, [binding, LIB, *headers])):
        import pybind11

        _run(
            [
                os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-shared", "-fPIC", "-Wall",
                f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}", f"-I{INCLUDE}",
                binding, "-o", MODULE, f"-L{HERE}", "-lkge_b200", "-Wl,-rpath,$ORIGIN",
            ],
            verbose,
        )


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args()
    build(args.force, args.verbose)
    print("built", LIB.name, MODULE.name if MODULE.exists() else "")
