"""Build the compiled parts of the oracle (TEST INFRASTRUCTURE ONLY).

    python oracle/build.py

  oracle/_build/libbess_oracle.so   the C++ / OpenMP restatement of the step (csrc/bess_step.cpp)
  oracle/_ref/libref_distance.so    the reference's own portable L1 / L2 distance code, compiled
                                    from its codelet sources where they lie; built only when a
                                    checkout of the reference is present: the directory named by
                                    the environment variable REFERENCE_ROOT, or a directory
                                    `reference` beside this repository.  The stand-in Poplar headers under
                                    oracle/stubs/ let those two files compile on the host.
"""

from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REFERENCE_ROOT = Path(os.environ.get("REFERENCE_ROOT") or HERE.parent.parent / "reference")
ORACLE_LIB = HERE / "_build" / "libbess_oracle.so"
REF_LIB = HERE / "_ref" / "libref_distance.so"


def _stale(target: Path, sources) -> bool:
    return not target.exists() or any(Path(s).stat().st_mtime > target.stat().st_mtime for s in sources)


def _run(cmd) -> None:
    proc = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("oracle build step failed: " + " ".join(str(c) for c in cmd))


def _compiler() -> str:
    for candidate in ("/usr/bin/g++", os.environ.get("CXX", ""), "g++"):
        if candidate and subprocess.run([candidate, "--version"], capture_output=True).returncode == 0:
            return candidate
    raise RuntimeError("no C++ compiler found")


def build() -> None:
    cxx = _compiler()
    src = HERE / "csrc" / "bess_step.cpp"
    if _stale(ORACLE_LIB, [src, __file__]):
        ORACLE_LIB.parent.mkdir(exist_ok=True)
        base = [cxx, "-O3", "-march=x86-64-v3", "-std=c++17", "-shared", "-fPIC", "-Wall", src, "-o", ORACLE_LIB]
        try:
            _run(base + ["-fopenmp"])
        except RuntimeError:
            _run(base)  # a compiler without OpenMP still gives a (single-threaded) checker
    codelets = REFERENCE_ROOT / "src" / "poplar_extensions"
    if (codelets / "l1distance.codelet.cpp").exists():
        wrappers = [HERE / "csrc" / "ref_l1.cpp", HERE / "csrc" / "ref_l2.cpp"]
        if _stale(REF_LIB, wrappers + [codelets / "l1distance.codelet.cpp", codelets / "l2distance.codelet.cpp"]):
            REF_LIB.parent.mkdir(exist_ok=True)
            _run([cxx, "-O2", "-std=c++17", "-shared", "-fPIC", f"-I{HERE / 'stubs'}", f"-I{codelets}", *wrappers, "-o", REF_LIB])


if __name__ == "__main__":
    build()
    print("built", ORACLE_LIB, REF_LIB if REF_LIB.exists() else "(no reference checkout: _ref skipped)")
