"""Builds the CPU oracle (TEST INFRASTRUCTURE, not product).

* ``oracle/_build/libzen_oracle.so``  from ``oracle/zen_oracle.c`` (gcc, -ffp-contract=off).
* ``oracle/_ref/libzenith_ref_cpu.so`` from the REFERENCE's own ``core/src/cpu_kernels.cpp``, compiled
  where it lies under the mounted reference tree (environment variable ``ZENITH_REFERENCE``, else a directory
  named ``reference`` beside this repository) with
  ``g++ -O3 -mavx2 -mfma -std=c++20`` plus a C-linkage shim.  Skipped when the tree is absent: a
  prebuilt ``_ref`` library is then used as it is.

    python oracle/build.py
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
BUILD = HERE / "_build"
REF_OUT = HERE / "_ref"
ORACLE_SO = BUILD / "libzen_oracle.so"
REF_SO = REF_OUT / "libzenith_ref_cpu.so"
REFERENCE = Path(os.environ.get("ZENITH_REFERENCE") or HERE.parent.parent / "reference")


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(map(str, cmd)) + "\n" + r.stdout + r.stderr)


def build_oracle(force: bool = False) -> Path:
    src = HERE / "zen_oracle.c"
    hdr = HERE.parent / "zenith_b200" / "csrc" / "det_math.h"
    BUILD.mkdir(exist_ok=True)
    newest = max(src.stat().st_mtime, hdr.stat().st_mtime)
    if force or not ORACLE_SO.exists() or ORACLE_SO.stat().st_mtime < newest:
        _run(["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-shared", "-fPIC", str(src), "-o", str(ORACLE_SO),
              "-lm"])
    return ORACLE_SO


def build_ref(force: bool = False) -> Path | None:
    src = REFERENCE / "core" / "src" / "cpu_kernels.cpp"
    if not src.exists():
        return REF_SO if REF_SO.exists() else None
    REF_OUT.mkdir(exist_ok=True)
    if force or not REF_SO.exists():
        _run(["g++", "-O3", "-mavx2", "-mfma", "-std=c++20", "-shared", "-fPIC", "-I", str(REFERENCE / "core" / "include"),
              str(src), str(HERE / "ref_shim.cpp"), "-o", str(REF_SO)])
    return REF_SO


if __name__ == "__main__":
    print(build_oracle("--force" in sys.argv))
    print(build_ref("--force" in sys.argv))
