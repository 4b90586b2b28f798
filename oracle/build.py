"""Builds the CPU oracle (test infrastructure) into ``oracle/libfk_oracle.so``.

The reference itself is Rust on a pinned nightly plus the un-vendored
cuda-oxide git dependency, so none of it compiles with the C/C++ toolchain
here and there is no ``oracle/_ref`` build; this file only compiles the plain-C
restatement in ``fk_oracle.c``.
"""
from __future__ import annotations

import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SOURCE = HERE / "fk_oracle.c"
LIBRARY = HERE / "libfk_oracle.so"


def build_oracle(force: bool = False) -> Path:
    if not force and LIBRARY.exists() and LIBRARY.stat().st_mtime >= SOURCE.stat().st_mtime:
        return LIBRARY
    command = ["gcc", "-O3", "-march=x86-64-v3", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared", "-o", str(LIBRARY),
               str(SOURCE), "-lm"]
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError("gcc failed:\n" + result.stdout + result.stderr)
    return LIBRARY


if __name__ == "__main__":
    print(build_oracle(force=True))
