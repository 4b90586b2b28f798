"""The C++ spelling of the crate's host surface (include/ferro_kittens.hpp) and a C++ caller.

On the CPU the caller program only has to compile and link against the library and the oracle;
on a GPU it runs the reference's two `check` sequences end to end through the C++ wrappers.
"""
import subprocess
from pathlib import Path

import pytest

from ferro_kittens_b200.build import LIBRARY, build_library
from oracle.build import LIBRARY as ORACLE, build_oracle

ROOT = Path(__file__).resolve().parent.parent
SOURCE = ROOT / "tests" / "cpp" / "check.cpp"
BINARY = ROOT / "tests" / "cpp" / "check.bin"


def _build() -> Path:
    build_library()
    build_oracle()
    inputs = [SOURCE, ROOT / "include" / "ferro_kittens.hpp", ROOT / "include" / "ferro_kittens.h", LIBRARY, ORACLE]
    if BINARY.exists() and all(BINARY.stat().st_mtime >= path.stat().st_mtime for path in inputs):
        return BINARY
    command = ["nvcc", "-std=c++17", "-O2", "-o", str(BINARY), str(SOURCE), f"-I{ROOT / 'include'}",
               f"-L{LIBRARY.parent}", f"-L{ORACLE.parent}", "-lferro_kittens_b200", "-lfk_oracle", "-lgomp",
               "-Xlinker", f"-rpath={LIBRARY.parent}", "-Xlinker", f"-rpath={ORACLE.parent}"]
    result = subprocess.run(command, capture_output=True, text=True)
    assert result.returncode == 0, result.stdout + result.stderr
    return BINARY


def test_cpp_caller_compiles_and_links():
    assert _build().exists()


@pytest.mark.gpu
def test_cpp_caller_runs_the_reference_checks(device):
    result = subprocess.run([str(_build())], capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stdout + result.stderr
    assert "check ok" in result.stdout
    assert "exact at groups" in result.stdout and "rows attended" in result.stdout
    assert "+ bias, relu: 0 of" in result.stdout
    assert "gradients, worst error" in result.stdout and "rows normalized" in result.stdout
