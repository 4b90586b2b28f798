"""Builds the C-ABI shared library from the CUDA sources in ``csrc/``.

The library is compiled in-tree for sm_100a only (``-gencode
arch=compute_100a,code=sm_100a``; the arch-specific target is what admits
``tcgen05`` and the tensor-map TMA forms) and links the CUDA runtime
statically, so it loads on a machine with no driver installed and reaches
``cuTensorMapEncodeTiled`` through the runtime's driver entry point query.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
LIBRARY = PACKAGE / "libferro_kittens_b200.so"
CUBLASLT_LIBRARY = PACKAGE / "libfk_cublaslt.so"

SOURCES = ["host.cu", "gemm.cu", "flash.cu", "flash_bwd.cu", "rows.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-cudart", "static",
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")
    return found


def _stale(target: Path, inputs: list[Path]) -> bool:
    if not target.exists():
        return True
    built = target.stat().st_mtime
    return any(path.stat().st_mtime > built for path in inputs)


def build_library(force: bool = False, verbose: bool = False, defines: tuple[str, ...] = (),
                  output: Path | None = None) -> Path:
    """Compile ``csrc/*.cu`` into ``libferro_kittens_b200.so`` if out of date.

    ``defines`` (``NAME=value`` strings) and ``output`` build a tuning variant beside the default.
    """
    target = Path(output) if output else LIBRARY
    sources = [CSRC / name for name in SOURCES if (CSRC / name).exists()]
    inputs = sources + list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + [
        PACKAGE.parent / "include" / "ferro_kittens.h"]
    # The define set a library was built with is recorded beside it, so that a tuning build is never
    # mistaken for the default one: a library whose record differs from what is asked for is stale.
    record = target.with_name(target.name + ".defines")
    wanted = "\n".join(sorted(defines))
    recorded = record.read_text() if record.exists() else None
    if not force and not _stale(target, inputs) and recorded == wanted:
        return target
    command = [_nvcc(), *NVCC_FLAGS, *[f"-D{item}" for item in defines], "-shared", "-o", str(target),
               *map(str, sources)]
    if verbose:
        command.insert(1, "-Xptxas=-v")
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + result.stdout + result.stderr)
    if verbose:
        sys.stderr.write(result.stderr)
    record.write_text(wanted)
    return target


def build_cublaslt(force: bool = False) -> Path:
    """Compile the cuBLASLt denominator used only by the benchmark."""
    source = CSRC / "cublaslt_baseline.cu"
    if not force and not _stale(CUBLASLT_LIBRARY, [source]):
        return CUBLASLT_LIBRARY
    command = [_nvcc(), "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-cudart", "static", "-shared",
               "-o", str(CUBLASLT_LIBRARY), str(source), "-lcublasLt"]
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + result.stdout + result.stderr)
    return CUBLASLT_LIBRARY


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_cublaslt(force="--force" in sys.argv))
