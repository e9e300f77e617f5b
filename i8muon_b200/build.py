"""Build the sm_100a shared library in-tree with nvcc.

The library is a plain C-ABI ``.so`` (no torch headers); it is compiled next to
its sources so that it travels with the source tree.  ``build()`` is idempotent:
it recompiles only when a source file is newer than the library.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
LIBRARY = CSRC / "libi8muon_b200.so"
SOURCES = ("ns_api.cu",)
HEADERS = ("ptx_sm100.cuh", "gemm_core.cuh", "gemm_bq_persistent.cuh", "gemm_wholek_persistent.cuh", "epi_float.cuh", "epi_int8.cuh", "epi_bq.cuh",
           "passes.cuh")
NVCC_FLAGS = (
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    # FP32 expressions are evaluated exactly as written; fused multiply-adds
    # appear only where the code asks for them.
    "--fmad=false", "-Xcompiler", "-fPIC", "-shared",
)


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; the sm_100a library cannot be built")
    return found


def needs_build() -> bool:
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    header = Path(__file__).resolve().parents[1] / "include" / "i8muon_b200.h"
    deps = [CSRC / name for name in SOURCES + HEADERS] + [header]
    return any(dep.stat().st_mtime > built for dep in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile ``csrc/*.cu`` into ``csrc/libi8muon_b200.so`` for sm_100a."""
    if not force and not needs_build():
        return LIBRARY
    command = [_nvcc(), *NVCC_FLAGS, "-o", str(LIBRARY), *[str(CSRC / s) for s in SOURCES]]
    if verbose or os.environ.get("I8MUON_BUILD_VERBOSE", "0") not in ("", "0"):
        command.insert(1, "-Xptxas=-v")
        print(" ".join(command))
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{result.stdout}\n{result.stderr}")
    if verbose:
        print(result.stderr)
    return LIBRARY


if __name__ == "__main__":
    print(build(force=True, verbose=True))
