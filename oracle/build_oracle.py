"""TEST INFRASTRUCTURE - compile the oracle's C helpers with gcc.

Output goes to ``oracle/_build/libns_exact.so`` (git-ignored).  Building the
checker is not using it: only tests, the smoke check and the benchmark's CPU
baseline load the result.
"""
from __future__ import annotations

import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SOURCE = HERE / "exact_kernels.c"
OUTPUT = HERE / "_build" / "libns_exact.so"


def build(force: bool = False) -> Path:
    if not force and OUTPUT.exists() and OUTPUT.stat().st_mtime >= SOURCE.stat().st_mtime:
        return OUTPUT
    OUTPUT.parent.mkdir(exist_ok=True)
    command = ["gcc", "-O2", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off", "-o", str(OUTPUT),
               str(SOURCE), "-lm"]
    subprocess.run(command, check=True)
    return OUTPUT


if __name__ == "__main__":
    print(build(force=True))
