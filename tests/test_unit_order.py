"""The tile / unit enumerations of the persistent GEMM kernels (which output tile a CTA takes next) checked on
the host: the index functions are ``__host__ __device__``, so a small program built with nvcc walks them for
every tile count up to 120 x 36 (and 120 x 120 lower triangles), every group size the launcher can choose."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
NVCC = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


@pytest.mark.skipif(not Path(NVCC).exists(), reason="nvcc not found")
def test_every_tile_is_enumerated_exactly_once(tmp_path):
    binary = tmp_path / "unit_order_check"
    build = subprocess.run([NVCC, "-std=c++17", "-O1", "-gencode", "arch=compute_100a,code=sm_100a", "-I", str(ROOT / "i8muon_b200" / "csrc"), "-o", str(binary),
                            str(ROOT / "tests" / "native" / "unit_order_check.cu")], capture_output=True, text=True)
    assert build.returncode == 0, build.stderr[-2000:]
    run = subprocess.run([str(binary)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0 and run.stdout.strip() == "ok", run.stdout[-500:]
