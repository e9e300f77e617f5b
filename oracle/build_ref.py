"""TEST INFRASTRUCTURE - build the reference's own CUDA modules for sm_100a.

The reference (i8muon 0.2.0) keeps its Newton-Schulz arithmetic in three
pybind11 CUDA modules that it JIT-builds on first use
(``src/i8muon/_cutlass_build.py:26-56``): ``csrc/int8.cu`` -> ``i8muon_cutlass_native``,
``csrc/prec.cu`` -> ``i8muon_cutlass_prec_native``, ``csrc/bq.cu`` ->
``i8muon_cutlass_bq_native``.  Its loader refuses to run without a GPU, so this
recipe compiles the same three files with nvcc directly, with the flags of
``_cutlass_build.py:40-49`` (``-O3 --expt-relaxed-constexpr --fmad=true
-lineinfo``), for ``sm_100a`` only, from the sources where they lie in the
reference checkout, and installs the reference's Python package next to them.

Outputs go only to ``oracle/_ref/`` (git-ignored):

    oracle/_ref/ext/<module>.so     the three compiled modules
    oracle/_ref/site/i8muon/...     ``pip install --no-deps --target`` of the checkout

Nothing of the reference enters the history.  Only the fixture generator in
``tests/golden/``, the tests and the benchmark's reference leg load the result,
as the checker and the same-box baseline; the product never does.
"""
from __future__ import annotations

import shutil
import subprocess
import sys
import sysconfig
import tempfile
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
MODULES = (("int8.cu", "i8muon_cutlass_native"), ("prec.cu", "i8muon_cutlass_prec_native"),
           ("bq.cu", "i8muon_cutlass_bq_native"))


def _compile(reference: Path, source: str, name: str, force: bool) -> Path:
    import torch
    from torch.utils import cpp_extension as ce

    src = reference / "src" / "i8muon" / "csrc" / source
    cutlass = reference / "src" / "i8muon" / "_vendor" / "cutlass" / "include"
    out = OUT / "ext" / f"{name}.so"
    if not force and out.exists() and out.stat().st_mtime >= src.stat().st_mtime:
        return out
    out.parent.mkdir(parents=True, exist_ok=True)
    torch_lib = Path(torch.__file__).resolve().parent / "lib"
    command = ["nvcc", "-std=c++17", "-O3", "--fmad=true", "-lineinfo", *ce.COMMON_NVCC_FLAGS,
               "-gencode", "arch=compute_100a,code=sm_100a",
               f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H",
               f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
               "-Xcompiler", "-fPIC", "-Xcompiler", "-O3", "-shared",
               *[f"-I{p}" for p in ce.include_paths("cuda")], f"-I{sysconfig.get_paths()['include']}",
               f"-I{cutlass}", "-o", str(out), str(src),
               f"-L{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
               "-L/usr/local/cuda/lib64/stubs", "-lcuda"]
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed for {source}:\n{result.stdout[-4000:]}\n{result.stderr[-4000:]}")
    return out


def _install_python(reference: Path, force: bool) -> Path:
    site = OUT / "site"
    if not force and (site / "i8muon" / "__init__.py").exists():
        return site
    with tempfile.TemporaryDirectory() as tmp:
        # the checkout is read-only and setuptools writes into the tree it builds
        copy = Path(tmp) / "i8muon"
        shutil.copytree(reference, copy, ignore=shutil.ignore_patterns("src_old_tilelang", ".git"))
        subprocess.run([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
                        "--quiet", "--upgrade", "--target", str(site), str(copy)], check=True)
    # the compiled modules replace the packaged sources and the vendored CUTLASS headers
    for unused in ("_vendor", "csrc"):
        shutil.rmtree(site / "i8muon" / unused, ignore_errors=True)
    return site


def build(reference: str = "/root/reference", force: bool = False) -> Path:
    ref = Path(reference)
    if not (ref / "src" / "i8muon" / "csrc").is_dir():
        raise FileNotFoundError(f"no reference checkout at {ref}")
    _install_python(ref, force)
    with ThreadPoolExecutor(len(MODULES)) as pool:
        for path in pool.map(lambda m: _compile(ref, m[0], m[1], force), MODULES):
            print("built", path)
    return OUT


if __name__ == "__main__":
    build(*(sys.argv[1:2] or ["/root/reference"]), force="--force" in sys.argv)
