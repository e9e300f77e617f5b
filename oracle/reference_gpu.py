"""TEST INFRASTRUCTURE - load the reference's own CUDA build (``oracle/_ref``) on a GPU box.

``build_ref.py`` leaves the reference's Python package under ``oracle/_ref/site``
and its three CUDA modules, compiled for sm_100a, under ``oracle/_ref/ext``.  This
module imports that package unmodified and replaces only its JIT loader
(``i8muon/_cutlass_build.py:26-56``, which would re-compile for minutes on first
use) by a function that imports the prebuilt modules.  The arithmetic, the
Python drivers (``_cutlass.py``, ``_cutlass_prec.py``, ``_cutlass_bq.py``) and the
optimizer are the reference's own code.

``tma=False`` (default) reports no TMA-capable target, so the reference picks the
``cp.async`` + ``mma.sync`` tiles it runs on its supported GPUs (SM87/89).

Used by the fixture generator ``tests/golden/make_ns_golden.py``, by the GPU
tests that compare this library with the reference on identical inputs, and by
the benchmark's "reference on this GPU" leg.  Never by the product.
"""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

REF = Path(__file__).resolve().parent / "_ref"
_NAMES = {"int8.cu": "i8muon_cutlass_native", "prec.cu": "i8muon_cutlass_prec_native",
          "bq.cu": "i8muon_cutlass_bq_native"}
_modules: dict = {}
_hooks: list = []


def available() -> bool:
    return (REF / "site" / "i8muon" / "__init__.py").exists() and all(
        (REF / "ext" / f"{name}.so").exists() for name in _NAMES.values())


def _import_so(name: str):
    if name not in _modules:
        import torch  # noqa: F401  (the modules link against torch's libraries)
        spec = importlib.util.spec_from_file_location(name, REF / "ext" / f"{name}.so")
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
        _modules[name] = module
    return _modules[name]


class _Proxy:
    """Forwards to a compiled module; lets a recorder see every call and its tensors afterwards."""

    def __init__(self, source, module, tma):
        self._source, self._module = source, module
        self._tma_arches = frozenset({(10, 0)}) if tma else frozenset()

    def __getattr__(self, op):
        fn = getattr(self._module, op)

        def call(*args, **kwargs):
            result = fn(*args, **kwargs)
            for hook in _hooks:
                hook(self._source, op, args, kwargs)
            return result
        return call


def load(tma: bool = False):
    """Return the reference package ``i8muon`` wired to the prebuilt modules, or raise."""
    if not available():
        raise FileNotFoundError("oracle/_ref is not built; run oracle/build_ref.py where the reference checkout is")
    site = str(REF / "site")
    if site not in sys.path:
        sys.path.insert(0, site)
    import i8muon
    from i8muon import _cutlass, _cutlass_bq, _cutlass_build, _cutlass_prec

    proxies: dict = {}

    def load_extension(source="int8.cu", name="i8muon_cutlass"):
        if source not in proxies:
            proxies[source] = _Proxy(source, _import_so(_NAMES[source]), tma)
        return proxies[source]

    for module in (_cutlass_build, _cutlass, _cutlass_prec, _cutlass_bq):
        module.load_extension = load_extension
    for cached in (_cutlass_bq._bq_tma, _cutlass_prec._floating_tiles):
        cached.cache_clear()
    return i8muon


class record:
    """Context manager: collects ``(source, op, args, kwargs)`` after every native call of the reference."""

    def __init__(self, sink):
        self.sink = sink

    def __enter__(self):
        _hooks.append(self.sink)
        return self

    def __exit__(self, *exc):
        _hooks.remove(self.sink)
        return False
