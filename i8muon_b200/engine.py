"""Newton-Schulz engine: the object the optimizer routes every matrix through.

Drop-in for the reference's ``CutlassNSInt8`` (src/i8muon/_cutlass.py:15-49):
same constructor arguments, the same four entry points ``_regular_prec``,
``_gram_prec``, ``_regular_i8`` and ``_regular_bq`` with the call convention
``fn(x, coeffs=None, eps=1e-7, deterministic=True, precision=...) -> Tensor``
(same shape and dtype as ``x``; leading dimensions fold into the batch), and the
same ``router``.  Each entry point is one call into the sm_100a library
(``i8m_ns_run``), which sequences the fused kernels on the current stream.

Differences that a caller can observe:
  * only compute capability 10.x devices are accepted;
  * ``deterministic=False`` selects one-pass statistics with atomics on every route (the reference
    only has that flavour for global INT8); the default is the two-pass reduction in a fixed order;
  * the result is a fresh tensor, not a view into the call's workspace;
  * ``tiles`` selects, per product of the global-INT8 route (``aat``, ``square``, ``update``), between this
    library's kernels for whole-K products: the reference's tile id 4 (its TMA tile) maps to the
    persistent kernel with 128 x 256 units (also the default), ids 0-3 (its cp.async tiles) to the
    one-CTA-per-tile kernel;
    ``autotune`` times the library's kernel variants (``tuning.py``).
"""
from __future__ import annotations

import ctypes
import math
import os
from functools import lru_cache

import torch

from . import native
from .coefficients import DEFAULT_COEFFICIENTS
from .routing import matrix_spec, normalize_precision, select_route
from .tuning import KernelFactory

_COMPUTE_CODES = {"float32": native.F32, "float16": native.F16, "bfloat16": native.BF16}
_STATUS_WORDS = {}


def status_word(device: torch.device) -> torch.Tensor:
    """One zeroed int32 per device that kernels write an error code to when a
    bounded device-side wait gives up."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    word = _STATUS_WORDS.get(index)
    if word is None:
        word = _STATUS_WORDS[index] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", index))
    return word


def check_status(device=None) -> None:
    """Synchronise and raise if any kernel on ``device`` reported a timed-out wait."""
    devices = list(_STATUS_WORDS) if device is None else [torch.device(device).index or 0]
    for index in devices:
        word = _STATUS_WORDS.get(index)
        if word is None:
            continue
        code = int(word.item())
        if code:
            word.zero_()
            raise native.NativeError(f"device-side wait timed out, status word 0x{code:x}")


_STATUS_HOST = {}


def post_status(device) -> None:
    """Queue a copy of the device's status word to pinned host memory on the current stream; nothing
    waits for it.  ``raise_if_reported`` looks at the copy once it has landed."""
    index = torch.device(device).index
    index = torch.cuda.current_device() if index is None else index
    word = _STATUS_WORDS.get(index)
    if word is None or torch.cuda.is_current_stream_capturing():
        return
    slot = _STATUS_HOST.get(index)
    if slot is None:
        slot = _STATUS_HOST[index] = (torch.zeros(1, dtype=torch.int32).pin_memory(), torch.cuda.Event())
    host, event = slot
    with torch.cuda.device(index):
        host.copy_(word, non_blocking=True)
        event.record()


def raise_if_reported() -> None:
    """Raise if a status word copied by ``post_status`` has arrived and is not zero (no synchronisation)."""
    for index, (host, event) in _STATUS_HOST.items():
        if event.query() and int(host[0]) != 0:
            code = int(host[0])
            host.zero_()
            _STATUS_WORDS[index].zero_()
            raise native.NativeError(f"device-side wait timed out on cuda:{index}, status word 0x{code:x}; the "
                                     "results of the previous step are incomplete")


def _coefficient_array(coeffs):
    rows = [tuple(float(v) for v in row) for row in coeffs]
    if not rows or any(len(row) != 3 for row in rows):
        raise ValueError("Expected a nonempty list of (a, b, c) coefficients")
    flat = [v for row in rows for v in row]
    return (ctypes.c_double * len(flat))(*flat), len(rows)


class CutlassNSInt8:
    """Native floating-point regular/Gram NS and regular INT8 / INT8-BQ / FP8-BQ NS."""

    def __init__(self, autotune=False, *, tiles=None, fp16_first=True):
        self.fp16_first = fp16_first
        self.autotune = autotune
        self.tiles = dict(tiles or {})
        # kernel selection of calls that neither ``tiles`` nor the tuner decides, in i8m_ns_run's packing
        # (block-quantised GEMM | whole-K GEMM << 8 | its square << 16 | its update << 24); 0: the defaults
        # (environment I8MUON_B200_KERNEL_VARIANTS presets it: an integer, e.g. 0x02020200)
        self.kernel_variants = int(os.environ.get("I8MUON_B200_KERNEL_VARIANTS", "0"), 0)
        if (set(self.tiles) - {"aat", "square", "update"}
                or any(v not in (0, 1, 2, 3, 4) for v in self.tiles.values())):
            raise ValueError("tiles accepts aat/square/update with values 0/1/2/3/4")
        self._routes = {}
        self._factory = KernelFactory(autotune)

    # ------------------------------------------------------------ routing
    def router(self, M: int, N: int, precision: str, use_gram: bool, gram_aspect_threshold: float):
        key = (M, N, precision, use_gram, gram_aspect_threshold)
        hit = self._routes.get(key)
        if hit is None:
            name, compute = select_route(M, N, precision, use_gram, gram_aspect_threshold)
            hit = self._routes[key] = (getattr(self, name), compute)
        return hit

    # ------------------------------------------------------------- launch
    def _run(self, route, x, coeffs, eps, compute, alignment, spec_precision, fp16_first, out=None,
             deterministic=True, stats=None):
        coeffs = DEFAULT_COEFFICIENTS if coeffs is None else coeffs
        shape = x.shape
        batch, rows, cols, *_ = matrix_spec(tuple(shape), x.dtype, x.device, spec_precision, alignment)
        x = x.contiguous()
        dtype = native.torch_dtype_code(x.dtype)
        array, steps = _coefficient_array(coeffs)
        order = os.environ.get("I8MUON_GRAM_RESET", "00100") if route == native.ROUTE_GRAM else None
        if order is not None and (not order or order[0] != "0" or set(order) - {"0", "1"}):
            raise ValueError("I8MUON_GRAM_RESET must be a binary string starting with 0")
        with torch.cuda.device(x.device):
            size = native.ns_workspace_bytes(route, batch, rows, cols, dtype, compute, steps, fp16_first)
            if out is None:
                out = torch.empty_like(x)
            elif (out.shape != x.shape or out.dtype != x.dtype or out.device != x.device
                  or not out.is_contiguous() or out.data_ptr() == x.data_ptr()):
                raise ValueError("out must be a contiguous tensor like x that does not alias it")
            if stats is not None and (stats.dtype != torch.float32 or stats.device != x.device or not stats.is_contiguous()
                                      or stats.numel() * 4 < native.stats_scratch_bytes(batch, rows * cols)):
                raise ValueError("stats must be the FP32 partials that i8m_momentum left for x")

            def launch(variant):
                workspace = torch.empty(size, dtype=torch.uint8, device=x.device)
                native.call("i8m_ns_run", route, x.data_ptr(), out.data_ptr(), dtype, batch, rows, cols,
                            compute, array, steps, float(eps), int(bool(fp16_first)), int(bool(deterministic)),
                            int(variant),
                            order.encode() if order is not None else None,
                            stats.data_ptr() if stats is not None else None, workspace.data_ptr(), size,
                            status_word(x.device).data_ptr(), torch.cuda.current_stream().cuda_stream)

            variant = self.kernel_variants
            key = (x.device.index, x.dtype, batch, rows, cols, route, compute, steps, bool(fp16_first))
            if route in (native.ROUTE_INT8, native.ROUTE_INT8_FACTORED) and self.tiles:
                # explicit tiles take precedence over measurements, as in the reference
                per_op = [0 if self.tiles.get(op, 4) == 4 else 2 for op in ("aat", "square", "update")]
                variant = (per_op[0] << 8) | (per_op[1] << 16) | (per_op[2] << 24)
            elif self._factory.autotune:
                # per operation first (median of three graph replays, >= 2 % to replace the default), then the
                # tuned call as a whole against the all-default call (>= 1 %), as the reference's factory does
                tuned = 0
                if route in (native.ROUTE_BQ_INT8, native.ROUTE_BQ_FP8):
                    tuned = self._factory.select("bq_gemm", key, tuple(range(native.variant_count("bq_gemm"))), 0, launch)
                if route != native.ROUTE_BQ_FP8 and not (route == native.ROUTE_FLOAT and compute == native.F32):
                    # routes with whole-K products (the FP16 first row included): bits 8.. select their kernel
                    choice = self._factory.select("wholek_gemm", key, tuple(range(native.variant_count("wholek_gemm"))), 0,
                                                  lambda v: launch(tuned | (v << 8) | (v << 16) | (v << 24)))
                    tuned |= (choice << 8) | (choice << 16) | (choice << 24)
                if tuned and self._factory.select_pipeline("ns_call", key, lambda use: launch(tuned if use else 0)):
                    variant = tuned
            launch(variant)
        # The workspace may be reused by later allocations on this stream only.
        return out.view(shape)

    # Every entry point takes the reference's arguments plus two keyword-only extras: ``out``, a caller-owned
    # tensor for the result (the sharded step lets NS write straight into its gather buffer), and ``stats``,
    # the statistics partials that the momentum kernel left for ``x`` (then no pass over ``x`` is needed
    # for its norm).
    def _regular_prec(self, x, coeffs=None, eps=1e-7, deterministic=True, precision="float16", *, out=None, stats=None):
        """FP32 / BF16 / FP16 regular NS (src/i8muon/_cutlass_prec.py:90-106)."""
        precision = normalize_precision(precision)
        if precision not in _COMPUTE_CODES:
            raise ValueError(f"Unsupported floating-point precision: {precision}")
        return self._run(native.ROUTE_FLOAT, x, coeffs, eps, _COMPUTE_CODES[precision], 16, precision, False, out,
                         deterministic, stats)

    def _gram_prec(self, x, coeffs=None, eps=1e-7, deterministic=True, precision="float16", *, out=None, stats=None):
        """Gram-space NS with restarts given by I8MUON_GRAM_RESET (src/i8muon/_cutlass_prec.py:107-130)."""
        precision = normalize_precision(precision)
        if precision not in _COMPUTE_CODES:
            raise ValueError(f"Unsupported floating-point precision: {precision}")
        return self._run(native.ROUTE_GRAM, x, coeffs, eps, _COMPUTE_CODES[precision], 16, precision, False, out,
                         deterministic, stats)

    def _regular_i8(self, x, coeffs=None, eps=1e-7, deterministic=True, precision="int8", *, block=False, out=None,
                    stats=None):
        """Global-scale INT8 NS, optionally after one FP16 iteration (src/i8muon/_cutlass.py:130-142)."""
        if block:
            return self._run(native.ROUTE_BQ_INT8, x, coeffs, eps, native.F16, 128, "int8", self.fp16_first, out,
                             deterministic, stats)
        return self._run(native.ROUTE_INT8, x, coeffs, eps, native.F16, 16, "int8", self.fp16_first, out, deterministic,
                         stats)

    # ------------------------------------------------ opt-in polynomial entry points
    def _regular_i8_factored(self, X, factor_rows, eps=1e-7, deterministic=True, *, out=None):
        """Completed-square rows ``(c, p, q)``: X <- c * ((G + p I)^2 + q I) X per row, all in the
        global-INT8 stages (the first row in FP16 when ``fp16_first``); src/i8muon/_cutlass.py:93-128."""
        factors = tuple(tuple(float(v) for v in row) for row in factor_rows)
        if not factors or any(len(row) != 3 or not all(map(math.isfinite, row)) for row in factors):
            raise ValueError("Expected nonempty finite (c,p,q) factor rows")
        return self._run(native.ROUTE_INT8_FACTORED, X, factors, eps, native.F16, 16, "int8", self.fp16_first, out,
                         deterministic)

    def _regular_i8_grouped_cubic(self, X, input_gain, cubic_gains, terminal_abc, eps=1e-7):
        """All-INT8 grouped cubics T <- -gain * (T T^T - I) T followed by one quintic; ignores
        ``fp16_first`` (src/i8muon/_cutlass.py:78-84, _cutlass_cubic.py:8-71)."""
        from .polynomial import grouped_cubic
        return grouped_cubic(self, X, input_gain, cubic_gains, terminal_abc, eps)

    def _regular_i8_cubic_abc(self, X, coeffs, eps=1e-7, deterministic=True, precision="int8"):
        """Saved cubic rows ``(a, b, 0)`` with a > 0 > b, then one terminal quintic row; all INT8
        (src/i8muon/_cutlass.py:86-91, _cutlass_cubic.py:74-87)."""
        if precision != "int8":
            raise ValueError("Cubic ABC evaluation requires INT8")
        from .polynomial import cubic_abc
        return cubic_abc(self, X, coeffs, eps)

    def _regular_bq(self, x, coeffs=None, eps=1e-7, deterministic=True, precision="float8_e4m3fn", *, out=None,
                    stats=None):
        """128x128 block-quantised NS: INT8 honours fp16_first, E4M3 never does
        (src/i8muon/_cutlass.py:71-76)."""
        precision = normalize_precision(precision)
        if precision in ("int8_bq", "int8"):
            return self._regular_i8(x, coeffs, eps, deterministic, "int8", block=True, out=out, stats=stats)
        if precision != "float8_e4m3fn":
            raise ValueError(f"Unsupported block-quantised precision: {precision}")
        return self._run(native.ROUTE_BQ_FP8, x, coeffs, eps, native.F16, 128, precision, False, out, deterministic,
                         stats)


__all__ = ["CutlassNSInt8", "check_status", "status_word", "post_status", "raise_if_reported"]
