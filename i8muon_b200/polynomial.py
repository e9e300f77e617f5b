"""Opt-in polynomial evaluations of the global-INT8 engine: grouped cubics with a terminal quintic.

The arithmetic is the reference's (src/i8muon/_cutlass_cubic.py:8-87); the stages are sequenced by the
library itself (route ``I8M_ROUTE_INT8_CUBIC`` of ``i8m_ns_run``) out of the call's workspace, so this
module only checks the arguments and packs the rows:

    row 0            (input_gain, 0, 0)
    rows 1 .. n      (gain, diagonal shift, 0) of  T <- -gain (T T^T + shift I) T
    row n + 1        the terminal quintic (a, b, c)
"""
from __future__ import annotations

import math

import torch

from . import native

_INPUT_ERROR = "Expected a nonempty FP32/FP16/BF16 CUDA matrix or matrix batch"


def _finite(values) -> bool:
    return all(math.isfinite(v) for v in values)


def _pack(input_gain, gains, shifts, abc):
    return [(float(input_gain), 0.0, 0.0), *((g, s, 0.0) for g, s in zip(gains, shifts)), tuple(abc)]


def grouped_cubic(engine, x, input_gain, cubic_gains, terminal_abc, eps, *, diagonal_shifts=None):
    """T = input_gain * normalised(X); one cubic per gain (shift -1 unless given); then the quintic."""
    gains = [float(g) for g in cubic_gains]
    abc = [float(v) for v in terminal_abc]
    shifts = [-1.0] * len(gains) if diagonal_shifts is None else [float(v) for v in diagonal_shifts]
    well_formed = bool(gains) and len(abc) == 3 and len(shifts) == len(gains)
    if not (well_formed and _finite([*gains, *abc, *shifts, input_gain, eps]) and input_gain > 0 and eps > 0):
        raise ValueError("Expected finite cubic gains, terminal ABC, positive input_gain and eps")
    if engine.autotune or engine.tiles:
        raise ValueError("Grouped cubic evaluation uses default tiles with autotune=False")
    usable = (isinstance(x, torch.Tensor) and x.ndim >= 2 and x.is_cuda and min(x.shape[-2:]) >= 1
              and x.dtype in (torch.float32, torch.float16, torch.bfloat16))
    if not usable:
        raise ValueError(_INPUT_ERROR)
    batch = math.prod(x.shape[:-2])
    padded = -(-max(x.shape[-2:]) // 16) * 16
    if not 1 <= batch <= 65535 or padded * 127 * 127 > 2 ** 31 - 1:
        raise ValueError("Invalid batch or int32 accumulator overflow")
    return engine._run(native.ROUTE_INT8_CUBIC, x, _pack(input_gain, gains, shifts, abc), eps, native.F16, 16, "int8",
                       False)


def cubic_abc(engine, x, coefficients, eps):
    """Saved cubic rows (a, b, 0) with a > 0 > b, i.e. (a I + b G) X = b (G + (a / b) I) X, then one quintic."""
    rows = [tuple(float(v) for v in row) for row in coefficients]
    cubics, last = rows[:-1], rows[-1:]
    acceptable = (len(rows) >= 2 and all(len(r) == 3 and _finite(r) for r in rows)
                  and all(c == 0.0 and a > 0.0 and b < 0.0 for a, b, c in cubics))
    if not acceptable:
        raise ValueError("Expected finite cubic ABC rows (a>0,b<0,c=0), then one terminal quintic")
    return grouped_cubic(engine, x, 1.0, [-b for _, b, _ in cubics], last[0], eps,
                         diagonal_shifts=[a / b for a, b, _ in cubics])


__all__ = ["grouped_cubic", "cubic_abc"]
