"""Opt-in polynomial evaluations of the global-INT8 engine: grouped cubics with a terminal quintic.

Counterpart of the reference's ``_cutlass_cubic.py``.  Like there, the drivers live on the host and
sequence the stage-level operators, here the C-ABI entry points of ``include/i8muon_b200.h``:
each cubic is four launches (Gram, shifted symmetric quantisation, update with the gain folded into
the right-hand scale, output quantisation); the terminal row is the regular five-stage quintic.
"""
from __future__ import annotations

import math

import torch

from . import native
from .engine import status_word


def _ptr(t):
    return None if t is None else t.data_ptr()


def grouped_cubic(engine, x, input_gain, cubic_gains, terminal_abc, eps, *, diagonal_shifts=None):
    """T = input_gain * normalised(X); T <- -gain * (T T^T + shift I) T per cubic (shift = -1 by
    default); then the quintic ``terminal_abc`` (src/i8muon/_cutlass_cubic.py:8-71)."""
    gains = tuple(float(g) for g in cubic_gains)
    abc = tuple(float(v) for v in terminal_abc)
    shifts = (-1.0,) * len(gains) if diagonal_shifts is None else tuple(float(v) for v in diagonal_shifts)
    if (not gains or len(abc) != 3 or not all(map(math.isfinite, (*gains, *abc, input_gain, eps)))
            or len(shifts) != len(gains) or not all(map(math.isfinite, shifts))
            or input_gain <= 0 or eps <= 0):
        raise ValueError("Expected finite cubic gains, terminal ABC, positive input_gain and eps")
    if engine.autotune or engine.tiles:
        raise ValueError("Grouped cubic evaluation uses default tiles with autotune=False")
    if (x.ndim < 2 or not x.is_cuda or min(x.shape[-2:]) < 1
            or x.dtype not in (torch.float32, torch.float16, torch.bfloat16)):
        raise ValueError("Expected a nonempty FP32/FP16/BF16 CUDA matrix or matrix batch")
    shape = x.shape
    x = x.contiguous().reshape(-1, *shape[-2:])
    batch, rows, cols = x.shape
    l, h = min(rows, cols), max(rows, cols)
    lp, hp = (l + 15) // 16 * 16, (h + 15) // 16 * 16
    if not 1 <= batch <= 65535 or hp * 127 * 127 > 2 ** 31 - 1:
        raise ValueError("Invalid batch or int32 accumulator overflow")
    dev, dt, transpose = x.device, native.torch_dtype_code(x.dtype), int(rows > cols)
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream().cuda_stream
        status = status_word(dev).data_ptr()
        f32 = dict(dtype=torch.float32, device=dev)
        maxima = torch.zeros((2 * len(gains) + 3, batch), **f32)       # one zeroed slot per reduction
        aq = torch.empty((batch, lp, hp), dtype=torch.int8, device=dev)
        at = torch.empty((batch, hp, lp), dtype=torch.int8, device=dev)
        gq = torch.empty((batch, lp, lp), dtype=torch.int8, device=dev)
        work = torch.empty((batch, lp, hp), **f32)                     # int32 Gram / FP32 polynomial / update
        sa, sg, sp = (torch.empty(batch, **f32) for _ in range(3))
        dg, dp = (torch.empty((batch, lp), **f32) for _ in range(2))
        norm, amax = torch.empty(batch, **f32), torch.empty(batch, **f32)
        out = torch.empty_like(x)
        nbytes = native.stats_scratch_bytes(batch, rows * cols)
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        native.call("i8m_stats", x.data_ptr(), dt, batch, rows * cols, scratch.data_ptr(), nbytes, norm.data_ptr(),
                    amax.data_ptr(), stream)
        # the input gain is folded into the dequantisation scale: normalise by max(norm, eps) / gain
        norm = norm.clamp_min(eps) / input_gain
        native.call("i8m_input_quant", x.data_ptr(), dt, amax.data_ptr(), norm.data_ptr(), aq.data_ptr(),
                    at.data_ptr(), sa.data_ptr(), batch, rows, cols, lp, hp, transpose, 0.0, stream)

        def gemm(mode, a, b_t, row_b, dst, mx, a_scale, b_scale, diag, m, n, k, lm, ln, alpha, beta, final):
            native.call("i8m_i8_gemm", mode, a.data_ptr(), b_t.data_ptr(), _ptr(row_b), dst.data_ptr(), _ptr(mx),
                        _ptr(a_scale), _ptr(b_scale), _ptr(diag), batch, m, n, k, lm, ln, float(alpha), float(beta),
                        int(final), transpose if final else 0, dt, status, stream)

        def symq(src, mx, orig_scale, orig_diag, dst, scale, diag, quad, c0, c1, c2):
            native.call("i8m_symmetric_quant", src.data_ptr(), mx.data_ptr(), orig_scale.data_ptr(), _ptr(orig_diag),
                        dst.data_ptr(), scale.data_ptr(), diag.data_ptr(), batch, lp, int(quad), float(c0),
                        float(c1), float(c2), stream)

        for i, gain in enumerate(gains):
            gm, ym = maxima[2 * i], maxima[2 * i + 1]
            gemm(0, aq, aq, None, work, gm, None, None, None, lp, lp, hp, l, l, 0, 0, False)
            symq(work, gm, sa, None, gq, sg, dg, False, shifts[i], 0, 0)
            gemm(4, gq, at, aq, work, ym, sg, sa, dg, lp, hp, lp, l, h, -gain, 0, False)
            native.call("i8m_output_quant", work.data_ptr(), ym.data_ptr(), aq.data_ptr(), at.data_ptr(),
                        sa.data_ptr(), batch, lp, hp, stream)
        gm, pm = maxima[2 * len(gains)], maxima[2 * len(gains) + 1]
        a, b, c = abc
        gemm(0, aq, aq, None, work, gm, None, None, None, lp, lp, hp, l, l, 0, 0, False)
        symq(work, gm, sa, None, gq, sg, dg, False, 0, 0, 0)
        gemm(1, gq, gq, None, work, pm, sg, None, dg, lp, lp, lp, l, l, b, c, False)
        symq(work, pm, sg, dg, gq, sp, dp, True, a, b, c)
        gemm(2, gq, at, aq, out, None, sp, sa, dp, lp, hp, lp, l, h, 0, 0, True)
    return out.reshape(shape)


def cubic_abc(engine, x, coefficients, eps):
    """(a I + b G) X = b (G + (a / b) I) X per saved cubic row, then the terminal quintic
    (src/i8muon/_cutlass_cubic.py:74-87)."""
    rows = tuple(tuple(float(v) for v in row) for row in coefficients)
    if (len(rows) < 2 or any(len(r) != 3 or not all(map(math.isfinite, r)) for r in rows)
            or any(c != 0.0 or a <= 0.0 or b >= 0.0 for a, b, c in rows[:-1])):
        raise ValueError("Expected finite cubic ABC rows (a>0,b<0,c=0), then one terminal quintic")
    return grouped_cubic(engine, x, 1.0, [-r[1] for r in rows[:-1]], rows[-1], eps,
                         diagonal_shifts=[r[0] / r[1] for r in rows[:-1]])


__all__ = ["grouped_cubic", "cubic_abc"]
