"""Thin torch-tensor wrappers over the stage-level C-ABI calls, for the GPU tests."""
from __future__ import annotations

import torch

from i8muon_b200 import native
from i8muon_b200.engine import status_word

DT = {torch.float32: native.F32, torch.float16: native.F16, torch.bfloat16: native.BF16}


def _stream():
    return torch.cuda.current_stream().cuda_stream


def ptr(t):
    return None if t is None else t.data_ptr()


def status_ok(device) -> int:
    torch.cuda.synchronize()
    word = status_word(device)
    code = int(word.item())
    word.zero_()
    return code


def geometry(rows, cols, align):
    l, h = min(rows, cols), max(rows, cols)
    return l, h, -(-l // align) * align, -(-h // align) * align, int(rows > cols)


def stats(x):
    b = x.shape[0]
    count = x[0].numel()
    nbytes = native.stats_scratch_bytes(b, count)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    norm = torch.empty(b, device=x.device)
    amax = torch.empty(b, device=x.device)
    native.call("i8m_stats", x.data_ptr(), DT[x.dtype], b, count, scratch.data_ptr(), nbytes, norm.data_ptr(),
                amax.data_ptr(), _stream())
    return norm, amax


def normalize(x, norm, compute, eps=1e-7):
    b, rows, cols = x.shape
    l, h, lp, hp, tr = geometry(rows, cols, 16)
    f32 = compute == torch.float32
    a = torch.full((b, lp, hp), float("nan"), device=x.device, dtype=compute)
    at = torch.full((b, hp, lp), float("nan"), device=x.device, dtype=compute)
    alo = torch.full_like(a, float("nan")) if f32 else None
    atlo = torch.full_like(at, float("nan")) if f32 else None
    native.call("i8m_normalize", x.data_ptr(), DT[x.dtype], ptr(norm), a.data_ptr(), at.data_ptr(), ptr(alo),
                ptr(atlo), DT[compute], b, rows, cols, lp, hp, tr, eps, _stream())
    return a, at, alo, atlo


def float_gemm(left, right_t, *, mode=0, sym=False, final=False, transpose=False, out_dtype=None, lm=None,
               ln=None, coeffs=(0.0, 0.0, 0.0), want_t=False, left_lo=None, right_lo=None):
    b, m, k = left.shape
    n = right_t.shape[1]
    lm = m if lm is None else lm
    ln = n if ln is None else ln
    dev = left.device
    f32 = left.dtype == torch.float32
    out_t = out_lo = out_t_lo = None
    if final:
        shape = (b, ln, lm) if transpose else (b, lm, ln)
        out = torch.full(shape, float("nan"), device=dev, dtype=out_dtype)
    else:
        out = torch.full((b, m, n), float("nan"), device=dev, dtype=left.dtype)
        out_lo = torch.full_like(out, float("nan")) if f32 else None
        if want_t:
            out_t = torch.full((b, n, m), float("nan"), device=dev, dtype=left.dtype)
            out_t_lo = torch.full_like(out_t, float("nan")) if f32 else None
    native.call("i8m_float_gemm", left.data_ptr(), ptr(left_lo), right_t.data_ptr(), ptr(right_lo),
                out.data_ptr(), ptr(out_t), ptr(out_lo), ptr(out_t_lo), DT[left.dtype], mode, b, m, n, k, lm,
                ln, int(sym), int(final), int(transpose), DT[out_dtype] if final else 0, *map(float, coeffs),
                status_word(dev).data_ptr(), _stream())
    return out, out_t, out_lo, out_t_lo


def input_quant(x, amax, norm, eps=1e-7):
    b, rows, cols = x.shape
    l, h, lp, hp, tr = geometry(rows, cols, 16)
    a8 = torch.full((b, lp, hp), 99, device=x.device, dtype=torch.int8)
    a8t = torch.full((b, hp, lp), 99, device=x.device, dtype=torch.int8)
    scale = torch.empty(b, device=x.device)
    native.call("i8m_input_quant", x.data_ptr(), DT[x.dtype], amax.data_ptr(), ptr(norm), a8.data_ptr(),
                a8t.data_ptr(), scale.data_ptr(), b, rows, cols, lp, hp, tr, eps, _stream())
    return a8, a8t, scale


def i8_gemm(mode, a, b_t, *, row_b=None, a_scale=None, b_scale=None, diag=None, lm, ln, alpha=0.0, beta=0.0,
            final=False, transpose=False, out_dtype=torch.float32):
    b, m, k = a.shape
    n = b_t.shape[1]
    dev = a.device
    if mode == 0:
        out = torch.zeros((b, m, n), device=dev, dtype=torch.int32)
        mx = torch.zeros(b, device=dev, dtype=torch.int32)
    elif final:
        out = torch.full((b, ln, lm) if transpose else (b, lm, ln), float("nan"), device=dev, dtype=out_dtype)
        mx = None
    else:
        out = torch.zeros((b, m, n), device=dev, dtype=torch.float32)
        mx = torch.zeros(b, device=dev, dtype=torch.float32)
    native.call("i8m_i8_gemm", mode, a.data_ptr(), b_t.data_ptr(), ptr(row_b), out.data_ptr(), ptr(mx),
                ptr(a_scale), ptr(b_scale), ptr(diag), b, m, n, k, lm, ln, float(alpha), float(beta), int(final),
                int(transpose), DT[out_dtype], status_word(dev).data_ptr(), _stream())
    return out, mx


def symmetric_quant(inp, mx, orig_scale, orig_diag, quad, coeffs=(0.0, 0.0, 0.0)):
    b, m, _ = inp.shape
    dev = inp.device
    out = torch.full((b, m, m), 99, device=dev, dtype=torch.int8)
    scale = torch.empty(b, device=dev)
    diag = torch.zeros((b, m), device=dev)
    native.call("i8m_symmetric_quant", inp.data_ptr(), mx.data_ptr(), orig_scale.data_ptr(), ptr(orig_diag),
                out.data_ptr(), scale.data_ptr(), diag.data_ptr(), b, m, int(quad), *map(float, coeffs), _stream())
    return out, scale, diag


def output_quant(y, mx):
    b, m, n = y.shape
    a8 = torch.empty((b, m, n), device=y.device, dtype=torch.int8)
    a8t = torch.empty((b, n, m), device=y.device, dtype=torch.int8)
    scale = torch.empty(b, device=y.device)
    native.call("i8m_output_quant", y.data_ptr(), mx.data_ptr(), a8.data_ptr(), a8t.data_ptr(), scale.data_ptr(),
                b, m, n, _stream())
    return a8, a8t, scale


def bq_quant(x, norm, fp8, eps=1e-7):
    b, rows, cols = x.shape
    l, h, lp, hp, tr = geometry(rows, cols, 128)
    a = torch.full((b, lp, hp), 77, device=x.device, dtype=torch.uint8)
    at = torch.full((b, hp, lp), 77, device=x.device, dtype=torch.uint8)
    scale = torch.empty((b, lp // 128, hp // 128), device=x.device)
    native.call("i8m_bq_quant", x.data_ptr(), DT[x.dtype], ptr(norm), a.data_ptr(), at.data_ptr(),
                scale.data_ptr(), int(fp8), b, rows, cols, lp, hp, tr, eps, _stream())
    return a, at, scale


def bq_gemm(fp8, mode, a, sa, b_t, sb, *, da=None, row_b=None, lm, ln, coeffs=(0.0, 0.0, 0.0), final=False,
            transpose=False, out_dtype=torch.float32):
    b, m, k = a.shape
    n = b_t.shape[1]
    dev = a.device
    out_t = so = dout = None
    if final:
        out = torch.full((b, ln, lm) if transpose else (b, lm, ln), float("nan"), device=dev, dtype=out_dtype)
    else:
        out = torch.full((b, m, n), 77, device=dev, dtype=torch.uint8)
        so = torch.empty((b, m // 128, n // 128), device=dev)
        if mode == 2:
            out_t = torch.full((b, n, m), 77, device=dev, dtype=torch.uint8)
        else:
            dout = torch.empty((b, m), device=dev)
    native.call("i8m_bq_gemm", int(fp8), mode, a.data_ptr(), sa.data_ptr(), ptr(da), b_t.data_ptr(), sb.data_ptr(),
                ptr(row_b), out.data_ptr(), ptr(out_t), ptr(so), ptr(dout), b, m, n, k, lm, ln,
                *map(float, coeffs), int(final), int(transpose), DT[out_dtype], status_word(dev).data_ptr(),
                _stream())
    return out, out_t, so, dout


def decode_q(t, fp8):
    """Quantised bytes -> float values."""
    return t.view(torch.float8_e4m3fn).float() if fp8 else t.view(torch.int8).float()
