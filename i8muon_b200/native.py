"""ctypes binding of the C-ABI library declared in ``include/i8muon_b200.h``.

There is no fallback of any kind: if the shared library is missing or a symbol
cannot be resolved, loading raises.  Every wrapper takes raw device pointers
(``tensor.data_ptr()``) and a raw stream handle, mirrors the C signature one to
one, and raises :class:`NativeError` on a negative return code.
"""
from __future__ import annotations

import ctypes
from ctypes import (POINTER, c_char_p, c_double, c_float, c_int, c_longlong, c_size_t, c_ulonglong,
                    c_void_p)
from functools import lru_cache

from .build import LIBRARY

F32, F16, BF16 = 0, 1, 2
ROUTE_FLOAT, ROUTE_GRAM, ROUTE_INT8, ROUTE_BQ_INT8, ROUTE_BQ_FP8, ROUTE_INT8_FACTORED, ROUTE_INT8_CUBIC = range(7)


class NativeError(RuntimeError):
    """A C-ABI call returned a negative code."""


_P = c_void_p
_SIGNATURES = {
    "i8m_version": (c_int, []),
    "i8m_build_info": (c_char_p, []),
    "i8m_last_error": (c_char_p, []),
    "i8m_launch_count": (c_ulonglong, []),
    "i8m_set_debug_core": (c_int, [c_int]),
    "i8m_variant_count": (c_int, [c_char_p]),
    "i8m_set_variant": (c_int, [c_char_p, c_int]),
    "i8m_set_cta_limit": (c_int, [c_int]),
    "i8m_stats_scratch_bytes": (c_int, [c_int, c_longlong, POINTER(c_size_t)]),
    "i8m_stats": (c_int, [_P, c_int, c_int, c_longlong, _P, c_size_t, _P, _P, _P]),
    "i8m_stats_static": (c_int, [_P, c_int, c_int, c_longlong, _P, _P, _P]),
    "i8m_stats_onepass": (c_int, [_P, c_int, c_int, c_longlong, _P, c_size_t, _P, _P, _P]),
    "i8m_normalize": (c_int, [_P, c_int, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int,
                              c_int, c_int, c_float, _P]),
    "i8m_float_gemm": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int,
                               c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                               c_float, _P, _P]),
    "i8m_float_gemm_to_bq": (c_int, [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                     c_int, c_int, _P, _P]),
    "i8m_input_quant": (c_int, [_P, c_int, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int,
                                c_int, c_float, _P]),
    "i8m_i8_gemm": (c_int, [c_int, _P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int,
                            c_int, c_int, c_float, c_float, c_int, c_int, c_int, _P, _P]),
    "i8m_symmetric_quant": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_float,
                                    c_float, c_float, _P]),
    "i8m_output_quant": (c_int, [_P, _P, _P, _P, _P, c_int, c_int, c_int, _P]),
    "i8m_bq_quant": (c_int, [_P, c_int, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int,
                             c_int, c_float, _P]),
    "i8m_bq_gemm": (c_int, [c_int, c_int, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int,
                            c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_int, c_int,
                            c_int, _P, _P]),
    "i8m_ns_workspace_bytes": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                       POINTER(c_size_t)]),
    "i8m_ns_run": (c_int, [c_int, _P, _P, c_int, c_int, c_int, c_int, c_int, POINTER(c_double),
                           c_int, c_float, c_int, c_int, c_int, c_char_p, _P, _P, c_size_t, _P, _P]),
    "i8m_momentum": (c_int, [POINTER(_P), POINTER(_P), c_int, _P, c_longlong, c_int, c_float,
                             c_float, c_int, _P, _P]),
    "i8m_apply": (c_int, [POINTER(_P), c_int, _P, c_longlong, c_int, c_int, c_int, c_float,
                          c_float, _P]),
    "i8m_adamw": (c_int, [POINTER(_P), POINTER(_P), POINTER(_P), POINTER(_P), POINTER(c_longlong), c_int,
                          c_int, c_int, c_float, c_float, c_float, c_float, c_float, c_float, c_float, _P]),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)


@lru_cache(maxsize=1)
def library() -> ctypes.CDLL:
    """Load ``libi8muon_b200.so``; raise if it has not been built."""
    import os
    path = os.environ.get("I8MUON_B200_LIBRARY", str(LIBRARY))  # explicit path to another build of the same ABI
    if not os.path.exists(path):
        raise NativeError(
            f"{path} is missing: build it with `python -m i8muon_b200.build` "
            "(there is no fallback path)")
    lib = ctypes.CDLL(path)
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


def check(code: int) -> None:
    if code != 0:
        message = library().i8m_last_error().decode(errors="replace")
        raise NativeError(f"i8muon_b200 native call failed ({code}): {message}")


def call(name: str, *args) -> None:
    check(getattr(library(), name)(*args))


def pointer_array(pointers):
    """Host array of device pointers for the multi-tensor optimizer kernels."""
    return (_P * len(pointers))(*pointers)


def torch_dtype_code(dtype) -> int:
    import torch
    try:
        return {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}[dtype]
    except KeyError:
        raise ValueError("Input must be float32, float16 or bfloat16") from None


def ns_workspace_bytes(route, batch, rows, cols, dtype, compute, steps, fp16_first) -> int:
    size = c_size_t(0)
    call("i8m_ns_workspace_bytes", route, batch, rows, cols, dtype, compute, steps,
         int(bool(fp16_first)), ctypes.byref(size))
    return size.value


def stats_scratch_bytes(batch, count) -> int:
    size = c_size_t(0)
    call("i8m_stats_scratch_bytes", batch, count, ctypes.byref(size))
    return size.value


def variant_count(operation: str) -> int:
    """Number of kernel variants the library offers for an operation ("bq_gemm", "wholek_gemm")."""
    return int(library().i8m_variant_count(operation.encode()))


def launch_count() -> int:
    return int(library().i8m_launch_count())


def build_info() -> str:
    return library().i8m_build_info().decode()
