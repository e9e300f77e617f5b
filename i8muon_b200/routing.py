"""Precision names, route selection, matrix geometry and learning-rate scaling.

Host-side logic with the behaviour of the reference's ``_optimizer.py``:
precision aliases (:25-41), ``RoutingMixin.router`` (:70-93), ``_matrix_spec``
(:109-130) and ``_adjust_lr`` (:142-162).  The device check differs on purpose:
this library targets sm_100a only.
"""
from __future__ import annotations

import math
from functools import lru_cache

import torch

GRAM_ASPECT_THRESHOLD = 5.0
EPS = 1e-7

_ALIASES = {
    "auto": ("auto", "default"),
    "int8": ("int8", "i8"),
    "float16": ("float16", "half", "f16", "fp16"),
    "bfloat16": ("bfloat16", "bf16"),
    "float32": ("float32", "float", "fp32"),
    "float8_e4m3fn": ("fp8", "fp8_bq", "float8", "float8_e4m3", "float8_e4m3fn"),
    "int8_bq": ("int8_bq", "int8_block", "i8bq", "i8block"),
}
PRECISIONS = {alias: canonical for canonical, names in _ALIASES.items() for alias in names}


def normalize_precision(precision) -> str:
    if not isinstance(precision, str) or precision.lower() not in PRECISIONS:
        raise ValueError(f"Unsupported precision: {precision}")
    return PRECISIONS[precision.lower()]


def select_route(rows: int, cols: int, precision: str, use_gram: bool, gram_aspect_threshold: float):
    """Return (route name, compute precision) for one matrix shape."""
    if min(rows, cols) <= 0:
        raise ValueError("Matrix dimensions must be positive")
    precision = normalize_precision(precision)
    aspect = max(rows, cols) / min(rows, cols)
    if use_gram and aspect >= gram_aspect_threshold:
        quantised = precision in ("auto", "int8", "int8_bq", "float8_e4m3fn")
        return "_gram_prec", ("float16" if quantised else precision)
    if precision == "auto":
        if rows * cols < 1024 * 1024:
            return "_regular_prec", "float16"
        return "_regular_i8", "int8"
    if precision == "int8_bq":
        return "_regular_bq", "int8"
    if precision == "float8_e4m3fn":
        return "_regular_bq", precision
    if precision == "int8":
        return "_regular_i8", precision
    return "_regular_prec", precision


@lru_cache(maxsize=None)
def validate_ns_device(device: torch.device, compute_precision: str) -> None:
    """The kernels are sm_100a binaries: require a CUDA device of compute capability 10.x."""
    if device.type != "cuda" or not torch.cuda.is_available():
        raise ValueError("Muon requires CUDA parameters; move matrix parameters to a CUDA device.")
    major, _minor = torch.cuda.get_device_capability(device)
    if major != 10:
        raise ValueError("The i8muon_b200 kernels are built for sm_100a (B200) only.")


@lru_cache(maxsize=None)
def matrix_spec(shape, dtype, device, precision, alignment=16):
    """Fold leading dimensions into a batch and pad the matrix geometry.

    Returns (batch, rows, cols, l, h, lp, hp) with l/h the smaller/larger
    dimension and lp/hp their padded sizes (16, or 128 for block quantisation).
    """
    shape = tuple(shape)
    if len(shape) < 2 or device.type != "cuda":
        raise ValueError("Expected a CUDA tensor with at least two dimensions")
    if dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError("Input must be float32, float16 or bfloat16")
    if min(shape[-2:]) < 1:
        raise ValueError("Matrix dimensions must be positive")
    batch = math.prod(shape[:-2])
    if not 1 <= batch <= 65535:
        raise ValueError("Batch size must be between 1 and 65535")
    validate_ns_device(device, precision)
    rows, cols = shape[-2:]
    l, h = min(rows, cols), max(rows, cols)
    lp = -(-l // alignment) * alignment
    hp = -(-h // alignment) * alignment
    if alignment == 16 and precision == "int8" and hp * 127 * 127 > 2 ** 31 - 1:
        raise ValueError("Inner dimension can overflow the int32 accumulator")
    if hp > 2 ** 31 - 1:
        raise ValueError("Padded matrix dimensions exceed the CUDA integer range")
    return batch, rows, cols, l, h, lp, hp


def adjust_lr(lr, adjust_lr_fn, param_shape):
    """Scale the learning rate by the matrix shape.

    A callable receives (lr, rows, cols) and returns the adjusted value.  Built-in
    names: "spectral" sqrt(rows/cols), "original" sqrt(max(1, rows/cols)),
    "match_rms_adamw" 0.2 sqrt(max(rows, cols)); "none" or None leave lr unchanged.
    """
    rows, cols = param_shape[-2], param_shape[-1]
    if callable(adjust_lr_fn):
        return adjust_lr_fn(lr, rows, cols)
    if adjust_lr_fn == "spectral":
        ratio = math.sqrt(rows / cols)
    elif adjust_lr_fn == "original":
        ratio = math.sqrt(max(1, rows / cols))
    elif adjust_lr_fn == "match_rms_adamw":
        ratio = 0.2 * math.sqrt(max(rows, cols))
    else:
        ratio = 1.0
    return lr * ratio
