"""Generate the Newton-Schulz fixtures by RUNNING THE REFERENCE'S OWN CUDA KERNELS on a GPU.

    python oracle/build_ref.py /path/to/reference        # where the checkout is (no GPU needed)
    python tests/golden/make_ns_golden.py OUT_DIR         # on a machine with an sm_100 GPU

The reference (i8muon 0.2.0) is imported unmodified from ``oracle/_ref`` (see
``oracle/reference_gpu.py``); its engine entry points ``_regular_i8``,
``_regular_bq``, ``_regular_prec`` and ``_gram_prec`` run on seeded inputs while a
recorder snapshots the tensors of every native call they make.  One ``.npz`` per
case is written to OUT_DIR: the input, the coefficient rows, the result, and for
the staged cases every native call in order with the state of its tensor
arguments after the call (identical contents are stored once).  Copy the files
into ``tests/golden/``; ``tests/test_reference_fixtures.py`` checks the CPU oracle
against them and the GPU tests check this library's kernels against them.

16-bit and 8-bit float tensors are stored as integer bit patterns with the torch
dtype name in the manifest.
"""
from __future__ import annotations

import hashlib
import json
import os
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle import reference_gpu  # noqa: E402

_BITS = {torch.bfloat16: torch.int16, torch.float16: torch.int16, torch.float8_e4m3fn: torch.uint8}


def seeded(shape, dtype, seed, std=0.02, outliers=False):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g) * std
    if outliers:
        x = x * torch.where(torch.rand(shape, generator=g) < 0.01, 50.0, 1.0)
    return x.to(dtype)


class Store:
    def __init__(self):
        self.arrays, self.dtypes = {}, {}

    def put(self, t: torch.Tensor) -> str:
        t = t.detach().contiguous().cpu()
        raw = t.view(_BITS[t.dtype]) if t.dtype in _BITS else t
        a = raw.numpy()
        key = "t" + hashlib.sha1(a.tobytes() + str((a.shape, t.dtype)).encode()).hexdigest()[:16]
        self.arrays[key] = a
        self.dtypes[key] = str(t.dtype)
        return key


def run_case(ref, name, out_dir, *, entry, x, coeffs, precision, fp16_first=False, staged=(), env=None):
    """entry: engine method name; staged: native ops whose tensors are recorded."""
    engine = ref.CutlassNSInt8(fp16_first=fp16_first)
    store, calls = Store(), []

    def sink(source, op, args, kwargs):
        if op not in staged:
            return
        torch.cuda.synchronize()
        rec = []
        for position, a in enumerate(args):
            if isinstance(a, torch.Tensor):
                # of the floating routes' normalize(x, norm, out, out_t, ...) only the norm is kept
                skip = op == "normalize" and position != 1
                rec.append({"t": store.put(a)} if a.numel() and not skip else {"t": None})
            else:
                rec.append(a)
        calls.append({"source": source, "op": op, "args": rec})

    old = {k: os.environ.get(k) for k in (env or {})}
    os.environ.update(env or {})
    try:
        xd = x.cuda()
        with reference_gpu.record(sink):
            y = getattr(engine, entry)(xd, coeffs, 1e-7, True, precision)
        torch.cuda.synchronize()
    finally:
        for k, v in old.items():
            os.environ.pop(k, None) if v is None else os.environ.__setitem__(k, v)
    assert y.shape == x.shape and y.dtype == x.dtype
    manifest = {"name": name, "entry": entry, "precision": precision, "fp16_first": fp16_first,
                "coeffs": [list(map(float, r)) for r in coeffs], "eps": 1e-7, "env": env or {},
                "x": store.put(x), "y": store.put(y), "calls": calls, "dtypes": store.dtypes,
                "reference": "i8muon 0.2.0 csrc/{int8,prec,bq}.cu built for sm_100a, non-TMA tiles",
                "gpu": torch.cuda.get_device_name(0)}
    np.savez_compressed(out_dir / f"reference_ns_{name}.npz", manifest=np.array(json.dumps(manifest)),
                        **store.arrays)
    finite = bool(torch.isfinite(y.float()).all())
    print(f"{name}: {len(calls)} calls, {len(store.arrays)} tensors, finite={finite}", flush=True)


def main(out_dir: str) -> None:
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    ref = reference_gpu.load()
    c5 = ref.recommend_coefficients(5)
    c6 = ref.recommend_coefficients(6)
    pe8 = ref.recommend_coefficients(8, method="polar_express")
    I8 = ("stats", "input_quant", "aat", "symmetric_quant", "square", "update", "output_quant")
    BQ = ("quant", "gemm")
    f32, bf16, f16 = torch.float32, torch.bfloat16, torch.float16

    # global INT8, every stage (int8.cu), wide and tall, all five rows / two rows
    run_case(ref, "i8_staged_wide", out, entry="_regular_i8", x=seeded((2, 144, 272), f32, 11, outliers=True),
             coeffs=c5, precision="int8", staged=I8)
    run_case(ref, "i8_staged_tall", out, entry="_regular_i8", x=seeded((1, 272, 144), bf16, 12, outliers=True),
             coeffs=c5[:2], precision="int8", staged=I8)
    # block-quantised, every stage (bq.cu)
    run_case(ref, "bq_int8_staged", out, entry="_regular_bq", x=seeded((2, 256, 384), bf16, 13, std=1e-3),
             coeffs=c5[:3], precision="int8_bq", staged=BQ)
    run_case(ref, "bq_int8_staged_tall", out, entry="_regular_bq", x=seeded((1, 384, 200), bf16, 14, std=1e-3),
             coeffs=c5[:2], precision="int8_bq", staged=BQ)
    run_case(ref, "bq_fp8_staged", out, entry="_regular_bq", x=seeded((2, 256, 384), bf16, 15, std=1e-3),
             coeffs=c5[:3], precision="float8_e4m3fn", staged=BQ)
    # floating routes: the normalised operands and the result
    for prec, dt in (("float32", f32), ("bfloat16", bf16), ("float16", f16)):
        run_case(ref, f"float_regular_{prec}", out, entry="_regular_prec", x=seeded((2, 144, 272), dt, 16),
                 coeffs=c5, precision=prec, staged=("normalize",))
    run_case(ref, "float_regular_tall_bf16", out, entry="_regular_prec", x=seeded((1, 272, 144), bf16, 17),
             coeffs=c5, precision="bfloat16", staged=("normalize",))
    run_case(ref, "float_first_row_fp16_of_fp32", out, entry="_regular_prec", x=seeded((2, 144, 272), f32, 18),
             coeffs=c5[:1], precision="float16", staged=("normalize",))
    # Gram space: default restart order, an alternating order, Polar Express x8
    run_case(ref, "gram_bf16_00100", out, entry="_gram_prec", x=seeded((2, 128, 1024), bf16, 19),
             coeffs=c5, precision="bfloat16", staged=("normalize",))
    run_case(ref, "gram_fp16_00100", out, entry="_gram_prec", x=seeded((2, 128, 1024), f16, 20),
             coeffs=c5, precision="float16", staged=("normalize",))
    run_case(ref, "gram_fp32_00100", out, entry="_gram_prec", x=seeded((1, 128, 1024), f32, 21),
             coeffs=c5, precision="float32", staged=("normalize",))
    run_case(ref, "gram_fp16_pe8_default", out, entry="_gram_prec", x=seeded((1, 128, 1024), bf16, 22, std=1e-3),
             coeffs=pe8, precision="float16", staged=("normalize",))
    run_case(ref, "gram_fp16_pe8_01010101", out, entry="_gram_prec", x=seeded((1, 128, 1024), bf16, 22, std=1e-3),
             coeffs=pe8, precision="float16", staged=("normalize",), env={"I8MUON_GRAM_RESET": "01010101"})
    run_case(ref, "gram_fp16_0010010", out, entry="_gram_prec", x=seeded((1, 96, 640), f16, 23),
             coeffs=c5 + c5[3:], precision="float16", staged=("normalize",), env={"I8MUON_GRAM_RESET": "0010010"})
    # whole entry points with the FP16 first row (the reference's default engine setting)
    run_case(ref, "i8_fp16first", out, entry="_regular_i8", x=seeded((2, 144, 272), f32, 24, outliers=True),
             coeffs=c6, precision="int8", fp16_first=True, staged=("normalize", "stats", "input_quant"))
    run_case(ref, "bq_int8_fp16first", out, entry="_regular_bq", x=seeded((2, 256, 384), bf16, 25, std=1e-3),
             coeffs=c5, precision="int8_bq", fp16_first=True, staged=("normalize", "quant"))
    run_case(ref, "bq_int8_fp16first_512x1024", out, entry="_regular_bq", x=seeded((1, 512, 1024), bf16, 26, std=1e-3),
             coeffs=c5, precision="int8_bq", fp16_first=True, staged=("normalize", "quant"))
    run_case(ref, "bq_fp8_5rows", out, entry="_regular_bq", x=seeded((2, 256, 384), bf16, 27, std=1e-3),
             coeffs=c5, precision="float8_e4m3fn", staged=("quant",))
    run_case(ref, "bq_int8_5rows", out, entry="_regular_bq", x=seeded((2, 256, 384), bf16, 28, std=1e-3),
             coeffs=c5, precision="int8_bq", staged=("quant",))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "ns_golden_out")
