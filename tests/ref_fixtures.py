"""Loader for the ``reference_ns_*.npz`` fixtures in ``tests/golden/``.

Each file was written by ``tests/golden/make_ns_golden.py`` while the reference's own CUDA kernels
(built for sm_100a) ran on a B200: the seeded input, the coefficient rows, the result, and for the
staged cases every native call of the reference's driver with its tensors after the call.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"
_FLOAT_BITS = {"torch.bfloat16": torch.bfloat16, "torch.float16": torch.float16,
               "torch.float8_e4m3fn": torch.float8_e4m3fn}


def names():
    return sorted(p.name[len("reference_ns_"):-len(".npz")] for p in GOLDEN.glob("reference_ns_*.npz"))


class Case:
    def __init__(self, name: str, folder: Path = GOLDEN):
        self.data = np.load(folder / f"reference_ns_{name}.npz")
        self.manifest = json.loads(str(self.data["manifest"]))
        self.name = name
        self.coeffs = [tuple(r) for r in self.manifest["coeffs"]]
        self.eps = self.manifest["eps"]
        self.calls = self.manifest["calls"]

    def tensor(self, key):
        """A stored tensor with its original torch dtype (None for an argument that was not kept)."""
        if key is None:
            return None
        t = torch.from_numpy(self.data[key])
        dtype = self.manifest["dtypes"][key]
        return t.view(_FLOAT_BITS[dtype]) if dtype in _FLOAT_BITS else t

    @property
    def x(self):
        return self.tensor(self.manifest["x"])

    @property
    def y(self):
        return self.tensor(self.manifest["y"])

    def args(self, call):
        """Arguments of one recorded native call: tensors as torch tensors, the rest as stored."""
        return [self.tensor(a["t"]) if isinstance(a, dict) else a for a in call["args"]]

    def ops(self, op):
        return [self.args(c) for c in self.calls if c["op"] == op]
