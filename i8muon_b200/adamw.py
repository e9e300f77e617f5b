"""Fused AdamW for the parameters that Muon does not take.

The reference's ``Muon(..., scalar_optimizer=...)`` accepts any torch optimizer for embeddings,
heads and vectors (src/i8muon/_optimizer.py:223,254-255) and steps it next to the matrices.
``FusedAdamW`` is a drop-in for that slot: the same hyper-parameters and update rule as
``torch.optim.AdamW`` (decoupled decay, bias correction, no amsgrad / maximize), FP32 moments,
one multi-tensor kernel launch per 24 parameters instead of several element-wise kernels each.
"""
from __future__ import annotations

import ctypes

import torch
from torch.optim import Optimizer

from . import native


class FusedAdamW(Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2):
        if lr < 0 or eps < 0 or weight_decay < 0 or not (0 <= betas[0] < 1 and 0 <= betas[1] < 1):
            raise ValueError("FusedAdamW: invalid hyper-parameter")
        super().__init__(params, dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            buckets = {}
            for p in group["params"]:
                if p.grad is None:
                    continue
                if not p.is_cuda or p.grad.is_sparse:
                    raise ValueError("FusedAdamW needs dense CUDA parameters")
                state = self.state[p]
                if not state:
                    state["step"] = 0
                    state["exp_avg"] = torch.zeros_like(p, dtype=torch.float32, memory_format=torch.contiguous_format)
                    state["exp_avg_sq"] = torch.zeros_like(state["exp_avg"])
                state["step"] += 1
                if not p.is_contiguous() or not p.grad.is_contiguous():
                    raise ValueError("FusedAdamW needs contiguous parameters and gradients")
                buckets.setdefault((p.device, p.dtype, p.grad.dtype, state["step"]), []).append(p)
            for (device, pdtype, gdtype, step), plist in buckets.items():
                pointers = lambda ts: native.pointer_array([t.data_ptr() for t in ts])  # noqa: E731
                counts = (ctypes.c_longlong * len(plist))(*[p.numel() for p in plist])
                with torch.cuda.device(device):
                    native.call("i8m_adamw", pointers(plist), pointers([p.grad for p in plist]),
                                pointers([self.state[p]["exp_avg"] for p in plist]),
                                pointers([self.state[p]["exp_avg_sq"] for p in plist]), counts, len(plist),
                                native.torch_dtype_code(pdtype), native.torch_dtype_code(gdtype),
                                float(group["lr"]), float(beta1), float(beta2), float(group["eps"]),
                                float(group["weight_decay"]), 1.0 - beta1 ** step, 1.0 - beta2 ** step,
                                torch.cuda.current_stream().cuda_stream)
        return loss


__all__ = ["FusedAdamW"]
