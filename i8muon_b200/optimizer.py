"""Muon optimizer and the functional ``muon_step``.

Same public surface and update rule as the reference (src/i8muon/_optimizer.py:
``Muon`` 168-408, ``muon_step`` 416-511).  What differs is how the step runs on
the device:

  * parameters with the same (device, dtypes, shape) form a group and go through
    Newton-Schulz as ONE batched call, instead of one call per parameter;
  * the momentum blend (both lerps) is one multi-tensor kernel that writes the
    stacked update tensor directly, and weight decay + the learning-rate-scaled
    update is one multi-tensor kernel; their roundings match the eager torch
    sequence of the reference;
  * with ``use_cuda_graph`` the whole Newton-Schulz call of a group (some thirty launches) is
    captured over a static update buffer and replayed; the two multi-tensor kernels run eagerly
    around it because they take the addresses of gradients and parameters and the learning
    rate as arguments, so the graph survives re-allocated gradients and learning-rate schedules.
"""
from __future__ import annotations

import contextlib
import os
from typing import Optional

import torch
from torch import Tensor
from torch.optim.optimizer import Optimizer, ParamsT

from . import native
from .coefficients import recommend_coefficients
from .engine import CutlassNSInt8, post_status, raise_if_reported
from .routing import (EPS, GRAM_ASPECT_THRESHOLD, adjust_lr, matrix_spec, normalize_precision,
                      validate_ns_device)

__all__ = ["Muon", "muon_step", "native_step_ops"]

# Largest stacked update (bytes) that one Newton-Schulz call may take; larger
# groups are processed in several batched calls to bound the workspace.
MAX_GROUP_BYTES = int(os.environ.get("I8MUON_B200_MAX_GROUP_BYTES", str(2 << 30)))


# ------------------------------------------------------------------ group settings
# One rule per setting: (name, test on the value, message).  The messages are part of the
# drop-in contract (src/i8muon/_optimizer.py:39-67); the table is this library's own.
_ADJUST_NAMES = ("spectral", "original", "match_rms_adamw", "none")
_DECAY_MODES = ("absolute", "base_lr", "adjusted_lr")


def _momentum_tuple(value):
    values = (value,) if isinstance(value, (int, float)) else tuple(value)
    if len(values) not in (1, 2) or any(not 0.0 <= m for m in values):
        raise ValueError("momentum must contain one or two nonnegative values")
    return values


_GROUP_RULES = (
    ("lr", lambda v: not isinstance(v, Tensor) or v.numel() == 1, "Tensor lr must be 1-element"),
    ("weight_decay", lambda v: 0.0 <= v, "weight_decay must be >= 0"),
    ("eps", lambda v: 0.0 <= v, "eps must be >= 0"),
    ("ns_coefficients", lambda v: v is None or (len(v) > 0 and all(len(row) == 3 for row in v)),
     "Expected a nonempty list of (a, b, c) coefficients"),
    ("adjust_lr_fn", lambda v: v is None or callable(v) or v in _ADJUST_NAMES, None),
    ("weight_decay_mode", lambda v: v in _DECAY_MODES,
     "weight_decay_mode must be 'absolute', 'base_lr' or 'adjusted_lr'"),
)


def _check_group(group) -> None:
    """Validate one parameter group's settings and bring momentum / precision to canonical form."""
    for name, accept, message in _GROUP_RULES:
        if not accept(group[name]):
            raise ValueError(message or f"{name} {group[name]} is not supported")
    group["momentum"] = _momentum_tuple(group["momentum"])
    group["precision"] = normalize_precision(group["precision"])


def _graph_key(ns_fn, layout, count, precision, coefficients, eps, deterministic, engine):
    """What one captured Newton-Schulz call depends on.  No tensor address is part of it: the graph
    reads a static update buffer and writes a static result, so it outlives re-allocated gradients
    (``zero_grad(set_to_none=True)``), as the reference's does (src/i8muon/_optimizer.py:133-139, 476-497)."""
    schedule = recommend_coefficients() if coefficients is None else coefficients
    return (id(engine), ns_fn.__name__, layout.device, layout.dtype, tuple(layout.shape), count, precision,
            tuple(tuple(row) for row in schedule), eps, deterministic, engine.fp16_first,
            tuple(sorted(engine.tiles.items())), os.environ.get("I8MUON_GRAM_RESET", "00100"))


# captured graphs kept per optimizer; the least recently used one is dropped beyond this
MAX_CAPTURED_GRAPHS = int(os.environ.get("I8MUON_B200_MAX_GRAPHS", "64"))


class Muon(Optimizer):
    """Muon: momentum updates orthogonalised by Newton-Schulz on B200 tensor cores.

    Matrix parameters (two or more dimensions; leading dimensions are batches)
    use Newton-Schulz; scalar and vector parameters can be handed to
    ``scalar_optimizer``, which is stepped after the Muon groups.  A scalar
    ``momentum`` keeps one moving average; ``(mu, mu2)`` blends Nesterov-style
    with buffer decay ``mu2``.

    ``precision``: auto, int8, int8_bq, fp8, float16, bfloat16 or float32.  Both
    INT8 routes run their first iteration in FP16 when ``fp16_first`` is true.
    ``use_gram`` allows the Gram-space iteration for matrices whose aspect ratio
    reaches ``gram_aspect_threshold``.  ``ns_coefficients`` gives one (a, b, c)
    row per iteration; otherwise ``ns_steps`` (default 5) selects the INT8-safety
    schedule.  ``adjust_lr_fn``: "spectral", "original", "match_rms_adamw",
    "none"/None, or a callable (lr, rows, cols).  ``weight_decay_mode``:
    "base_lr" (default), "adjusted_lr" or "absolute".

    A device-side wait that runs out (it never should) is reported through a status word.
    ``step()`` reads it without stalling: the word is copied to pinned host memory at the end of
    a step and examined at the start of the next one, which then raises ``NativeError``;
    ``check_status()`` synchronises and examines it at once.
    """

    def __init__(
        self,
        params: ParamsT,
        lr: float = 0.01,
        weight_decay: float = 0.0,
        momentum=(0.95, 0.95),
        ns_coefficients=None,
        ns_steps: Optional[int] = None,
        eps: float = EPS,
        adjust_lr_fn="spectral",
        *,
        weight_decay_mode: str = "base_lr",
        precision: str = "auto",
        autotune: bool = False,
        fp16_first: bool = True,
        use_gram: bool = True,
        use_cuda_graph: bool = False,
        gram_aspect_threshold: float = GRAM_ASPECT_THRESHOLD,
        deterministic: bool = True,
        scalar_optimizer: Optional[Optimizer] = None,
    ) -> None:
        precision = normalize_precision(precision)
        if ns_coefficients is None:
            ns_coefficients = recommend_coefficients(iters=5 if ns_steps is None else ns_steps)
        self._ns = CutlassNSInt8(autotune=autotune, fp16_first=fp16_first)
        self._use_cuda_graph = use_cuda_graph
        self._ns_graphs: dict = {}
        self._gram_aspect_threshold = gram_aspect_threshold
        self.scalar_optimizer = None  # attached once the Muon groups exist
        defaults = dict(lr=lr, weight_decay=weight_decay, weight_decay_mode=weight_decay_mode,
                        momentum=momentum, ns_coefficients=ns_coefficients, eps=eps,
                        adjust_lr_fn=adjust_lr_fn, deterministic=deterministic, use_gram=use_gram,
                        precision=precision)
        super().__init__(params, defaults)
        self._refuse_shared_parameters(scalar_optimizer, self._muon_param_groups)
        self.scalar_optimizer = scalar_optimizer

    # ---------------------------------------------------------- validation
    @staticmethod
    def _refuse_shared_parameters(scalar, muon_groups):
        """A parameter belongs to Muon or to the scalar optimizer, never to both."""
        if scalar is None:
            return
        theirs = {id(p) for group in scalar.param_groups for p in group["params"]}
        if any(id(p) in theirs for group in muon_groups for p in group["params"]):
            raise ValueError("Muon and scalar_optimizer must have disjoint parameters")

    def _validate_param_group(self, group):
        _check_group(group)
        for p in group["params"]:
            if p.ndim < 2 or min(p.shape[-2:]) < 1 or not p.is_floating_point():
                raise ValueError("Muon only supports nonempty real floating >=2D parameters")
            if p.is_cuda:
                method, compute = self._ns.router(*p.shape[-2:], group["precision"], group["use_gram"],
                                                  self._gram_aspect_threshold)
                matrix_spec(tuple(p.shape), p.dtype, p.device, compute,
                            128 if method.__name__ == "_regular_bq" else 16)

    @contextlib.contextmanager
    def _muon_groups_only(self):
        """While active, ``param_groups`` and the base class see the Muon groups alone."""
        scalar, self.scalar_optimizer = self.scalar_optimizer, None
        try:
            yield scalar
        finally:
            self.scalar_optimizer = scalar

    def add_param_group(self, param_group):
        members = param_group["params"]
        if isinstance(members, set):
            raise TypeError("Optimizer parameters must have a deterministic order")
        members = [members] if isinstance(members, Tensor) else list(members)
        settings = {**self.defaults, **param_group, "params": members}
        self._validate_param_group(settings)
        self._refuse_shared_parameters(self.scalar_optimizer, [settings])
        with self._muon_groups_only():
            super().add_param_group(settings)

    # -------------------------------------------- param_groups / state dict
    @property
    def param_groups(self):
        """Muon groups followed by the scalar optimizer's, so that learning-rate
        schedulers see both."""
        if self.scalar_optimizer is None:
            return self._muon_param_groups
        return self._muon_param_groups + self.scalar_optimizer.param_groups

    @param_groups.setter
    def param_groups(self, value):
        self._muon_param_groups = value

    def __setstate__(self, state):
        # pickles and checkpoints carry the Muon groups under the base class's name
        renamed = {("_muon_param_groups" if key == "param_groups" else key): value for key, value in state.items()}
        super().__setstate__(renamed)
        for group in self._muon_param_groups:
            if "weight_decay_mode" not in group:
                # written before the setting existed, when the decay used the adjusted rate
                group["weight_decay_mode"] = "adjusted_lr"

    def state_dict(self):
        """Muon state only; the scalar optimizer keeps its own state dict."""
        with self._muon_groups_only():
            return super().state_dict()

    def load_state_dict(self, state_dict):
        with self._muon_groups_only():
            Optimizer.load_state_dict(self, state_dict)
            self._ns_graphs.clear()

    # ---------------------------------------------------------------- step
    def step(self, closure=None):
        with torch.no_grad():
            raise_if_reported()
            loss = None
            if closure is not None:
                with torch.enable_grad():
                    loss = closure()
            for group in self._muon_param_groups:
                params, grads, bufs = [], [], []
                for p in group["params"]:
                    if p.grad is None:
                        continue
                    state = self.state[p]
                    buf = state.get("momentum_buffer")
                    if buf is None:
                        buf = state["momentum_buffer"] = torch.zeros_like(
                            p.grad, memory_format=torch.preserve_format)
                    params.append(p)
                    grads.append(p.grad)
                    bufs.append(buf)
                muon_step(params, grads, bufs, lr=group["lr"], weight_decay=group["weight_decay"],
                          weight_decay_mode=group["weight_decay_mode"], momentum=group["momentum"],
                          ns_coefficients=group["ns_coefficients"], eps=group["eps"],
                          adjust_lr_fn=group["adjust_lr_fn"], deterministic=group["deterministic"],
                          ns_engine=self._ns, precision=group["precision"], use_gram=group["use_gram"],
                          use_cuda_graph=self._use_cuda_graph, ns_graphs=self._ns_graphs,
                          gram_aspect_threshold=self._gram_aspect_threshold)
            if self.scalar_optimizer is not None:
                self.scalar_optimizer.step()
            return loss


def _as_float(value) -> float:
    return float(value.item()) if isinstance(value, Tensor) else float(value)


def _stats_buffer(count, numel, device):
    """FP32 tensor for the statistics partials of ``count`` stacked tensors of ``numel`` elements."""
    return torch.empty(native.stats_scratch_bytes(count, numel) // 4, dtype=torch.float32, device=device)


def _momentum(grads, bufs, update, w_buf, mu, nesterov, stats=None):
    """buf <- lerp(buf, grad, w_buf); update[i] <- lerp(grad, buf, mu) (Nesterov) or buf: one launch per 32
    tensors.  ``stats`` receives the partial sums of squares and maxima of the update, so that the
    Newton-Schulz call that follows needs no pass over it for its norm."""
    native.call("i8m_momentum", native.pointer_array([g.data_ptr() for g in grads]),
                native.pointer_array([b.data_ptr() for b in bufs]), len(grads), update.data_ptr(),
                grads[0].numel(), native.torch_dtype_code(update.dtype), w_buf, mu, int(nesterov),
                stats.data_ptr() if stats is not None else None, torch.cuda.current_stream().cuda_stream)


def muon_step(
    params,
    grads,
    momentum_bufs,
    *,
    lr,
    weight_decay,
    momentum,
    ns_coefficients,
    eps,
    adjust_lr_fn,
    deterministic: bool = True,
    ns_engine: CutlassNSInt8,
    precision: str = "auto",
    use_gram: bool = True,
    use_cuda_graph: bool = False,
    ns_graphs: Optional[dict] = None,
    gram_aspect_threshold: float = GRAM_ASPECT_THRESHOLD,
    weight_decay_mode: str = "base_lr",
) -> None:
    """Apply one Muon update in place to ``params`` and ``momentum_bufs``.

    For every parameter: buf <- lerp(buf, grad, 1 - mu2); update = lerp(grad, buf, mu)
    (Nesterov, two momentum values) or buf; update <- NewtonSchulz(update); decoupled
    weight decay; param <- param - adjusted_lr * update.
    """
    if ns_graphs is None:
        ns_graphs = {}
    if not params:
        return
    raise_if_reported()      # a device-side wait of an earlier step that ran out (no synchronisation)
    lr = _as_float(lr)
    weight_decay = float(weight_decay)
    if weight_decay_mode not in ("absolute", "base_lr", "adjusted_lr"):
        raise ValueError("weight_decay_mode must be 'absolute', 'base_lr' or 'adjusted_lr'")
    momentum = tuple(momentum) if not isinstance(momentum, (int, float)) else (momentum,)
    nesterov = len(momentum) == 2
    mu, mu2 = float(momentum[0]), float(momentum[-1])
    precision = normalize_precision(precision)

    # group parameters that can share one batched Newton-Schulz call
    groups: dict = {}
    for index, param in enumerate(params):
        grad, buf = grads[index], momentum_bufs[index]
        if grad.shape != param.shape or buf.shape != grad.shape or buf.dtype != grad.dtype:
            raise ValueError("parameter, gradient and momentum buffer must agree in shape; "
                             "gradient and buffer in dtype")
        key = (grad.device, grad.dtype, param.dtype, tuple(grad.shape))
        groups.setdefault(key, []).append(index)

    for (device, gdtype, pdtype, shape), members in groups.items():
        M, N = shape[-2], shape[-1]
        ns_fn, actual = ns_engine.router(M, N, precision, use_gram, gram_aspect_threshold)
        validate_ns_device(device, actual)
        native.torch_dtype_code(gdtype)
        adjusted = adjust_lr(lr, adjust_lr_fn, shape)
        ns_kwargs = dict(coeffs=ns_coefficients, eps=eps, deterministic=deterministic, precision=actual)
        # this library's engine takes the statistics partials that the momentum kernel leaves; a foreign
        # engine with the reference's call convention does not
        takes_stats = isinstance(ns_engine, CutlassNSInt8) and deterministic and len(shape) == 2
        per_tensor = 1
        for d in shape:
            per_tensor *= d
        leading = per_tensor // (M * N)
        chunk = max(1, min(len(members), MAX_GROUP_BYTES // max(1, per_tensor * grads[members[0]].element_size()),
                           65535 // max(1, leading)))
        with torch.cuda.device(device):
            for first in range(0, len(members), chunk):
                part = members[first:first + chunk]
                g_list = [grads[i] if grads[i].is_contiguous() else grads[i].contiguous() for i in part]
                b_list, p_list, copy_back = [], [], []
                for i in part:
                    b, p = momentum_bufs[i], params[i]
                    if not b.is_contiguous():
                        c = b.contiguous(); copy_back.append((b, c)); b = c
                    if not p.is_contiguous():
                        c = p.contiguous(); copy_back.append((p, c)); p = c
                    b_list.append(b); p_list.append(p)
                count = len(part)
                update = None
                if use_cuda_graph:
                    key = _graph_key(ns_fn, g_list[0], count, actual, ns_coefficients, eps, deterministic, ns_engine)
                    captured = ns_graphs.pop(key, None)
                    if captured is None:
                        # The graph holds the Newton-Schulz call only, over a static update buffer and a
                        # static result.  The momentum kernel (which takes the gradients' addresses) and the
                        # decay + update kernel (addresses of the parameters, the learning rate) run eagerly,
                        # so neither re-allocated gradients nor a learning-rate schedule invalidates it.
                        update = torch.empty((count, *shape), device=device, dtype=gdtype)
                        update.zero_()
                        stats = _stats_buffer(count, per_tensor, device).zero_() if takes_stats else None
                        extra = dict(stats=stats) if takes_stats else {}
                        for _ in range(2):   # warm up outside capture: first-use work, the tuner, workspaces
                            ns_fn(update, **ns_kwargs, **extra)
                        torch.cuda.current_stream().synchronize()
                        graph = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(graph):
                            ortho = ns_fn(update, **ns_kwargs, **extra)
                        captured = (graph, update, ortho, stats)
                    ns_graphs[key] = captured            # most recently used last
                    while len(ns_graphs) > MAX_CAPTURED_GRAPHS:
                        ns_graphs.pop(next(iter(ns_graphs)))
                    graph, update, ortho, stats = captured
                    _momentum(g_list, b_list, update, 1.0 - mu2, mu, nesterov, stats)
                    graph.replay()
                else:
                    update = torch.empty((count, *shape), device=device, dtype=gdtype)
                    stats = _stats_buffer(count, per_tensor, device) if takes_stats else None
                    _momentum(g_list, b_list, update, 1.0 - mu2, mu, nesterov, stats)
                    ortho = ns_fn(update, **ns_kwargs, **(dict(stats=stats) if takes_stats else {}))

                if callable(adjust_lr_fn):
                    adjusted = adjust_lr(lr, adjust_lr_fn, shape)
                adjusted = _as_float(adjusted)
                if weight_decay == 0:
                    mode, decay = 0, 0.0
                elif weight_decay_mode == "adjusted_lr":
                    mode, decay = 2, weight_decay
                elif weight_decay_mode == "absolute":
                    mode, decay = 1, 1.0 - weight_decay
                else:
                    mode, decay = 1, 1.0 - lr * weight_decay
                native.call("i8m_apply", native.pointer_array([p.data_ptr() for p in p_list]), count,
                            ortho.data_ptr(), per_tensor, native.torch_dtype_code(pdtype),
                            native.torch_dtype_code(gdtype), mode, decay, -adjusted,
                            torch.cuda.current_stream().cuda_stream)
                for original, contiguous in copy_back:
                    original.copy_(contiguous)
    for device in {g.device for g in grads if g.device.type == "cuda"}:
        post_status(device)


def native_step_ops(ns_engine: CutlassNSInt8, *, lr, weight_decay, momentum, ns_coefficients, eps=EPS,
                    adjust_lr_fn="spectral", precision="auto", use_gram=True,
                    gram_aspect_threshold=GRAM_ASPECT_THRESHOLD, weight_decay_mode="base_lr"):
    """The three device operations of one step as callables over stacked same-shape
    matrices, for ``sharding.ShardedMuonStep``: fused momentum kernel, one batched
    Newton-Schulz call, fused decay + update kernel."""
    from .sharding import StepOps
    lr = _as_float(lr)
    momentum = tuple(momentum) if not isinstance(momentum, (int, float)) else (momentum,)
    nesterov = len(momentum) == 2
    mu, mu2 = float(momentum[0]), float(momentum[-1])
    precision = normalize_precision(precision)

    partials = {}     # (device, count, numel) -> statistics partials, reused from step to step

    def do_momentum(grads, bufs, out):
        if grads[0].ndim != 2:        # leading dimensions fold into the batch: the partials are per tensor
            _momentum(grads, bufs, out[:len(grads)], 1.0 - mu2, mu, nesterov)
            return None
        key = (out.device, len(grads), grads[0].numel())
        stats = partials.get(key)
        if stats is None:
            stats = partials[key] = _stats_buffer(len(grads), grads[0].numel(), out.device)
        _momentum(grads, bufs, out[:len(grads)], 1.0 - mu2, mu, nesterov, stats)
        return stats

    def do_ns(x, out=None, stats=None):
        fn, actual = ns_engine.router(x.shape[-2], x.shape[-1], precision, use_gram, gram_aspect_threshold)
        return fn(x, coeffs=ns_coefficients, eps=eps, deterministic=True, precision=actual, out=out, stats=stats)

    def do_apply(params, updates):
        shape = params[0].shape
        adjusted = _as_float(adjust_lr(lr, adjust_lr_fn, shape))
        if weight_decay == 0:
            mode, decay = 0, 0.0
        elif weight_decay_mode == "adjusted_lr":
            mode, decay = 2, weight_decay
        elif weight_decay_mode == "absolute":
            mode, decay = 1, 1.0 - weight_decay
        else:
            mode, decay = 1, 1.0 - lr * weight_decay
        native.call("i8m_apply", native.pointer_array([p.data_ptr() for p in params]), len(params),
                    updates.data_ptr(), params[0].numel(), native.torch_dtype_code(params[0].dtype),
                    native.torch_dtype_code(updates.dtype), mode, decay, -adjusted,
                    torch.cuda.current_stream().cuda_stream)

    return StepOps(momentum=do_momentum, orthogonalise=do_ns, apply=do_apply, begin=raise_if_reported, end=post_status)
