"""Host-side kernel selection by measurement.

Counterpart of the reference's ``KernelFactory`` (src/i8muon/_cuda_factory.py:15-102):
with ``autotune`` off every query returns the default; with it on, the first query for a key
times each candidate by replaying a CUDA graph of the launch, takes the median of three trials
run in rotated order, and keeps the default unless another candidate is at least 2 % faster
(1 % for a whole pipeline).  Tuning inside a stream capture is refused, as in the reference:
the shape has to be warmed up first.  What is tuned here are the library's kernel variants
(``i8m_variant_count`` / ``i8m_set_variant``), not CUTLASS tile ids.
"""
from __future__ import annotations

import statistics
from typing import Callable, Dict, Hashable, Optional, Sequence

OPERATION_MARGIN = 0.98   # a candidate replaces the default only below this fraction of its time
PIPELINE_MARGIN = 0.99
TRIALS = 3


def _graph_replay_timer(launch: Callable[[object], object], candidate, trial: int) -> float:
    """Milliseconds per launch of ``launch(candidate)``, measured by replaying a captured batch."""
    import torch
    launch(candidate)                      # warm-up outside the capture (allocations, lazy init)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(5):
            launch(candidate)
    for _ in range(4):
        graph.replay()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(20):
        graph.replay()
    end.record()
    end.synchronize()
    return start.elapsed_time(end) / 100.0


def _capturing() -> bool:
    import torch
    return torch.cuda.is_available() and torch.cuda.is_current_stream_capturing()


class KernelFactory:
    """Per-engine tuning cache."""

    def __init__(self, autotune: bool = False, timer: Optional[Callable] = None, capturing: Optional[Callable] = None):
        self.autotune = autotune
        self.cache: Dict[Hashable, object] = {}
        self.timings: Dict[Hashable, Dict[object, float]] = {}
        self._timer = timer or _graph_replay_timer
        self._capturing = capturing or _capturing

    def _measure(self, candidates: Sequence, launch) -> Dict[object, float]:
        samples = {c: [] for c in candidates}
        for trial in range(TRIALS):
            shift = trial % len(candidates)
            for candidate in list(candidates[shift:]) + list(candidates[:shift]):
                samples[candidate].append(self._timer(launch, candidate, trial))
        return {c: statistics.median(v) for c, v in samples.items()}

    def select(self, operation: str, key: Hashable, candidates: Sequence, default, launch, margin=OPERATION_MARGIN):
        """The candidate to use for ``operation`` on ``key``; ``launch(candidate)`` runs it once."""
        if not self.autotune or len(candidates) < 2:
            return default
        full_key = (operation, key, tuple(candidates))
        if full_key in self.cache:
            return self.cache[full_key]
        if self._capturing():
            raise RuntimeError("Warm up this shape and dtype before capturing autotuned CUDA kernels")
        if default not in candidates:
            raise ValueError("the default must be one of the candidates")
        scores = self._measure(candidates, launch)
        best = min(candidates, key=lambda c: scores[c])
        choice = best if scores[best] < scores[default] * margin else default
        self.cache[full_key] = choice
        self.timings[full_key] = scores
        return choice

    def select_pipeline(self, family: str, key: Hashable, launch) -> bool:
        """Whether the tuned choices beat the all-default pipeline as a whole (``launch(tuned)``)."""
        if not self.autotune:
            return False
        return bool(self.select(("pipeline", family), key, (False, True), False, launch, margin=PIPELINE_MARGIN))


__all__ = ["KernelFactory", "OPERATION_MARGIN", "PIPELINE_MARGIN"]
