"""Multi-GPU Muon step: parameter matrices are partitioned across ranks by their
Newton-Schulz cost, each rank orthogonalises its own share, and the updates are
exchanged with one all-gather per shape group.

The reference is single-device (it contains no collective at all); this module
is the one place where the step shards naturally, because every matrix is an
independent unit.  Every rank holds all parameters and all gradients (data-
parallel training), keeps the momentum buffers of the matrices it owns, and
after the all-gather applies weight decay and the scaled update to every
parameter locally, so parameters stay replicated without a broadcast.

Only local memory is read by kernels: the collective (NCCL over NVLink, or gloo
in CPU tests) lands remote updates in this rank's own buffer first.

The arithmetic is injected through ``StepOps`` so that the partition and gather
bookkeeping can be exercised on CPU ranks with stand-in operations.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Sequence, Tuple

import inspect

import torch
import torch.distributed as dist


def ns_flops(shape: Sequence[int], steps: int) -> float:
    """Algorithmic cost of regular Newton-Schulz: steps * (4 l^2 h + 2 l^3) per matrix
    (Gram 2 l^2 h, square 2 l^3, update 2 l^2 h; symmetry savings not deducted)."""
    rows, cols = shape[-2], shape[-1]
    l, h = min(rows, cols), max(rows, cols)
    batch = 1
    for d in shape[:-2]:
        batch *= d
    return float(batch) * steps * (4.0 * l * l * h + 2.0 * l ** 3)


def partition_by_flops(costs: Sequence[float], world: int) -> List[int]:
    """Longest-processing-time greedy: heaviest matrix first onto the least loaded rank.
    Ties break toward the lower rank and the lower index, so every rank computes the
    same assignment."""
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    load = [0.0] * world
    owner = [0] * len(costs)
    for i in order:
        r = min(range(world), key=lambda q: (load[q], q))
        owner[i] = r
        load[r] += costs[i]
    return owner


@dataclass
class ShardGroup:
    """Matrices of one (shape, dtypes) signature."""
    key: Tuple
    members: List[int]                       # indices into the parameter list
    owner: List[int]                         # owning rank per member
    slots: List[List[int]] = field(default_factory=list)   # per rank: members it owns, in order
    width: int = 0                           # max matrices any rank owns in this group


@dataclass
class ShardPlan:
    world: int
    groups: List[ShardGroup]
    load: List[float]

    def owned(self, rank: int) -> List[int]:
        return [i for g in self.groups for i in g.slots[rank]]


def build_plan(shapes: Sequence[Sequence[int]], keys: Sequence[Tuple], world: int, steps: int) -> ShardPlan:
    """Assign every matrix to a rank and lay out the all-gather slots per shape group."""
    costs = [ns_flops(s, steps) for s in shapes]
    owner = partition_by_flops(costs, world)
    load = [0.0] * world
    for i, r in enumerate(owner):
        load[r] += costs[i]
    by_key: Dict[Tuple, List[int]] = {}
    for i, k in enumerate(keys):
        by_key.setdefault(k, []).append(i)
    groups = []
    for k, members in by_key.items():
        g = ShardGroup(key=k, members=members, owner=[owner[i] for i in members])
        g.slots = [[i for i in members if owner[i] == r] for r in range(world)]
        g.width = max(len(s) for s in g.slots)
        groups.append(g)
    # The gather and the update of the last group have nothing to hide behind: take the groups in
    # order of decreasing bytes per rank so that the cheapest one comes last (stable, and the same
    # on every rank).
    def exposed(g: ShardGroup) -> int:
        numel = 1
        for d in shapes[g.members[0]]:
            numel *= int(d)
        return g.width * numel
    groups.sort(key=exposed, reverse=True)
    return ShardPlan(world=world, groups=groups, load=load)


@dataclass
class StepOps:
    """momentum(grads, bufs, out): write stacked updates of len(grads) matrices into out[:len(grads)].
    orthogonalise(x) -> same shape; if it takes ``out=``, the result is written there (the step
    then lets it write straight into the gather buffer and gathers in place).
    apply(params, updates): updates is (len(params), *shape)."""
    momentum: Callable
    orthogonalise: Callable
    apply: Callable


class ShardedMuonStep:
    """One Muon step over replicated parameters with sharded Newton-Schulz.

    ``buffers`` maps parameter index -> momentum buffer and only needs entries for
    the matrices this rank owns (``plan.owned(rank)``).
    """

    def __init__(self, params, steps: int, ops: StepOps, group=None, max_group_bytes: int = 2 << 30):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.ops = ops
        shapes = [tuple(p.shape) for p in params]
        keys = [(p.device.type, p.dtype, tuple(p.shape)) for p in params]
        self.plan = build_plan(shapes, keys, self.world, steps)
        self.max_group_bytes = max_group_bytes
        self._staging: Dict[Tuple, Tuple[torch.Tensor, torch.Tensor]] = {}
        self._copy_stream = None
        self._ns_takes_out = "out" in inspect.signature(ops.orthogonalise).parameters
        self._consumed: Dict[int, object] = {}   # chunk -> event: its gradients were read

    def _buffers_for(self, g: ShardGroup, width: int, like: torch.Tensor, parity: int):
        # two staging sets per signature: chunk n+1 is produced while chunk n is gathered and applied
        key = (g.key, width, parity)
        hit = self._staging.get(key)
        if hit is None:
            send = torch.zeros((width, *like.shape), dtype=like.dtype, device=like.device)
            recv = torch.empty((self.world * width, *like.shape), dtype=like.dtype, device=like.device)
            hit = self._staging[key] = (send, recv)
        return hit

    def _chunks(self, grads):
        """(group, first slot, width, staging parity) in the order the step consumes them."""
        out = []
        for g in self.plan.groups:
            like = grads[g.members[0]]
            per_matrix = like.numel() * like.element_size()
            # bound the stacked batch: process the group's slots in column chunks
            chunk = max(1, min(g.width, self.max_group_bytes // max(1, per_matrix)))
            for first in range(0, g.width, chunk):
                out.append((g, first, min(chunk, g.width - first), len(out) & 1))
        return out

    def _stream_gradients(self, chunks, grads, host_grads):
        """Queue the host-to-device copies of every chunk this rank owns on a copy stream.

        Returns one "ready" event per chunk.  The copy of a chunk waits for the previous step's
        momentum kernel of the same chunk (the only reader of those gradient tensors), so the
        copies of step n+1 run under the Newton-Schulz kernels of step n and of earlier chunks.
        """
        device = grads[chunks[0][0].members[0]].device
        if device.type != "cuda":
            for g, first, width, _ in chunks:
                for i in g.slots[self.rank][first:first + width]:
                    grads[i].copy_(host_grads[i])
            return [None] * len(chunks)
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=device)
        ready = []
        if any(self._consumed.get(c) is None for c, (g, first, width, _) in enumerate(chunks)
               if g.slots[self.rank][first:first + width]):
            # nothing recorded yet says when these gradient tensors were last touched (a fill, an earlier
            # use): order the copies after everything already queued on the compute stream
            self._copy_stream.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(self._copy_stream):
            for c, (g, first, width, _) in enumerate(chunks):
                consumed = self._consumed.get(c)
                if consumed is not None:
                    self._copy_stream.wait_event(consumed)
                for i in g.slots[self.rank][first:first + width]:
                    grads[i].copy_(host_grads[i], non_blocking=True)
                event = torch.cuda.Event()
                event.record(self._copy_stream)
                ready.append(event)
        return ready

    def step(self, params, grads, buffers, host_grads=None) -> None:
        """One step.  With ``host_grads`` (pinned host tensors, indexed like ``grads``) the
        gradients of the matrices this rank owns are first copied into ``grads`` on a separate
        stream, chunk by chunk, overlapped with the kernels of the chunks before them."""
        chunks = self._chunks(grads)
        ready = self._stream_gradients(chunks, grads, host_grads) if host_grads is not None else None
        pending = []
        for c, (g, first, width, parity) in enumerate(chunks):
            like = grads[g.members[0]]
            mine = g.slots[self.rank][first:first + width]
            send, recv = self._buffers_for(g, width, like, parity)
            if mine:
                if ready is not None and ready[c] is not None:
                    torch.cuda.current_stream(like.device).wait_event(ready[c])
                self.ops.momentum([grads[i] for i in mine], [buffers[i] for i in mine], send)
                if like.device.type == "cuda":
                    # recorded on every step, streamed or not: a later streamed step must not overwrite
                    # a gradient that this step's momentum kernel is still reading
                    consumed = torch.cuda.Event()
                    consumed.record(torch.cuda.current_stream(like.device))
                    self._consumed[c] = consumed
                if self._ns_takes_out:
                    own = recv[self.rank * width:self.rank * width + len(mine)]
                    self.ops.orthogonalise(send[:len(mine)], out=own)
                else:
                    send[:len(mine)].copy_(self.ops.orthogonalise(send[:len(mine)]))
            if self.world > 1:
                source = recv[self.rank * width:(self.rank + 1) * width] if self._ns_takes_out else send
                work = dist.all_gather_into_tensor(recv, source, group=self.group, async_op=True)
            elif self._ns_takes_out:
                work = None
            else:
                work, recv = None, send
            pending.append((g, first, width, recv, work))
            # apply the previous chunk while this chunk's collective is in flight
            if len(pending) > 1:
                self._apply(params, *pending.pop(0))
        while pending:
            self._apply(params, *pending.pop(0))

    def _apply(self, params, g: ShardGroup, first: int, width: int, recv, work) -> None:
        if work is not None:
            work.wait()
        for r in range(self.world):
            theirs = g.slots[r][first:first + width]
            if theirs:
                self.ops.apply([params[i] for i in theirs], recv[r * width:r * width + len(theirs)])
