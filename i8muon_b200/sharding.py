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
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import inspect
import os

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
    """momentum(grads, bufs, out): write stacked updates of len(grads) matrices into out[:len(grads)]; it
    may return statistics of what it wrote, which are handed to orthogonalise as ``stats=`` if that takes it.
    orthogonalise(x) -> same shape; if it takes ``out=``, the result is written there (the step
    then lets it write straight into the gather buffer and gathers in place).
    apply(params, updates): updates is (len(params), *shape).
    begin() / end(device), optional: called when a step starts / after its last kernel is queued (the
    native operations use them to surface a device-side wait that ran out: end queues a copy of the status
    word, the next begin raises if it arrived non-zero; neither synchronises)."""
    momentum: Callable
    orthogonalise: Callable
    apply: Callable
    begin: Optional[Callable] = None
    end: Optional[Callable] = None


class ShardedMuonStep:
    """One Muon step over replicated parameters with sharded Newton-Schulz.

    ``buffers`` maps parameter index -> momentum buffer and only needs entries for
    the matrices this rank owns (``plan.owned(rank)``).

    Two ways to bring the other ranks' results home:

    * default: the orthogonalised updates are all-gathered and every rank applies weight decay and
      the update to all parameters (three tensors of traffic over the whole parameter set per rank);
    * ``adopt_parameters=True``: the parameter tensors are re-homed, once, as views into flat
      all-gather buffers laid out ``[rank][slot]`` per shape-group chunk (``param.data`` is
      re-pointed; values are kept).  Each rank then updates only the parameters it owns and the
      in-place all-gather delivers every other rank's *updated parameters* straight into this rank's
      parameter storage: no apply pass over foreign parameters, no staging copy.  Every collective of
      a step is in flight under the kernels of the chunks after it; the step waits for them at its end.

    ``gather`` (adopted parameters on CUDA only) chooses what carries the updated parameters:

    * ``"collective"``: ``all_gather_into_tensor`` in place.  NCCL's kernel needs SMs, and the
      persistent GEMM kernels own every SM they run on, so the caller has to keep some SMs free
      (``i8m_set_cta_limit`` plus ``NCCL_MAX_CTAS``): the GEMMs lose that share of the GPU.
    * ``"copy"``: the flat buffers are allocated as torch symmetric memory (driver virtual-memory
      allocations that every rank of the node maps; multicast is switched off), and after a chunk's
      update a rank *pushes* its own block into each peer's buffer with plain device-to-device
      copies on a side stream: copy engines over NVLink, no SM.  One one-element all-reduce per step,
      queued behind the pushes on that stream, tells every rank that all blocks addressed to it have
      landed.  (Buffers shared through the legacy CUDA IPC handles are no substitute: copies into
      them are staged through host memory, 25 GB/s against 770 GB/s measured.)
    * ``"auto"``: ``"copy"`` when the symmetric-memory rendezvous succeeds, else ``"collective"``;
      ``self.gather`` names what is in use.
    """

    def __init__(self, params, steps: int, ops: StepOps, group=None, max_group_bytes: int = 2 << 30,
                 adopt_parameters: bool = False, gather: str = "collective"):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.ops = ops
        self.steps = steps
        shapes = [tuple(p.shape) for p in params]
        keys = [(p.device.type, p.dtype, tuple(p.shape)) for p in params]
        self.plan = build_plan(shapes, keys, self.world, steps)
        self.max_group_bytes = max_group_bytes
        self.first_chunk_bytes = min(max_group_bytes, 192 << 20)
        self.tail_chunk_bytes = min(max_group_bytes, 128 << 20)
        self._staging: Dict[Tuple, Tuple[torch.Tensor, torch.Tensor]] = {}
        self._copy_stream = None
        self._ns_takes_out = "out" in inspect.signature(ops.orthogonalise).parameters
        self._ns_takes_stats = "stats" in inspect.signature(ops.orthogonalise).parameters
        self._consumed: Dict[int, object] = {}   # chunk -> event: its gradients were read
        self._chunk_list = self._plan_chunks(params)
        self._flat: Dict[int, torch.Tensor] = {}
        self._peer_flat: Dict[int, List[Optional[torch.Tensor]]] = {}
        self._push_stream = None
        self._landed = None
        if gather not in ("collective", "copy", "auto"):
            raise ValueError("gather must be 'collective', 'copy' or 'auto'")
        self.gather = "collective"
        if adopt_parameters and self.world > 1:
            self._adopt(params, gather)

    def _plan_chunks(self, like_tensors):
        """(group, first slot, width, staging parity) in the order the step consumes them."""
        out = []
        groups = self.plan.groups
        for n, g in enumerate(groups):
            like = like_tensors[g.members[0]]
            per_matrix = like.numel() * like.element_size()
            # bound the stacked batch: process the group's slots in column chunks
            budget = self.max_group_bytes
            if self.world > 1 and n >= len(groups) - 2:
                # the transfers of the last chunks have little left to hide behind: finer chunks there, so
                # that a chunk's transfer runs under the kernels of the next chunk of the same group
                budget = min(budget, self.tail_chunk_bytes)
            chunk = max(1, min(g.width, budget // max(1, per_matrix)))
            first = 0
            while first < g.width:
                # the very first chunk of a step has nothing to hide its gradient copy behind (host
                # gradients are streamed one chunk ahead of the kernels): keep it small
                width = min(chunk, g.width - first)
                if not out:
                    width = max(1, min(width, self.first_chunk_bytes // max(1, per_matrix)))
                out.append((g, first, width, len(out) & 1))
                first += width
        return out

    def _adopt(self, params, gather: str = "collective") -> None:
        symm, failure_to_import = None, None
        if gather != "collective" and params[0].device.type == "cuda":
            # plain peer mappings only: no multicast object is ever bound to these buffers
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            try:
                import torch.distributed._symmetric_memory as symm
            except Exception as exc:       # agreed on with the other ranks below
                failure_to_import = exc
                symm = None
        failure = failure_to_import
        for c, (g, first, width, _) in enumerate(self._chunk_list):
            like = params[g.members[0]]
            shape = (self.world * width, *like.shape)
            flat = None
            if symm is not None and failure is None:
                try:
                    flat = symm.empty(shape, dtype=like.dtype, device=like.device).zero_()
                except Exception as exc:       # this rank cannot allocate symmetric memory: ordinary buffers
                    failure = exc
            if flat is None:
                flat = torch.zeros(shape, dtype=like.dtype, device=like.device)
            for r in range(self.world):
                for j, i in enumerate(g.slots[r][first:first + width]):
                    flat[r * width + j].copy_(params[i])
                    params[i].data = flat[r * width + j]
            self._flat[c] = flat
        if gather != "collective" and params[0].device.type == "cuda":
            # the rendezvous is collective: enter it only if every rank holds symmetric buffers
            everyone = [None] * self.world
            dist.all_gather_object(everyone, symm is not None and failure is None, group=self.group)
            if all(everyone):
                self._open_peer_buffers(symm, required=gather == "copy")
            elif gather == "copy":
                raise RuntimeError(f"gather='copy' needs torch symmetric memory on every rank: {failure}")

    def _open_peer_buffers(self, symm, required: bool) -> None:
        """Map every peer's flat buffers here (one rendezvous per buffer, same order on every rank)."""
        group = self.group if self.group is not None else dist.group.WORLD
        peers: Dict[int, List[Optional[torch.Tensor]]] = {c: [None] * self.world for c in self._flat}
        error = None
        try:
            handles = []
            for c, flat in self._flat.items():
                handle = symm.rendezvous(flat, group.group_name)
                handles.append(handle)
                for r in range(self.world):
                    if r != self.rank:
                        peers[c][r] = handle.get_buffer(r, tuple(flat.shape), flat.dtype)
            self._symm_handles = handles
        except Exception as exc:
            error = exc
        # all ranks must agree, or some would wait for pushes that never come
        verdict = [None] * self.world
        dist.all_gather_object(verdict, error is None, group=self.group)
        if all(verdict):
            self._peer_flat = peers
            self.gather = "copy"
            device = next(iter(self._flat.values())).device
            self._push_stream = torch.cuda.Stream(device=device)
            self._landed = torch.zeros(1, dtype=torch.int32, device=device)
        elif required:
            raise RuntimeError(f"gather='copy' needs symmetric memory between the ranks of one node: {error}")

    def _push(self, c: int, width: int, count: int) -> None:
        """Queue the copies of this rank's updated block of chunk c into every peer's flat buffer."""
        device = self._flat[c].device
        self._push_stream.wait_stream(torch.cuda.current_stream(device))
        lo = self.rank * width
        source = self._flat[c][lo:lo + count]
        with torch.cuda.stream(self._push_stream):
            for step in range(1, self.world):
                r = (self.rank + step) % self.world      # every rank starts with a different peer
                self._peer_flat[c][r][lo:lo + count].copy_(source, non_blocking=True)

    def _buffers_for(self, g: ShardGroup, width: int, like: torch.Tensor, parity: int):
        # two staging sets per signature: chunk n+1 is produced while chunk n is gathered and applied
        key = (g.key, width, parity)
        hit = self._staging.get(key)
        if hit is None:
            send = torch.zeros((width, *like.shape), dtype=like.dtype, device=like.device)
            recv = torch.empty((self.world * width, *like.shape), dtype=like.dtype, device=like.device)
            hit = self._staging[key] = (send, recv)
        return hit

    def _pair_for(self, width: int, like: torch.Tensor):
        # adopted parameters: one (update, orthogonalised update) pair per signature serves every chunk,
        # because the collective reads the parameter storage, not these
        key = ("pair", tuple(like.shape), like.dtype, width)
        hit = self._staging.get(key)
        if hit is None:
            hit = self._staging[key] = tuple(
                torch.zeros((width, *like.shape), dtype=like.dtype, device=like.device) for _ in range(2))
        return hit

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

    @staticmethod
    def _mark(phases, chunk, name, device):
        """Phase timing on request: a pair of CUDA events around a phase (see ``phase_milliseconds``)."""
        if phases is None or device.type != "cuda":
            return None
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        phases.append((chunk, name, start, end))
        return end

    def step(self, params, grads, buffers, host_grads=None, phases=None) -> None:
        """One step.  With ``host_grads`` (pinned host tensors, indexed like ``grads``) the
        gradients of the matrices this rank owns are first copied into ``grads`` on a separate
        stream, chunk by chunk, overlapped with the kernels of the chunks before them.
        ``phases``: a list that receives (chunk, phase, start event, end event) for every phase."""
        chunks = self._chunk_list
        if self.ops.begin is not None:
            self.ops.begin()
        ready = self._stream_gradients(chunks, grads, host_grads) if host_grads is not None else None
        pending = []
        for c, (g, first, width, parity) in enumerate(chunks):
            like = grads[g.members[0]]
            mine = g.slots[self.rank][first:first + width]
            flat = self._flat.get(c)
            if flat is not None:
                send, ortho = self._pair_for(width, like)
                recv = flat
            else:
                send, recv = self._buffers_for(g, width, like, parity)
            if mine:
                if ready is not None and ready[c] is not None:
                    torch.cuda.current_stream(like.device).wait_event(ready[c])
                end = self._mark(phases, c, "momentum", like.device)
                stats = self.ops.momentum([grads[i] for i in mine], [buffers[i] for i in mine], send)
                extra = dict(stats=stats) if (self._ns_takes_stats and stats is not None) else {}
                if end is not None:
                    end.record()
                if like.device.type == "cuda":
                    # recorded on every step, streamed or not: a later streamed step must not overwrite
                    # a gradient that this step's momentum kernel is still reading
                    consumed = torch.cuda.Event()
                    consumed.record(torch.cuda.current_stream(like.device))
                    self._consumed[c] = consumed
                end = self._mark(phases, c, "newton_schulz", like.device)
                if flat is not None:
                    if self._ns_takes_out:
                        self.ops.orthogonalise(send[:len(mine)], out=ortho[:len(mine)], **extra)
                        result = ortho[:len(mine)]
                    else:
                        result = self.ops.orthogonalise(send[:len(mine)], **extra)
                elif self._ns_takes_out:
                    own = recv[self.rank * width:self.rank * width + len(mine)]
                    self.ops.orthogonalise(send[:len(mine)], out=own, **extra)
                else:
                    send[:len(mine)].copy_(self.ops.orthogonalise(send[:len(mine)], **extra))
                if end is not None:
                    end.record()
                if flat is not None:
                    # this rank's own parameters are views into `flat`: update them where they live
                    end = self._mark(phases, c, "apply_own", like.device)
                    self.ops.apply([params[i] for i in mine], result)
                    if end is not None:
                        end.record()
            if self.world > 1 and flat is not None and self.gather == "copy":
                if mine:
                    self._push(c, width, len(mine))
                work = None
            elif self.world > 1:
                if flat is not None or self._ns_takes_out:
                    source = recv[self.rank * width:(self.rank + 1) * width]
                else:
                    source = send
                work = dist.all_gather_into_tensor(recv, source, group=self.group, async_op=True)
            elif self._ns_takes_out:
                work = None
            else:
                work, recv = None, send
            pending.append((c, g, first, width, recv, work, flat is not None))
            # apply the previous chunk while this chunk's collective is in flight
            if len(pending) > 1 and not pending[0][6]:
                self._apply(params, phases, *pending.pop(0)[:6])
        if self.gather == "copy" and self._flat:
            # one tiny all-reduce behind this rank's pushes: when it completes here, every rank has
            # issued it, i.e. every rank's pushes (to this rank too) are complete
            device = self._landed.device
            end = self._mark(phases, len(chunks) - 1, "gather_wait", device)
            self._push_stream.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(self._push_stream):
                dist.all_reduce(self._landed, group=self.group)
            torch.cuda.current_stream(device).wait_stream(self._push_stream)
            if end is not None:
                end.record()
        while pending:
            entry = pending.pop(0)
            if entry[6]:
                if entry[5] is not None:
                    end = self._mark(phases, entry[0], "gather_wait", grads[entry[1].members[0]].device)
                    entry[5].wait()          # the parameters of the other ranks have landed in place
                    if end is not None:
                        end.record()
            else:
                self._apply(params, phases, *entry[:6])
        if self.ops.end is not None and chunks:
            self.ops.end(grads[chunks[0][0].members[0]].device)

    def _apply(self, params, phases, c: int, g: ShardGroup, first: int, width: int, recv, work) -> None:
        device = recv.device
        if work is not None:
            end = self._mark(phases, c, "gather_wait", device)
            work.wait()
            if end is not None:
                end.record()
        end = self._mark(phases, c, "apply_all", device)
        for r in range(self.world):
            theirs = g.slots[r][first:first + width]
            if theirs:
                self.ops.apply([params[i] for i in theirs], recv[r * width:r * width + len(theirs)])
        if end is not None:
            end.record()

    @staticmethod
    def phase_milliseconds(phases):
        """Sum of device milliseconds per phase name, and per (chunk, phase); synchronises."""
        torch.cuda.synchronize()
        totals, detail = {}, []
        for chunk, name, start, end in phases:
            ms = start.elapsed_time(end)
            totals[name] = totals.get(name, 0.0) + ms
            detail.append((chunk, name, ms))
        return totals, detail

    # ------------------------------------------------------------------ optimizer state
    def state_dict(self, params, buffers, param_groups=None):
        """An optimizer state dict in the layout of ``torch.optim.Optimizer.state_dict()`` as the
        reference's ``Muon`` writes it (src/i8muon/_optimizer.py:319-336): ``state[index] =
        {"momentum_buffer": tensor}`` for EVERY matrix, gathered from the ranks that own them, plus
        ``param_groups``.  Every rank must call it (it is a collective); every rank receives the full dict,
        on the CPU.  The result loads into a single-device ``Muon`` and into a sharded step of any world size."""
        state = {}
        for c, (g, first, width, _) in enumerate(self._chunk_list):
            like = params[g.members[0]]
            mine = g.slots[self.rank][first:first + width]
            dtype = buffers[mine[0]].dtype if mine else None
            if self.world > 1:
                dtypes = [None] * self.world
                dist.all_gather_object(dtypes, dtype, group=self.group)
                dtype = next((d for d in dtypes if d is not None), like.dtype)
            elif dtype is None:
                dtype = like.dtype
            send = torch.zeros((width, *like.shape), dtype=dtype, device=like.device)
            for j, i in enumerate(mine):
                send[j].copy_(buffers[i])
            if self.world > 1:
                recv = torch.empty((self.world * width, *like.shape), dtype=dtype, device=like.device)
                dist.all_gather_into_tensor(recv, send, group=self.group)
            else:
                recv = send
            for r in range(self.world):
                for j, i in enumerate(g.slots[r][first:first + width]):
                    state[i] = {"momentum_buffer": recv[r * width + j].detach().cpu().clone()}
        groups = param_groups if param_groups is not None else [{"params": list(range(len(params)))}]
        return {"state": dict(sorted(state.items())), "param_groups": groups}

    def load_state_dict(self, state_dict, params, buffers) -> None:
        """Take from a full state dict (``state_dict()`` above at any world size, or a single-device
        ``Muon.state_dict()``) the momentum buffers of the matrices THIS rank owns; the others are
        ignored.  ``buffers`` is filled in place (missing entries are created)."""
        state = state_dict["state"]
        for i in self.plan.owned(self.rank):
            entry = state.get(i, state.get(str(i)))
            if entry is None:
                continue                                  # a parameter that never received a gradient
            saved = entry["momentum_buffer"]
            if i in buffers:
                buffers[i].copy_(saved)
            else:
                buffers[i] = saved.to(params[i].device).clone()
