"""Multi-rank step bookkeeping on CPU ranks (gloo, world size 2 and 3): the flop
partition, the all-gather slot layout, and equality with the unsharded step."""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from i8muon_b200.sharding import ShardedMuonStep, StepOps, build_plan, ns_flops, partition_by_flops
from oracle import ns_oracle as o

LLAMA_LAYER = [(4096, 4096), (1024, 4096), (1024, 4096), (4096, 4096), (14336, 4096), (14336, 4096), (4096, 14336)]


def test_flop_count_matches_stated_totals():
    total = sum(ns_flops(s, 5) for s in LLAMA_LAYER) * 32
    assert abs(total / 6.659e14 - 1) < 1e-3          # Llama-3-8B-shaped set, 5 steps
    assert abs(ns_flops((1024, 4096), 5) / 9.664e10 - 1) < 1e-3
    assert ns_flops((3, 64, 32), 2) == 3 * 2 * (4 * 32 * 32 * 64 + 2 * 32 ** 3)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_partition_of_llama_set_is_balanced(world):
    shapes = LLAMA_LAYER * 32
    keys = [("cuda", torch.bfloat16, s) for s in shapes]
    plan = build_plan(shapes, keys, world, 5)
    assert max(plan.load) / (sum(plan.load) / world) < 1.0001  # exact split for 1/2/4/8 ranks
    counts = {}
    for g in plan.groups:
        assert sorted(i for slot in g.slots for i in slot) == sorted(g.members)
        assert g.width == max(len(s) for s in g.slots)
        counts[g.key[2]] = [len(s) for s in g.slots]
    if world == 8:
        assert counts[(14336, 4096)] == [8] * 8 and counts[(4096, 14336)] == [4] * 8
        assert counts[(4096, 4096)] == [8] * 8 and counts[(1024, 4096)] == [8] * 8


def test_partition_is_deterministic_and_greedy():
    costs = [5.0, 3.0, 3.0, 2.0, 2.0, 1.0]
    owner = partition_by_flops(costs, 2)
    assert owner == partition_by_flops(costs, 2)
    loads = [sum(c for c, r in zip(costs, owner) if r == q) for q in range(2)]
    assert loads == [8.0, 8.0]
    assert partition_by_flops([1.0], 4) == [0]


def cpu_ops(momentum, lr, wd, mode, adjust):
    def do_momentum(grads, bufs, out):
        for j, (g, b) in enumerate(zip(grads, bufs)):
            out[j].copy_(o.momentum_update(g, b, momentum))

    def do_ns(x):
        return (x.float() * 3.0).to(x.dtype)  # stand-in, as in the golden fixtures

    def do_apply(params, updates):
        for p, u in zip(params, updates):
            o.apply_update(p, u.clone(), lr=lr, adjusted_lr=o.adjust_lr(lr, adjust, p.shape), weight_decay=wd,
                           weight_decay_mode=mode)
    return StepOps(momentum=do_momentum, orthogonalise=do_ns, apply=do_apply)


def make_problem():
    g = torch.Generator().manual_seed(77)
    shapes = [(24, 40), (24, 40), (24, 40), (40, 24), (2, 16, 16), (24, 40), (8, 64), (8, 64), (24, 40)]
    params = [(torch.randn(s, generator=g) * 0.02).bfloat16() for s in shapes]
    bufs = [(torch.randn(s, generator=g) * 1e-3).bfloat16() for s in shapes]
    grads = [[(torch.randn(s, generator=g) * 1e-3).bfloat16() for s in shapes] for _ in range(3)]
    return params, bufs, grads


def expected():
    params, bufs, grads = make_problem()
    for step_grads in grads:
        for p, b, g in zip(params, bufs, step_grads):
            u = o.momentum_update(g, b, (0.95, 0.9))
            u = (u.float() * 3.0).to(u.dtype)
            o.apply_update(p, u, lr=0.02, adjusted_lr=o.adjust_lr(0.02, "spectral", p.shape), weight_decay=0.01,
                           weight_decay_mode="base_lr")
    return params, bufs


def worker(rank, world, store_path, result_path):
    dist.init_process_group("gloo", init_method=f"file://{store_path}", rank=rank, world_size=world)
    try:
        params, bufs, grads = make_problem()
        ops = cpu_ops((0.95, 0.9), 0.02, 0.01, "base_lr", "spectral")
        # a tiny byte budget forces several chunks per group, exercising the ping-pong staging
        stepper = ShardedMuonStep(params, steps=5, ops=ops, max_group_bytes=2 * 24 * 40 * 2)
        owned = set(stepper.plan.owned(rank))
        buffers = {i: bufs[i] for i in owned}
        landing = [torch.zeros_like(g) for g in grads[0]]
        for n, step_grads in enumerate(grads):
            if n % 2 == 0:
                stepper.step(params, step_grads, buffers)
            else:
                # gradients handed over as host tensors: only the owned ones are copied in
                for t in landing:
                    t.fill_(float("nan"))
                stepper.step(params, landing, buffers, host_grads=step_grads)
                assert all(torch.equal(landing[i], step_grads[i]) for i in owned)
                assert all(torch.isnan(landing[i]).all() for i in range(len(landing)) if i not in owned)
        torch.save(dict(params=params, owned=sorted(owned), bufs={i: bufs[i] for i in owned}),
                   f"{result_path}.{rank}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_step_equals_unsharded(world):
    want_params, want_bufs = expected()
    with tempfile.TemporaryDirectory() as tmp:
        store, result = os.path.join(tmp, "store"), os.path.join(tmp, "result")
        mp.spawn(worker, args=(world, store, result), nprocs=world, join=True)
        seen = set()
        for rank in range(world):
            got = torch.load(f"{result}.{rank}")
            for p, w in zip(got["params"], want_params):
                assert torch.equal(p, w)           # parameters stay replicated and correct on every rank
            for i, b in got["bufs"].items():
                assert torch.equal(b, want_bufs[i])  # momentum lives with its owner
            seen |= set(got["owned"])
        assert seen == set(range(len(want_params)))


def test_step_with_host_gradients_equals_step_with_resident_gradients():
    """`host_grads` copies each owned gradient into the device-side tensor before its chunk runs
    (on CPU tensors the copy is synchronous; the stream/event plumbing is covered by the GPU test)."""
    want_params, want_bufs = expected()
    params, bufs, grads = make_problem()
    ops = cpu_ops((0.95, 0.9), 0.02, 0.01, "base_lr", "spectral")
    stepper = ShardedMuonStep(params, steps=5, ops=ops, max_group_bytes=2 * 24 * 40 * 2)
    buffers = {i: bufs[i] for i in stepper.plan.owned(0)}
    landing = [torch.zeros_like(g) for g in grads[0]]
    for step_grads in grads:
        stepper.step(params, landing, buffers, host_grads=step_grads)
    for p, w in zip(params, want_params):
        assert torch.equal(p, w)
    for i, b in buffers.items():
        assert torch.equal(b, want_bufs[i])


def adopting_worker(rank, world, store_path, result_path):
    dist.init_process_group("gloo", init_method=f"file://{store_path}", rank=rank, world_size=world)
    try:
        params, bufs, grads = make_problem()
        before = [p.clone() for p in params]
        ops = cpu_ops((0.95, 0.9), 0.02, 0.01, "base_lr", "spectral")
        stepper = ShardedMuonStep(params, steps=5, ops=ops, max_group_bytes=2 * 24 * 40 * 2, adopt_parameters=True)
        assert all(torch.equal(p, b) for p, b in zip(params, before))      # re-homing keeps the values
        flats = list(stepper._flat.values())
        assert flats and all(any(p.data_ptr() >= f.data_ptr() and p.data_ptr() < f.data_ptr() + f.numel() * f.element_size()
                                 for f in flats) for p in params)          # every parameter lives in a gather buffer
        buffers = {i: bufs[i] for i in stepper.plan.owned(rank)}
        for step_grads in grads:
            stepper.step(params, step_grads, buffers)
        torch.save(dict(params=[p.clone() for p in params]), f"{result_path}.{rank}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_adopted_parameters_are_updated_by_their_owner_and_gathered_in_place(world):
    """``adopt_parameters=True``: each rank applies the update only to the matrices it owns, and the in-place
    all-gather of the parameter storage gives every rank the same parameters as the unsharded step."""
    want_params, _ = expected()
    with tempfile.TemporaryDirectory() as tmp:
        store, result = os.path.join(tmp, "store"), os.path.join(tmp, "result")
        mp.spawn(adopting_worker, args=(world, store, result), nprocs=world, join=True)
        for rank in range(world):
            got = torch.load(f"{result}.{rank}")
            for p, w in zip(got["params"], want_params):
                assert torch.equal(p, w)


def checkpoint_worker(rank, world, store_path, result_path, phase):
    dist.init_process_group("gloo", init_method=f"file://{store_path}.{phase}", rank=rank, world_size=world)
    try:
        params, bufs, grads = make_problem()
        ops = cpu_ops((0.95, 0.9), 0.02, 0.01, "base_lr", "spectral")
        stepper = ShardedMuonStep(params, steps=5, ops=ops, max_group_bytes=2 * 24 * 40 * 2)
        owned = stepper.plan.owned(rank)
        if phase == "save":
            buffers = {i: bufs[i] for i in owned}
            for step_grads in grads[:2]:
                stepper.step(params, step_grads, buffers)
            full = stepper.state_dict(params, buffers)
            assert sorted(full["state"]) == list(range(len(params)))       # every matrix, on every rank
            if rank == 0:
                torch.save(dict(optimizer=full, params=params), result_path)
        else:
            saved = torch.load(result_path)
            for p, q in zip(params, saved["params"]):
                p.copy_(q)
            buffers = {}
            stepper.load_state_dict(saved["optimizer"], params, buffers)
            assert sorted(buffers) == sorted(owned)                          # only what this rank owns
            stepper.step(params, grads[2], buffers)
            torch.save(dict(params=params, bufs=buffers), f"{result_path}.{phase}.{rank}")
    finally:
        dist.destroy_process_group()


def test_sharded_state_dict_reloads_at_another_world_size_and_into_the_single_device_layout():
    """Two steps on 2 ranks, ``state_dict()`` (gathered: ``state[i]["momentum_buffer"]`` for every matrix, the
    layout of the reference's ``Muon.state_dict()``), reload on 3 ranks, one more step: parameters and
    momentum equal three unsharded steps."""
    want_params, want_bufs = expected()
    with tempfile.TemporaryDirectory() as tmp:
        store, result = os.path.join(tmp, "store"), os.path.join(tmp, "ckpt")
        mp.spawn(checkpoint_worker, args=(2, store, result, "save"), nprocs=2, join=True)
        saved = torch.load(result)["optimizer"]
        assert set(saved) == {"state", "param_groups"} and saved["param_groups"][0]["params"] == list(range(9))
        assert all(set(entry) == {"momentum_buffer"} for entry in saved["state"].values())
        mp.spawn(checkpoint_worker, args=(3, store, result, "load"), nprocs=3, join=True)
        seen = {}
        for rank in range(3):
            got = torch.load(f"{result}.load.{rank}")
            for p, w in zip(got["params"], want_params):
                assert torch.equal(p, w)
            seen.update(got["bufs"])
        assert sorted(seen) == list(range(9))
        for i, b in seen.items():
            assert torch.equal(b, want_bufs[i])


def test_sharded_state_dict_loads_into_the_single_device_optimizer():
    """The gathered state dict has the reference's layout (``state[i]["momentum_buffer"]`` per matrix and the
    caller's ``param_groups``), so ``Muon.load_state_dict`` takes it as it takes its own."""
    from i8muon_b200 import Muon
    params, bufs, grads = make_problem()
    ops = cpu_ops((0.95, 0.9), 0.02, 0.01, "base_lr", "spectral")
    stepper = ShardedMuonStep(params, steps=5, ops=ops)
    buffers = {i: bufs[i] for i in stepper.plan.owned(0)}
    stepper.step(params, grads[0], buffers)
    wrapped = [torch.nn.Parameter(p.clone()) for p in params]
    muon = Muon(wrapped, lr=0.02, weight_decay=0.01, momentum=(0.95, 0.9))
    full = stepper.state_dict(params, buffers, param_groups=muon.state_dict()["param_groups"])
    muon.load_state_dict(full)
    for i, p in enumerate(wrapped):
        assert torch.equal(muon.state[p]["momentum_buffer"], buffers[i])
    again = muon.state_dict()
    assert sorted(again["state"]) == list(range(len(params)))
    assert again["param_groups"][0]["weight_decay_mode"] == "base_lr"


def device_problem(dev):
    params, bufs, grads = make_problem()
    return ([p.to(dev) for p in params], [b.to(dev) for b in bufs], [[g.to(dev) for g in step] for step in grads])


def peer_copy_worker(rank, world, store_path, result_path):
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", init_method=f"file://{store_path}", rank=rank, world_size=world, device_id=dev)
    try:
        params, bufs, grads = device_problem(dev)
        ops = cpu_ops((0.95, 0.9), 0.02, 0.01, "base_lr", "spectral")
        stepper = ShardedMuonStep(params, steps=5, ops=ops, max_group_bytes=2 * 24 * 40 * 2, adopt_parameters=True,
                                  gather="copy")
        assert stepper.gather == "copy" and stepper._push_stream is not None
        buffers = {i: bufs[i] for i in stepper.plan.owned(rank)}
        for step_grads in grads:
            stepper.step(params, step_grads, buffers)
        torch.cuda.synchronize()
        torch.save(dict(params=[p.cpu() for p in params]), f"{result_path}.{rank}")
        dist.barrier()     # nobody unmaps a buffer that a peer may still hold open
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
def test_peer_copy_gather_gives_every_rank_the_unsharded_parameters(cuda_device):
    """``gather="copy"``: two ranks on two GPUs map each other's flat parameter buffers (symmetric
    memory) and push their updated blocks with device-to-device copies; both end up with the parameters
    of the unsharded step.  Symmetric memory refuses two ranks on one device, so a box with a single
    GPU skips this."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    params, bufs, grads = device_problem(cuda_device)
    ops = cpu_ops((0.95, 0.9), 0.02, 0.01, "base_lr", "spectral")
    single = ShardedMuonStep(params, steps=5, ops=ops, max_group_bytes=2 * 24 * 40 * 2)
    buffers = {i: bufs[i] for i in single.plan.owned(0)}
    for step_grads in grads:
        single.step(params, step_grads, buffers)
    want = [p.cpu() for p in params]
    with tempfile.TemporaryDirectory() as tmp:
        store, result = os.path.join(tmp, "store"), os.path.join(tmp, "result")
        mp.spawn(peer_copy_worker, args=(2, store, result), nprocs=2, join=True)
        for rank in range(2):
            got = torch.load(f"{result}.{rank}")
            for p, w in zip(got["params"], want):
                assert torch.equal(p, w)


def test_chunk_plan_keeps_the_first_chunk_small_and_the_tail_fine():
    """The step consumes shape groups in chunks: the very first chunk is at most ``first_chunk_bytes`` (nothing hides
    its gradient copy), and with more than one rank the last two groups are cut to ``tail_chunk_bytes`` (a chunk's
    transfer to the peers runs under the next chunk of the same group).  Every slot is covered exactly once."""
    shapes = LLAMA_LAYER * 32
    params = [torch.empty(s, dtype=torch.bfloat16, device="meta") for s in shapes]
    ops = cpu_ops((0.95, 0.9), 0.02, 0.01, "base_lr", "spectral")
    stepper = ShardedMuonStep(params, steps=5, ops=ops)          # one rank
    chunks = stepper._chunk_list
    first_group, _, first_width, _ = chunks[0]
    assert first_width * 14336 * 4096 * 2 <= stepper.first_chunk_bytes and first_width >= 1
    for g in stepper.plan.groups:
        covered = sorted((first, width) for grp, first, width, _ in chunks if grp is g)
        assert covered[0][0] == 0 and sum(w for _, w in covered) == g.width
        assert all(a + w == b for (a, w), (b, _) in zip(covered, covered[1:]))
    # eight ranks: same plan code, the rank count only enters through the partition and the tail rule
    keys = [("cuda", torch.bfloat16, s) for s in shapes]
    stepper.world = 8
    stepper.plan = build_plan(shapes, keys, 8, 5)
    chunks = stepper._plan_chunks(params)
    tail_groups = stepper.plan.groups[-2:]
    for grp, first, width, _ in chunks:
        numel = 1
        for d in shapes[grp.members[0]]:
            numel *= d
        if any(grp is t for t in tail_groups):
            assert width * numel * 2 <= stepper.tail_chunk_bytes or width == 1
    assert [parity for *_, parity in chunks] == [i & 1 for i in range(len(chunks))]
    assert len([c for c in chunks if any(c[0] is t for t in tail_groups)]) >= 3   # q/o in three chunks + k/v
