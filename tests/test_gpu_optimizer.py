"""The optimizer step on the GPU: fused momentum / apply kernels against fixtures
produced by the reference's own muon_step, grouping and CUDA-graph plumbing, and
the reference's example training loop."""
import numpy as np
import pytest
import torch

import gpu_helpers as H
from i8muon_b200 import CutlassNSInt8, Muon, check_status, muon_step, native, recommend_coefficients
from oracle import ns_oracle as o

pytestmark = pytest.mark.gpu
C5 = recommend_coefficients(5)
DT = {"torch.float32": torch.float32, "torch.bfloat16": torch.bfloat16, "torch.float16": torch.float16}


def fused_step(p, b, g, case):
    """momentum kernel -> stand-in NS (3x, as in the fixtures) -> apply kernel."""
    stream = torch.cuda.current_stream().cuda_stream
    momentum = case["momentum"]
    mu, mu2 = momentum[0], momentum[-1]
    update = torch.empty((1, *g.shape), device=g.device, dtype=g.dtype)
    native.call("i8m_momentum", native.pointer_array([g.data_ptr()]), native.pointer_array([b.data_ptr()]), 1,
                update.data_ptr(), g.numel(), H.DT[g.dtype], 1.0 - mu2, mu, int(len(momentum) == 2), None, stream)
    ortho = (update.float() * 3.0).to(update.dtype)
    lr, wd = case["lr"], case["wd"]
    adjusted = o.adjust_lr(lr, case["adjust"], p.shape)
    if wd == 0:
        mode, decay = 0, 0.0
    elif case["mode"] == "adjusted_lr":
        mode, decay = 2, wd
    elif case["mode"] == "absolute":
        mode, decay = 1, 1.0 - wd
    else:
        mode, decay = 1, 1.0 - lr * wd
    native.call("i8m_apply", native.pointer_array([p.data_ptr()]), 1, ortho.data_ptr(), p.numel(), H.DT[p.dtype],
                H.DT[g.dtype], mode, decay, -adjusted, stream)


def test_fused_step_kernels_match_reference_fixtures(cuda_device, host_golden, step_golden):
    """Against tensors produced by the reference's muon_step on CPU tensors.

    FP32 cases must match bit for bit.  For 16-bit tensors torch's CPU `add_(alpha=)`
    rounds alpha to the tensor's dtype while its CUDA kernel (the only device the
    reference runs on) keeps alpha in FP32, so those fixtures pin the momentum
    buffer bit for bit and the parameter to two units in the last place; the
    CUDA sequence itself is pinned exactly by the next test."""
    mismatched = []
    for case in host_golden["muon_step_cases"]:
        key = case["key"]
        dtype = DT[case["dtype"]]
        p = step_golden[key + ".param0"].to(cuda_device)
        b = step_golden[key + ".buf0"].to(cuda_device)
        for s in range(2):
            fused_step(p, b, step_golden[f"{key}.grad{s}"].to(cuda_device), case)
            want_p, want_b = step_golden[f"{key}.param{s + 1}"], step_golden[f"{key}.buf{s + 1}"]
            if dtype == torch.float32:
                good = torch.equal(p.cpu(), want_p) and torch.equal(b.cpu(), want_b)
            else:
                ulp = 2.0 ** (-7 if dtype == torch.bfloat16 else -10)
                scale = want_p.float().abs() + 0.03 * case["lr"] * 8  # cancellation between decay and update
                good = torch.equal(b.cpu(), want_b) and bool(
                    ((p.cpu().float() - want_p.float()).abs() <= 2 * ulp * scale).all())
                p.copy_(want_p)  # do not let a last-place difference compound into the next step
            if not good:
                mismatched.append((key, s))
    assert not mismatched, mismatched


def torch_cuda_step(p, b, g, *, momentum, lr, wd, mode, adjust):
    """The reference's statements (src/i8muon/_optimizer.py:446-511) executed by torch on the GPU."""
    mu, mu2 = momentum[0], momentum[-1]
    b.lerp_(g, 1 - mu2)
    update = g.lerp(b, mu) if len(momentum) == 2 else b
    update = (update.float() * 3.0).to(update.dtype)
    factor = {"absolute": 1 - wd, "base_lr": 1 - lr * wd, "adjusted_lr": None}[mode]
    if wd != 0:
        if factor is None:
            update.add_(p, alpha=wd)
        else:
            p.mul_(factor)
    p.add_(update, alpha=-o.adjust_lr(lr, adjust, p.shape))


@pytest.mark.parametrize("pdtype,gdtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                           (torch.float16, torch.float16), (torch.float32, torch.bfloat16)])
def test_fused_step_kernels_match_torch_cuda_sequence(cuda_device, pdtype, gdtype):
    """Bit-exact against the same statements run by torch's CUDA kernels, which is
    how the reference executes them; covers the vector path, the tail and every decay mode."""
    g = torch.Generator().manual_seed(31)
    for shape in [(257, 131), (64, 64), (3, 5, 7)]:
        for momentum in ((0.95, 0.95), (0.9,), (0.3, 0.8)):
            for mode, wd in (("base_lr", 0.01), ("adjusted_lr", 0.01), ("absolute", 0.001), ("base_lr", 0.0)):
                case = dict(momentum=list(momentum), mode=mode, wd=wd, adjust="match_rms_adamw", lr=0.02)
                p = (torch.randn(shape, generator=g) * 0.02).to(pdtype).to(cuda_device)
                b = (torch.randn(shape, generator=g) * 1e-3).to(gdtype).to(cuda_device)
                p_ref, b_ref = p.clone(), b.clone()
                for _ in range(2):
                    grad = (torch.randn(shape, generator=g) * 1e-3).to(gdtype).to(cuda_device)
                    fused_step(p, b, grad, case)
                    torch_cuda_step(p_ref, b_ref, grad, momentum=momentum, lr=0.02, wd=wd, mode=mode,
                                    adjust="match_rms_adamw")
                    assert torch.equal(b, b_ref), (shape, momentum, mode)
                    assert torch.equal(p, p_ref), (shape, momentum, mode)


def reference_step(params, grads, bufs, engine, **kw):
    """The reference's per-parameter loop: torch's CUDA kernels for the momentum /
    decay / update statements, one un-batched NS call per parameter."""
    for p, g, b in zip(params, grads, bufs):
        u = o.momentum_update(g, b, kw["momentum"])
        fn, actual = engine.router(*g.shape[-2:], kw["precision"], kw["use_gram"], 5.0)
        u = fn(u, kw["coeffs"], 1e-7, True, actual)
        o.apply_update(p, u, lr=kw["lr"], adjusted_lr=o.adjust_lr(kw["lr"], kw["adjust"], p.shape),
                       weight_decay=kw["wd"], weight_decay_mode=kw["mode"])


@pytest.mark.parametrize("precision,dtype", [("float16", torch.float32), ("bfloat16", torch.bfloat16),
                                             ("int8", torch.float32), ("int8_bq", torch.bfloat16),
                                             ("fp8", torch.bfloat16), ("auto", torch.float32)])
def test_muon_step_grouped_equals_per_parameter(cuda_device, precision, dtype):
    g = torch.Generator().manual_seed(21)
    shapes = [(64, 160), (64, 160), (160, 64), (2, 48, 48), (64, 160), (1100, 1024)]
    params = [(torch.randn(s, generator=g) * 0.02).to(dtype).to(cuda_device) for s in shapes]
    grads = [(torch.randn(s, generator=g) * 1e-3).to(dtype).to(cuda_device) for s in shapes]
    bufs = [(torch.randn(s, generator=g) * 1e-3).to(dtype).to(cuda_device) for s in shapes]
    ref = [[t.clone() for t in ts] for ts in (params, grads, bufs)]
    engine = CutlassNSInt8()
    kw = dict(lr=0.02, wd=0.01, momentum=(0.95, 0.95), adjust="match_rms_adamw", mode="base_lr",
              precision=precision, use_gram=False, coeffs=C5)
    for _ in range(2):
        muon_step(params, grads, bufs, lr=kw["lr"], weight_decay=kw["wd"], momentum=kw["momentum"],
                  ns_coefficients=C5, eps=1e-7, adjust_lr_fn=kw["adjust"], ns_engine=engine,
                  precision=precision, use_gram=False, weight_decay_mode=kw["mode"])
        reference_step(ref[0], ref[1], ref[2], engine, **kw)
    check_status()
    for got, want in zip(params + bufs, ref[0] + ref[2]):
        assert torch.equal(got, want)


def test_muon_optimizer_cuda_graph_matches_eager(cuda_device):
    def model_params(seed):
        g = torch.Generator().manual_seed(seed)
        return [torch.nn.Parameter((torch.randn(s, generator=g) * 0.02).to(torch.bfloat16).to(cuda_device))
                for s in [(96, 256), (96, 256), (256, 96), (3, 64, 64)]]
    results = []
    for use_graph in (False, True):
        params = model_params(5)
        opt = Muon(params, lr=0.02, weight_decay=0.01, precision="bfloat16", use_cuda_graph=use_graph,
                   adjust_lr_fn="match_rms_adamw")
        g = torch.Generator().manual_seed(6)
        for step in range(4):
            for p in params:
                # write into the same .grad storage every step, as autograd accumulation does
                new = (torch.randn(p.shape, generator=g) * 1e-3).to(p.dtype).to(cuda_device)
                if p.grad is None:
                    p.grad = new
                else:
                    p.grad.copy_(new)
            opt.step()
        check_status()
        results.append([p.detach().clone() for p in params])
        if use_graph:
            assert len(opt._ns_graphs) == 3  # one graph per distinct shape group
            state = opt.state_dict()
            opt.load_state_dict(state)
            assert len(opt._ns_graphs) == 0   # loading state drops captured graphs
    for eager, graphed in zip(*results):
        assert torch.equal(eager, graphed)


def test_example_training_loop(cuda_device):
    """The reference's offline example: a two-layer MLP, Muon for matrices and
    AdamW for vectors, three steps (examples/optimizer.py of the reference)."""
    torch.manual_seed(42)
    model = torch.nn.Sequential(torch.nn.Linear(128, 128), torch.nn.GELU(), torch.nn.Linear(128, 32)).to(cuda_device)
    matrices = [p for p in model.parameters() if p.ndim >= 2]
    vectors = [p for p in model.parameters() if p.ndim < 2]
    for precision in ("int8", "int8_bq", "fp8_bq", "float16"):
        optimizer = Muon(matrices, lr=1e-3, precision=precision, ns_steps=5, use_cuda_graph=True,
                         scalar_optimizer=torch.optim.AdamW(vectors, lr=1e-3))
        losses = []
        inputs = torch.randn(8, 128, device=cuda_device)
        targets = torch.randn(8, 32, device=cuda_device)
        for _ in range(3):
            loss = (model(inputs) - targets).square().mean()
            loss.backward()
            optimizer.step()
            optimizer.zero_grad(set_to_none=False)
            losses.append(loss.item())
        check_status()
        assert all(np.isfinite(losses)) and losses[-1] < losses[0]


def test_sharded_step_streams_host_gradients(cuda_device):
    """`ShardedMuonStep.step(host_grads=...)`: pinned host gradients copied chunk by chunk on a side
    stream give bit-identical parameters and momentum to the same steps on resident gradients,
    over several steps (the copies of step n+1 may only start once step n has read a chunk)."""
    from i8muon_b200.optimizer import native_step_ops
    from i8muon_b200.sharding import ShardedMuonStep
    g = torch.Generator().manual_seed(33)
    shapes = [(256, 384)] * 5 + [(384, 256)] * 2 + [(128, 128)] * 3
    host = [[(torch.randn(s, generator=g) * 1e-3).bfloat16().pin_memory() for s in shapes] for _ in range(3)]
    start = [(torch.randn(s, generator=g) * 0.02).bfloat16() for s in shapes]
    engine = CutlassNSInt8()
    ops = native_step_ops(engine, lr=0.02, weight_decay=0.01, momentum=0.95, ns_coefficients=C5,
                          adjust_lr_fn="match_rms_adamw", precision="int8_bq", use_gram=False)
    results = []
    for streamed in (False, True):
        params = [p.clone().to(cuda_device) for p in start]
        landing = [torch.zeros(s, dtype=torch.bfloat16, device=cuda_device) for s in shapes]
        stepper = ShardedMuonStep(params, 5, ops, max_group_bytes=2 * 256 * 384 * 2)  # several chunks per group
        buffers = {i: torch.zeros_like(landing[i]) for i in stepper.plan.owned(0)}
        for step_grads in host:
            if streamed:
                stepper.step(params, landing, buffers, host_grads=step_grads)
            else:
                stepper.step(params, [t.to(cuda_device) for t in step_grads], buffers)
        torch.cuda.synchronize()
        check_status()
        results.append((params, buffers))
    for a, b in zip(results[0][0], results[1][0]):
        assert torch.equal(a, b)
    for i in results[0][1]:
        assert torch.equal(results[0][1][i], results[1][1][i])


@pytest.mark.parametrize("pdtype", [torch.float32, torch.bfloat16])
def test_fused_adamw_matches_torch_adamw(cuda_device, pdtype):
    """FusedAdamW (one multi-tensor launch) against torch.optim.AdamW's single-tensor statements in
    FP32, on tensors of unequal, odd sizes over several steps; it also works in Muon's
    scalar_optimizer slot.  BF16 parameters are held to one BF16 ulp of the FP32 trajectory."""
    from i8muon_b200 import FusedAdamW
    g = torch.Generator().manual_seed(5)
    shapes = [(50257, 3), (7,), (1, 1025), (64,)] + [(33,)] * 30      # more than one table of 24
    start = [torch.randn(s, generator=g) * 0.1 for s in shapes]
    grads = [[torch.randn(s, generator=g) * 0.01 for s in shapes] for _ in range(4)]
    kw = dict(lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ref_params = [p.clone().to(cuda_device).requires_grad_() for p in start]
    ref = torch.optim.AdamW(ref_params, foreach=False, fused=False, **kw)
    ours_params = [p.clone().to(pdtype).to(cuda_device).requires_grad_() for p in start]
    ours = FusedAdamW(ours_params, **kw)
    for step_grads in grads:
        for p, q, gr in zip(ref_params, ours_params, step_grads):
            p.grad = gr.to(pdtype).float().to(cuda_device)   # both see the same (rounded) gradient values
            q.grad = gr.to(pdtype).to(cuda_device)
        ref.step()
        ours.step()
    for p, q in zip(ref_params, ours_params):
        if pdtype == torch.float32:
            torch.testing.assert_close(q, p, rtol=2e-6, atol=2e-8)   # parameters are O(0.1): a few FP32 ulps
        else:
            # a BF16 parameter re-rounds after every step: allow the accumulated half-ulps of a value
            # that moved by up to lr per step (Adam's normalised update) on its way to p
            # (five roundings of up to half an ulp = 2^-8 relative each, one spare)
            assert ((q.float() - p).abs() <= 6 * 2.0 ** -8 * (p.abs() + 4 * kw["lr"])).all()
    state = ours.state[ours_params[0]]
    assert state["step"] == 4 and state["exp_avg"].dtype == torch.float32
    # in Muon's scalar_optimizer slot
    w = (torch.randn((64, 96), generator=g) * 0.02).to(cuda_device).requires_grad_()
    v = torch.zeros(96, device=cuda_device, requires_grad=True)
    opt = Muon([w], lr=0.02, scalar_optimizer=FusedAdamW([v], lr=1e-2))
    w.grad = torch.randn_like(w) * 1e-3
    v.grad = torch.ones_like(v)
    opt.step()
    check_status()
    assert torch.all(v < 0) and len(opt.param_groups) == 2


def test_captured_graphs_survive_reallocated_gradients(cuda_device):
    """``backward()`` + ``zero_grad()`` with PyTorch's default ``set_to_none=True`` give every step freshly
    allocated gradients.  The captured Newton-Schulz graphs are keyed by shape and settings only (they
    read a static update buffer), so their number stays at the number of shape groups, and the graphed
    optimizer follows the eager one bit for bit."""
    torch.manual_seed(7)
    def model():
        torch.manual_seed(7)
        return torch.nn.Sequential(torch.nn.Linear(256, 128, bias=False), torch.nn.GELU(),
                                   torch.nn.Linear(128, 128, bias=False), torch.nn.GELU(),
                                   torch.nn.Linear(128, 128, bias=False), torch.nn.Linear(128, 64, bias=False)).to(cuda_device)
    nets = [model(), model()]
    opts = [Muon(nets[0].parameters(), lr=0.01, precision="int8_bq", use_cuda_graph=False),
            Muon(nets[1].parameters(), lr=0.01, precision="int8_bq", use_cuda_graph=True)]
    inputs = torch.randn(10, 16, 256, device=cuda_device)
    keep = []          # hold on to old gradients so that new ones cannot land on the same addresses
    for step in range(10):
        for net, opt in zip(nets, opts):
            net(inputs[step]).square().mean().backward()
            keep.extend(p.grad for p in net.parameters())
            opt.step()
            opt.zero_grad()                      # default: set_to_none=True
        assert len(opts[1]._ns_graphs) == 3      # 256x128, 128x128 (two matrices, one call), 128x64
    check_status()
    for p, q in zip(nets[0].parameters(), nets[1].parameters()):
        assert torch.equal(p, q)
    assert len({g.data_ptr() for g in keep}) == len(keep)


def test_captured_graph_cache_is_bounded(cuda_device, monkeypatch):
    from i8muon_b200 import optimizer as module
    monkeypatch.setattr(module, "MAX_CAPTURED_GRAPHS", 2)
    params = [torch.nn.Parameter(torch.randn(64 + 16 * i, 128, device=cuda_device) * 0.02) for i in range(4)]
    for p in params:
        p.grad = torch.randn_like(p) * 1e-3
    opt = Muon(params, lr=0.01, precision="float16", use_cuda_graph=True)
    opt.step()
    opt.step()
    check_status()
    assert len(opt._ns_graphs) == 2


def test_a_reported_status_word_raises_at_the_next_step(cuda_device):
    """A kernel that gave up a wait writes a code to the status word.  ``step()`` copies the word to pinned
    memory when it ends and looks at the copy when the next step begins, without a synchronisation in
    between; here the word is set by the test itself (no kernel is made to time out)."""
    from i8muon_b200.engine import status_word
    p = torch.nn.Parameter(torch.randn(64, 128, device=cuda_device) * 0.02)
    p.grad = torch.randn_like(p) * 1e-3
    opt = Muon([p], lr=0.01, precision="float16")
    opt.step()
    torch.cuda.synchronize()
    opt.step()                                   # clean word: nothing raised
    status_word(cuda_device).fill_(0x2007)       # what an epilogue timeout of CTA 7 would leave
    opt.step()                                   # this step ends by posting the word
    torch.cuda.synchronize()
    with pytest.raises(native.NativeError, match="0x2007"):
        opt.step()
    torch.cuda.synchronize()
    assert int(status_word(cuda_device).item()) == 0
    opt.step()                                   # cleared: training can go on (or stop) by the caller's choice
    check_status()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(300, 517), (64, 128), (1024, 4096)])
def test_momentum_kernel_leaves_the_statistics_of_its_update(cuda_device, dtype, shape):
    """The partial sums of squares and maxima that ``i8m_momentum`` writes for the update are the ones the
    statistics pass computes over the same tensor (one chunk mapping for both kernels), so the norm that
    Newton-Schulz takes from them is bit-identical and the entry point gives the same result with or without."""
    dev = cuda_device
    g = torch.Generator().manual_seed(3)
    count = 3
    grads = [(torch.randn(shape, generator=g) * 1e-3).to(dtype).to(dev) for _ in range(count)]
    bufs = [(torch.randn(shape, generator=g) * 1e-3).to(dtype).to(dev) for _ in range(count)]
    numel = grads[0].numel()
    update = torch.empty((count, *shape), device=dev, dtype=dtype)
    stats = torch.full((native.stats_scratch_bytes(count, numel) // 4,), float("nan"), device=dev)
    native.call("i8m_momentum", native.pointer_array([t.data_ptr() for t in grads]),
                native.pointer_array([t.data_ptr() for t in bufs]), count, update.data_ptr(), numel, H.DT[dtype],
                0.05, 0.95, 1, stats.data_ptr(), torch.cuda.current_stream().cuda_stream)
    # the statistics pass over the update, partials included
    nbytes = native.stats_scratch_bytes(count, numel)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    norm, amax = torch.empty(count, device=dev), torch.empty(count, device=dev)
    native.call("i8m_stats", update.data_ptr(), H.DT[dtype], count, numel, scratch.data_ptr(), nbytes, norm.data_ptr(),
                amax.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert torch.equal(stats, scratch.view(torch.float32))
    engine = CutlassNSInt8()
    plain = engine._regular_bq(update, C5, 1e-7, True, "int8_bq")
    fed = engine._regular_bq(update, C5, 1e-7, True, "int8_bq", stats=stats)
    check_status()
    assert torch.equal(plain, fed)
    with pytest.raises(ValueError, match="stats must be"):
        engine._regular_bq(update, C5, 1e-7, True, "int8_bq", stats=stats[:2])
