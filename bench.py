"""Benchmark of the Muon step over a Llama-3-8B-shaped parameter set on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference|reference-gpu]
                    [--config cfg4-int8bq|cfg4-fp8bq|cfg1|cfg2|cfg2-gram|cfg3|cfg5]

The default configuration (cfg4-int8bq) is the headline below; the others are the remaining
configurations of the baseline list, each timed through the drop-in ``Muon(...).step()``.

One "step" is one full optimizer step (momentum, Newton-Schulz, weight decay and
update) over 224 synthetic matrices: 32 layers x {q 4096x4096, k 1024x4096,
v 1024x4096, o 4096x4096, gate 14336x4096, up 14336x4096, down 4096x14336}, BF16
weights N(0, 0.02) and gradients N(0, 1e-3), 128x128 block-quantised INT8 with
the reference's default first FP16 iteration, five int8_safe iterations.

metric  muon_step_ns_tflops: algorithmic Newton-Schulz flops of the whole set
        (T (4 l^2 h + 2 l^3) per matrix = 6.659e14) per second of step time, all
        ranks together; ms_per_step is the step latency.
N > 1   launched by torch.distributed.run; matrices are partitioned across ranks
        by flops, each rank orthogonalises its share, updates are all-gathered
        (strong scaling: the parameter set is fixed).
e2e     the same step with that step's gradients copied from pinned host memory
        inside the timed region and a scalar metric read back.
roofline  the block-quantised INT8 update GEMM timed alone with CUDA events on
        the gate/up shape, against twice the measured BF16 tensor peak.
cpu_baseline / --impl reference
        the reference has no CPU implementation of this path; its README formula
        X <- (a I + b G + c G^2) X in FP32 torch, driven by the reference's step
        statements, is timed on the host cores on a bounded sample of the set.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LAYER = [("q", 4096, 4096), ("k", 1024, 4096), ("v", 1024, 4096), ("o", 4096, 4096),
         ("gate", 14336, 4096), ("up", 14336, 4096), ("down", 4096, 14336)]
NS_STEPS = 5
LR, WD, MOMENTUM = 0.02, 0.01, (0.95, 0.95)


def shapes(layers: int):
    return [(rows, cols) for _ in range(layers) for _, rows, cols in LAYER]


def ns_flops_of(shape_list):
    from i8muon_b200.sharding import ns_flops
    return sum(ns_flops(s, NS_STEPS) for s in shape_list)


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return data, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """nvidia-smi clock and throttle-reason samples during the timed region."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            pass

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        rows = [line.split(",") for line in Path(self.file.name).read_text().splitlines() if line.count(",") >= 8]
        os.unlink(self.file.name)
        clocks, maxima, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in rows:
            try:
                clocks.append(float(row[1]))
                maxima.append(float(row[2]))
            except ValueError:
                continue
            for name, value in zip(names, row[5:9]):
                if value.strip().lower().startswith("active"):
                    reasons.add(name)
        busy = [c for c in clocks if c > 0.5 * max(clocks)] if clocks else []
        return {"sm_mhz": statistics.median(busy) if busy else None,
                "sm_max_mhz": max(maxima) if maxima else None, "reasons": sorted(reasons), "samples": len(clocks)}


# ----------------------------------------------------------------------------- CPU arm
def cpu_sample_step(sample, coeffs):
    """The reference's step statements on CPU tensors with the FP32 torch Newton-Schulz."""
    from oracle import ns_oracle as o
    for p, g, b in sample:
        u = o.momentum_update(g, b, MOMENTUM)
        u = o.ns_fp32_torch(u, coeffs)
        o.apply_update(p, u, lr=LR, adjusted_lr=o.adjust_lr(LR, "match_rms_adamw", p.shape), weight_decay=WD,
                       weight_decay_mode="base_lr")


def make_cpu_sample():
    gen = torch.Generator().manual_seed(4000)
    sample_shapes = [(1024, 4096), (4096, 4096), (14336, 4096), (4096, 14336)]   # one matrix per distinct shape
    sample = []
    for s in sample_shapes:
        p = (torch.randn(s, generator=gen) * 0.02).bfloat16()
        g = (torch.randn(s, generator=gen) * 1e-3).bfloat16()
        sample.append((p, g, torch.zeros_like(g)))
    return sample, sample_shapes


def time_cpu(steps: int, warmup: int):
    from i8muon_b200 import recommend_coefficients
    torch.set_num_threads(os.cpu_count() or 1)
    coeffs = recommend_coefficients(NS_STEPS)
    sample, sample_shapes = make_cpu_sample()
    for _ in range(warmup):
        cpu_sample_step(sample, coeffs)
    start = time.perf_counter()
    for _ in range(steps):
        cpu_sample_step(sample, coeffs)
    seconds = (time.perf_counter() - start) / steps
    flops = ns_flops_of(sample_shapes)
    return {"value": flops / seconds / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": "one matrix per distinct shape per step (k 1024x4096, q 4096x4096, gate 14336x4096, down "
                      f"4096x14336), FP32 torch NS, {flops:.3e} flop, {seconds:.2f} s/step", "seconds_per_step": seconds}


def config_dict(world: int, layers: int, precision: str, fp16_first: bool):
    return {"workload": f"llama3-8b-shaped parameter set, {layers} layers x 7 matrices, bf16, "
                        f"precision={precision}, fp16_first={fp16_first}, ns_steps={NS_STEPS} int8_safe",
            "matrices": layers * len(LAYER), "ns_steps": NS_STEPS, "precision": precision,
            "fp16_first": fp16_first, "parallelism": f"flop-partitioned x{world}; updated parameters pushed to the peers (or all-gathered)",
            "l2": "inputs (3 x 14 GB) are larger than L2; no flush needed"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 5))
    cpu = time_cpu(steps, min(args.warmup, 1))
    line = {"impl": "reference", "metric": "muon_step_ns_tflops", "value": cpu["value"], "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 1),
            "ms_per_step": cpu["seconds_per_step"] * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_dict(args.gpus, args.layers, args.precision, bool(args.fp16_first)),
            "cpu_baseline": {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": cpu["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "the reference has no CPU implementation of this path (it refuses non-CUDA tensors); this is "
                    "its README formula in FP32 torch under its own step statements, on a bounded sample"}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- reference kernels on this GPU
def run_reference_gpu(args):
    """The reference's own optimizer and CUDA kernels (oracle/_ref, built for sm_100a) on the same set.

    A same-box baseline next to the headline, not the ``--impl reference`` arm (which stays the host-core
    path): ``Muon(...).step()`` of the unmodified reference, one Newton-Schulz call per matrix as it does,
    its cp.async + mma.sync tiles, timed with CUDA events.
    """
    from oracle import reference_gpu
    if not reference_gpu.available():
        print(json.dumps({"impl": "reference-gpu", "unavailable": "oracle/_ref is not built on this machine"}))
        return
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    ref = reference_gpu.load()
    shape_list = shapes(args.layers)
    gen = torch.Generator(device=dev).manual_seed(4000)
    params = [torch.nn.Parameter((torch.randn(s, device=dev, generator=gen) * 0.02).bfloat16()) for s in shape_list]
    for p in params:
        p.grad = (torch.randn(p.shape, device=dev, generator=gen) * 1e-3).bfloat16()
    opt = ref.Muon(params, lr=LR, weight_decay=WD, momentum=MOMENTUM, ns_steps=NS_STEPS,
                   adjust_lr_fn="match_rms_adamw", precision=args.precision, fp16_first=bool(args.fp16_first),
                   use_gram=False)
    steps, warmup = max(1, min(args.steps, 3)), max(1, min(args.warmup, 2))
    for _ in range(warmup):
        opt.step()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(steps):
        opt.step()
    end.record()
    torch.cuda.synchronize()
    seconds = start.elapsed_time(end) / 1e3 / steps
    flops = ns_flops_of(shape_list)
    finite = all(bool(torch.isfinite(p).all()) for p in params[:7])
    print(json.dumps({"impl": "reference-gpu", "metric": "muon_step_ns_tflops", "value": flops / seconds / 1e12,
                      "unit": "TFLOP/s", "ms_per_step": seconds * 1e3, "steps": steps, "warmup": warmup,
                      "config": config_dict(1, args.layers, args.precision, bool(args.fp16_first)),
                      "finite": finite, "gpu": torch.cuda.get_device_name(0),
                      "what": "i8muon 0.2.0 Muon.step(), its csrc/*.cu built for sm_100a (cp.async + mma.sync "
                              "tiles), one NS call per matrix"}), flush=True)


def reference_gpu_leg(args):
    """Run the leg above in a child process (its 42 GB of tensors are freed with it)."""
    from oracle import reference_gpu
    if not reference_gpu.available():
        return None
    command = [sys.executable, str(ROOT / "bench.py"), "--impl", "reference-gpu", "--steps", "2", "--warmup", "1",
               "--layers", str(args.layers), "--precision", args.precision, "--fp16-first", str(args.fp16_first)]
    try:
        done = subprocess.run(command, capture_output=True, text=True, timeout=600)
        lines = [ln for ln in done.stdout.splitlines() if ln.startswith("{")]
        if not lines:
            return {"unavailable": (done.stderr or "no output")[-300:]}
        full = json.loads(lines[-1])
        return {k: full[k] for k in ("value", "unit", "ms_per_step", "steps", "what", "gpu", "unavailable") if k in full}
    except (subprocess.TimeoutExpired, json.JSONDecodeError) as err:
        return {"unavailable": str(err)[-300:]}


# ----------------------------------------------------------------------------- the other configurations
def gram_flops(l, h, steps, order="00100"):
    """Algorithmic flops of the Gram-space iteration with restart string ``order``
    (the products of src/i8muon/_cutlass_prec.py:111-130, dense count)."""
    order = order + "0" * max(0, steps - len(order))
    wide, square = 2.0 * l * l * h, 2.0 * l ** 3
    total = wide                                             # final Q0 * A
    for t in range(steps):
        kind = order[t]
        refresh = t + 1 < steps and order[t + 1] == "0"
        if kind == "1":
            total += wide                                    # A <- Q0 * A
        total += (wide + square) if (kind == "1" or t == 0) else 2 * square
        if refresh:
            total += 2 * square
    return total


def other_config(name):
    """Synthetic stand-ins for the baseline configurations other than the headline one: shapes,
    dtypes and value distributions as the configuration states them, seeded."""
    from i8muon_b200 import recommend_coefficients
    bf16, f32 = torch.bfloat16, torch.float32
    if name == "cfg1":
        return dict(shapes=[(1024, 4096)], pdtype=f32, gdtype=f32, pstd=1.0, gstd=1.0, steps=5, method="int8_safe",
                    muon=dict(precision="float32", use_gram=False), graph=True, peak="tf32x3",
                    what="FP32 regular NS (3 x TF32 products), one 1024x4096 matrix, int8_safe x5")
    if name == "cfg2":
        return dict(shapes=[(768, 3072)] * 48, pdtype=bf16, gdtype=bf16, pstd=0.02, gstd=0.02, steps=5,
                    method="int8_safe", muon=dict(precision="bfloat16", use_gram=False), graph=True, peak="bf16",
                    what="BF16 regular NS, 48 matrices of 768x3072 in one batched call, int8_safe x5")
    if name == "cfg2-gram":
        return dict(shapes=[(1024, 8192)] * 48, pdtype=bf16, gdtype=bf16, pstd=0.02, gstd=0.02, steps=5,
                    method="int8_safe", muon=dict(precision="bfloat16", use_gram=True), graph=True, peak="bf16",
                    gram=True, what="BF16 Gram-space NS (aspect 8 >= 5, restart order 00100), 48 matrices of 1024x8192")
    if name == "cfg3":
        return dict(shapes=[(4096, 4096)] * 16, pdtype=f32, gdtype=f32, pstd=0.02, gstd=1e-3, steps=6,
                    method="int8_safe", outliers=True, muon=dict(precision="int8", use_gram=False, fp16_first=True),
                    graph=True, peak="int8",
                    what="global INT8 NS with FP16 first row, 16 matrices of 4096x4096 FP32, 1 % of entries x50, int8_safe x6")
    if name == "cfg5":
        layer = [(2048, 2048)] * 4 + [(8192, 2048), (2048, 8192)]
        return dict(shapes=layer * 24, pdtype=bf16, gdtype=bf16, pstd=0.02, gstd=1e-3, steps=8, method="polar_express",
                    muon=dict(precision="float16", use_gram=True, gram_aspect_threshold=4.0, weight_decay=0.01,
                              adjust_lr_fn="match_rms_adamw", momentum=(0.95, 0.95)),
                    graph=True, peak="bf16", gram_shapes={(8192, 2048), (2048, 8192)}, adamw_rows=50257,
                    what="full Muon step, FP16 NS with Polar Express x8 (Gram-space for the 8192x2048 / 2048x8192 "
                         "matrices: gram_aspect_threshold 4.0, order 00100), 24 layers d=2048, the 50257x2048 "
                         "embedding on the fused AdamW companion, CUDA graphs")
    raise SystemExit(f"unknown --config {name}")


def config_flops(cfg):
    from i8muon_b200.sharding import ns_flops
    total = 0.0
    for shape in cfg["shapes"]:
        l, h = min(shape), max(shape)
        gram = cfg.get("gram") or shape in cfg.get("gram_shapes", ())
        total += gram_flops(l, h, cfg["steps"]) if gram else ns_flops(shape, cfg["steps"])
    return total


def run_other_config(args):
    """One of cfg1 / cfg2 / cfg2-gram / cfg3 / cfg5 through the drop-in optimizer on one GPU, or sharded by
    flops over N GPUs (cfg5 is stated at 1/2/4/8)."""
    import torch.distributed as dist
    from i8muon_b200 import CutlassNSInt8, FusedAdamW, Muon, check_status, native, recommend_coefficients
    from i8muon_b200.optimizer import native_step_ops
    from i8muon_b200.sharding import ShardedMuonStep
    cfg = other_config(args.config)
    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run for N > 1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        if args.reserve_sms > 0:
            os.environ.setdefault("NCCL_MAX_CTAS", str(args.reserve_sms))
        dist.init_process_group("nccl", device_id=dev)
    gen = torch.Generator(device=dev).manual_seed(1000)
    coeffs = recommend_coefficients(cfg["steps"], method=cfg["method"])

    def draw(shape, std, dtype, outliers=False):
        x = torch.randn(shape, device=dev, generator=gen) * std
        if outliers:
            x = x * torch.where(torch.rand(shape, device=dev, generator=gen) < 0.01, 50.0, 1.0)
        return x.to(dtype)
    params = [torch.nn.Parameter(draw(s, cfg["pstd"], cfg["pdtype"])) for s in cfg["shapes"]]
    grads = [draw(s, cfg["gstd"], cfg["gdtype"], cfg.get("outliers", False)) for s in cfg["shapes"]]
    muon_kw = dict(lr=LR, weight_decay=WD, momentum=MOMENTUM, adjust_lr_fn="match_rms_adamw")
    muon_kw.update(cfg["muon"])
    total_flops = config_flops(cfg)
    scalar = None
    if cfg.get("adamw_rows"):
        table = torch.nn.Parameter(draw((cfg["adamw_rows"], 2048), 0.02, cfg["pdtype"]))
        table.grad = draw(table.shape, 1e-3, cfg["pdtype"])
        scalar = FusedAdamW([table], lr=1e-3)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, count):
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(count):
            fn()
        end.record()
        barrier()
        ms = torch.tensor([start.elapsed_time(end)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item() / 1e3

    if world == 1:
        for p, g in zip(params, grads):
            p.grad = g
        opt = Muon(params, ns_coefficients=coeffs, use_cuda_graph=cfg["graph"], scalar_optimizer=scalar, **muon_kw)
        step = opt.step
        host = [torch.empty(g.shape, dtype=g.dtype).pin_memory().copy_(g) for g in grads]

        def e2e_step():
            for p, h in zip(params, host):
                p.grad.copy_(h, non_blocking=True)
            opt.step()
            result_host.copy_(params[0].float().norm().reshape(1), non_blocking=True)
    else:
        engine = CutlassNSInt8(fp16_first=bool(muon_kw.pop("fp16_first", True)))
        ops = native_step_ops(engine, ns_coefficients=coeffs, **{k: v for k, v in muon_kw.items()})
        plain = [p.data for p in params]
        stepper = ShardedMuonStep(plain, cfg["steps"], ops, adopt_parameters=bool(args.adopt), gather=args.gather)
        reserve_sms_if_collective(args, stepper, dev, world)
        buffers = {i: torch.zeros_like(grads[i]) for i in stepper.plan.owned(rank)}
        host = [torch.empty(g.shape, dtype=g.dtype).pin_memory().copy_(g) for g in grads]

        def step():
            stepper.step(plain, grads, buffers)
            if scalar is not None:
                scalar.step()

        def e2e_step():
            stepper.step(plain, grads, buffers, host_grads=host)
            if scalar is not None:
                scalar.step()
            result_host.copy_(plain[0].float().norm().reshape(1), non_blocking=True)
    result_host = torch.empty(1, dtype=torch.float32).pin_memory()
    for _ in range(max(args.warmup, 3)):
        step()
    check_status()
    sampler = ClockSampler(local) if rank == 0 else None
    before = native.launch_count()
    seconds = timed(step, args.steps)
    launches = native.launch_count() - before
    clocks = sampler.stop() if sampler else None
    e2e_step()
    e2e_seconds = timed(e2e_step, args.steps)
    check_status()
    if rank == 0:
        peaks, source = measured_peaks()
        bf16 = peaks["bf16_tflops_sustained"]
        peak = {"bf16": bf16, "int8": 2 * bf16, "tf32x3": bf16 / 2 / 3}[cfg["peak"]]
        value = total_flops * args.steps / seconds / 1e12
        h2d = sum(g.numel() * g.element_size() for g in grads)
        l2 = "flushed by the step itself: its tensors exceed L2" if h2d * 3 > 256e6 else \
             "the step's tensors (%.0f MB) fit in L2; no flush between steps, as in a training loop" % (h2d * 3 / 1e6)
        print(json.dumps({
            "metric": "muon_step_ns_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": seconds / args.steps * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": cfg["muon"]["precision"], "data": "synthetic",
            "config": {"workload": f"{args.config}: {cfg['what']}", "matrices": len(cfg["shapes"]),
                       "ns_steps": cfg["steps"], "api": "Muon(...).step()" if world == 1 else "ShardedMuonStep",
                       "cuda_graph": bool(cfg["graph"]) and world == 1, "l2": l2,
                       **({"gather": stepper.gather} if world > 1 else {})},
            "algorithmic_flops_per_step": total_flops,
            "roofline": {"bound": "tensor", "achieved": value / world, "peak": peak, "unit": "TFLOP/s",
                         "frac": value / world / peak, "traffic": None,
                         "kernel": "whole step (every kernel of the configuration), dense flop count",
                         "peak_source": {"bf16": "bf16_tflops_sustained", "int8": "2 x bf16_tflops_sustained (inferred: "
                                         "INT8 dense rate is twice BF16)", "tf32x3": "bf16_tflops_sustained / 2 (TF32 "
                                         "rate, inferred) / 3 (three TF32 products per FP32 product)"}[cfg["peak"]]
                                        + f" of MEASURED_PEAKS.json ({source})"},
            "e2e": {"value": total_flops * args.steps / e2e_seconds / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 4, "ms_per_step": e2e_seconds / args.steps * 1e3, "steps": args.steps},
            "gpu_launches": launches, "clocks": clocks}), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ----------------------------------------------------------------------------- GPU arm
def dominant_kernel_roofline(dev, peaks, source, b=4):
    """Time the INT8 block-quantised update GEMM alone on the gate/up shape."""
    from i8muon_b200 import native
    from i8muon_b200.engine import status_word
    lp, hp = 4096, 14336
    gen = torch.Generator(device=dev).manual_seed(5)
    pq = torch.randint(-127, 128, (b, lp, lp), device=dev, dtype=torch.int8, generator=gen)
    at = torch.randint(-127, 128, (b, hp, lp), device=dev, dtype=torch.int8, generator=gen)
    a = at.mT.contiguous()
    sp = torch.rand((b, lp // 128, lp // 128), device=dev, generator=gen) * 1e-3 + 1e-4
    sa = torch.rand((b, lp // 128, hp // 128), device=dev, generator=gen) * 1e-3 + 1e-4
    dp = torch.rand((b, lp), device=dev, generator=gen)
    y, yt = torch.empty_like(a), torch.empty_like(at)
    sy = torch.empty_like(sa)
    stream = torch.cuda.current_stream().cuda_stream

    def launch():
        native.call("i8m_bq_gemm", 0, 2, pq.data_ptr(), sp.data_ptr(), dp.data_ptr(), at.data_ptr(), sa.data_ptr(),
                    a.data_ptr(), y.data_ptr(), yt.data_ptr(), sy.data_ptr(), None, b, lp, hp, lp, lp, hp, 0.0, 0.0,
                    0.0, 0, 0, 0, status_word(dev).data_ptr(), stream)
    for _ in range(3):
        launch()
    n = 10
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(n):
        launch()
    end.record()
    torch.cuda.synchronize()
    seconds = start.elapsed_time(end) / 1e3 / n
    flops = 2.0 * lp * lp * hp * b
    achieved = flops / seconds / 1e12
    # the kernel is timed alone in a burst of ten launches (about 12 ms), so the burst figure is its
    # denominator; the sustained one is reported beside it because the whole step runs power-capped
    peak = 2.0 * peaks["bf16_tflops"]
    sustained = 2.0 * peaks["bf16_tflops_sustained"]
    return {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
            "frac_of_sustained_peak": achieved / sustained, "peak_sustained": sustained,
            "traffic": 222.5e6 * b, "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one B=1 "
            "launch (134.6 + 87.9 MB), scaled by the batch: every batch matrix is an independent set of tiles",
            "kernel": f"bq_split_kernel<EpiBq<int8, update>> B={b} 4096x14336 (k=4096)",
            "flops_per_launch": flops, "ms_per_launch": seconds * 1e3,
            "peak_source": f"2 x bf16_tflops (burst) of MEASURED_PEAKS.json ({source}); there is no measured INT8 "
                           "figure: the factor 2 is inferred from the INT8 : BF16 dense rate of the part"}


def fp16_first_iteration_gemm(dev, peaks, source, b=2, variant=0):
    """Time the FP16 update GEMM of the first iteration alone (gate/up shape, transposed BF16 result)."""
    from i8muon_b200 import native
    from i8muon_b200.engine import status_word
    native.call("i8m_set_variant", b"wholek_gemm", variant)
    lp, hp = 4096, 14336
    gen = torch.Generator(device=dev).manual_seed(6)
    q = (torch.randn((b, lp, lp), device=dev, generator=gen) * 0.05).half()
    at = (torch.randn((b, hp, lp), device=dev, generator=gen) * 0.05).half()
    out = torch.empty((b, hp, lp), device=dev, dtype=torch.bfloat16)
    stream = torch.cuda.current_stream().cuda_stream

    def launch():
        native.call("i8m_float_gemm", q.data_ptr(), None, at.data_ptr(), None, out.data_ptr(), None, None, None,
                    native.F16, 0, b, lp, hp, lp, lp, hp, 0, 1, 1, native.BF16, 0.0, 0.0, 0.0,
                    status_word(dev).data_ptr(), stream)
    for _ in range(3):
        launch()
    n = 10
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(n):
        launch()
    end.record()
    torch.cuda.synchronize()
    seconds = start.elapsed_time(end) / 1e3 / n
    flops = 2.0 * lp * lp * hp * b
    achieved = flops / seconds / 1e12
    peak = peaks["bf16_tflops_sustained"]
    return {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
            "kernel": f"{('wholek_wide_kernel', 'wholek_persistent_kernel', 'ns_gemm_kernel')[variant]}"
                      f"<EpiFloat<half, final>> B={b} 4096x14336 (k=4096), transposed bf16 result",
            "flops_per_launch": flops, "ms_per_launch": seconds * 1e3,
            "peak_source": f"bf16_tflops_sustained of MEASURED_PEAKS.json ({source})"}


def single_kernel(dev, peaks, source, name, b=1):
    """Time one GEMM kernel of the path alone (small cases for ncu): the block-quantised Gram and polynomial
    products on a 4096 x 14336 matrix, the global-INT8 update product at 4096 x 4096, the 3xTF32 Gram
    product of an FP32 1024 x 4096 matrix."""
    from i8muon_b200 import native
    from i8muon_b200.engine import status_word
    gen = torch.Generator(device=dev).manual_seed(11)
    stream = torch.cuda.current_stream().cuda_stream
    status = status_word(dev).data_ptr()
    keep = []

    def rand_i8(*shape):
        t = torch.randint(-127, 128, shape, device=dev, dtype=torch.int8, generator=gen)
        keep.append(t)
        return t

    def rand_f(*shape, lo=1e-4, span=1e-3):
        t = torch.rand(shape, device=dev, generator=gen) * span + lo
        keep.append(t)
        return t

    if name in ("bq_gram", "bq_poly"):
        lp, hp = 4096, 14336
        k = hp if name == "bq_gram" else lp
        a, sa = rand_i8(b, lp, k), rand_f(b, lp // 128, k // 128)
        da = rand_f(b, lp, lo=0.5, span=0.5)
        out = torch.empty((b, lp, lp), device=dev, dtype=torch.uint8)
        so, dout = torch.empty((b, lp // 128, lp // 128), device=dev), torch.empty((b, lp), device=dev)
        mode = 0 if name == "bq_gram" else 1

        def launch():
            native.call("i8m_bq_gemm", 0, mode, a.data_ptr(), sa.data_ptr(), da.data_ptr() if mode else None,
                        a.data_ptr(), sa.data_ptr(), None, out.data_ptr(), None, so.data_ptr(), dout.data_ptr(), b,
                        lp, lp, k, lp, lp, 3.0, -4.0, 2.0, 0, 0, 0, status, stream)
        tiles = (lp // 128) * (lp // 128 + 1) // 2
        flops = 2.0 * 128 * 128 * tiles * k * b
        peak, sustained = 2.0 * peaks["bf16_tflops"], 2.0 * peaks["bf16_tflops_sustained"]
        kernel = f"bq_split_kernel<EpiBq<int8, {'gram' if mode == 0 else 'polynomial'}>> B={b} 4096x4096 lower tiles (k={k})"
    elif name == "i8_update":
        lp = hp = 4096
        p8, at, a8 = rand_i8(b, lp, lp), rand_i8(b, hp, lp), rand_i8(b, lp, hp)
        ps, a_s, diag = rand_f(b), rand_f(b), rand_f(b, lp, lo=0.5, span=0.5)
        out, mx = torch.empty((b, lp, hp), device=dev), torch.zeros(b, device=dev)

        def launch():
            native.call("i8m_i8_gemm", 2, p8.data_ptr(), at.data_ptr(), a8.data_ptr(), out.data_ptr(), mx.data_ptr(),
                        ps.data_ptr(), a_s.data_ptr(), diag.data_ptr(), b, lp, hp, lp, lp, hp, 0.0, 0.0, 0, 0, 0,
                        status, stream)
        flops = 2.0 * lp * lp * hp * b
        peak, sustained = 2.0 * peaks["bf16_tflops"], 2.0 * peaks["bf16_tflops_sustained"]
        kernel = f"whole-K kernel<EpiI8<update>> B={b} 4096x4096 (k=4096), FP32 result + maximum"
    elif name in ("i8_gram", "i8_square"):
        lp = 4096
        a8 = rand_i8(b, lp, lp)
        if name == "i8_gram":
            out, mx = torch.empty((b, lp, lp), device=dev, dtype=torch.int32), torch.zeros(b, device=dev, dtype=torch.int32)

            def launch():
                native.call("i8m_i8_gemm", 0, a8.data_ptr(), a8.data_ptr(), None, out.data_ptr(), mx.data_ptr(), None,
                            None, None, b, lp, lp, lp, lp, lp, 0.0, 0.0, 0, 0, 0, status, stream)
        else:
            gs, dg = rand_f(b), rand_f(b, lp, lo=0.5, span=0.5)
            out, mx = torch.empty((b, lp, lp), device=dev), torch.zeros(b, device=dev)

            def launch():
                native.call("i8m_i8_gemm", 1, a8.data_ptr(), a8.data_ptr(), None, out.data_ptr(), mx.data_ptr(),
                            gs.data_ptr(), None, dg.data_ptr(), b, lp, lp, lp, lp, lp, -4.0, 2.0, 0, 0, 0, status, stream)
        tiles = (lp // 128) * (lp // 128 + 1) // 2
        flops = 2.0 * 128 * 128 * tiles * lp * b
        peak, sustained = 2.0 * peaks["bf16_tflops"], 2.0 * peaks["bf16_tflops_sustained"]
        kernel = f"wholek_wide_kernel<EpiI8<{'gram' if name == 'i8_gram' else 'square'}>> B={b} 4096x4096 lower tiles (k=4096)"
    elif name == "bq_final":
        lp, hp = 4096, 14336
        pq, at, a8 = rand_i8(b, lp, lp), rand_i8(b, hp, lp), rand_i8(b, lp, hp)
        sp, sa = rand_f(b, lp // 128, lp // 128), rand_f(b, lp // 128, hp // 128)
        dp = rand_f(b, lp, lo=0.5, span=0.5)
        out = torch.empty((b, hp, lp), device=dev, dtype=torch.bfloat16)

        def launch():
            native.call("i8m_bq_gemm", 0, 2, pq.data_ptr(), sp.data_ptr(), dp.data_ptr(), at.data_ptr(), sa.data_ptr(),
                        a8.data_ptr(), out.data_ptr(), None, None, None, b, lp, hp, lp, lp, hp, 0.0, 0.0, 0.0, 1, 1,
                        native.BF16, status, stream)
        flops = 2.0 * lp * lp * hp * b
        peak, sustained = 2.0 * peaks["bf16_tflops"], 2.0 * peaks["bf16_tflops_sustained"]
        kernel = f"bq_split_kernel<EpiBq<int8, final update>> B={b} 4096x14336 (k=4096), transposed bf16 result"
    elif name == "float_to_bq":
        lp, hp = 4096, 14336
        q = (torch.randn((b, lp, lp), device=dev, generator=gen) * 0.05).half()
        at = (torch.randn((b, hp, lp), device=dev, generator=gen) * 0.05).half()
        codes, codes_t = torch.empty((b, lp, hp), device=dev, dtype=torch.uint8), torch.empty((b, hp, lp), device=dev, dtype=torch.uint8)
        scale = torch.empty((b, lp // 128, hp // 128), device=dev)

        def launch():
            native.call("i8m_float_gemm_to_bq", q.data_ptr(), at.data_ptr(), codes.data_ptr(), codes_t.data_ptr(),
                        scale.data_ptr(), native.F16, native.BF16, b, lp, hp, lp, lp, hp, lp, hp, status, stream)
        flops = 2.0 * lp * lp * hp * b
        peak, sustained = peaks["bf16_tflops"], peaks["bf16_tflops_sustained"]
        kernel = f"wholek_wide_kernel<EpiFloatToBq<half>> B={b} 4096x14336 (k=4096), INT8 codes of A and A^T + block scales"
    elif name == "fp32_gram":
        lp, hp = 1024, 4096
        x = torch.randn((b, lp, hp), device=dev, generator=gen) * 0.02
        hi = (x.view(torch.int32) & ~0x1FFF).view(torch.float32).contiguous()
        lo = ((x - hi).view(torch.int32) & ~0x1FFF).view(torch.float32).contiguous()
        out, out_lo = torch.empty((b, lp, lp), device=dev), torch.empty((b, lp, lp), device=dev)

        def launch():
            native.call("i8m_float_gemm", hi.data_ptr(), lo.data_ptr(), hi.data_ptr(), lo.data_ptr(), out.data_ptr(),
                        None, out_lo.data_ptr(), None, native.F32, 0, b, lp, lp, hp, lp, lp, 1, 0, 0, 0, 0.0, 0.0,
                        0.0, status, stream)
        tiles = (lp // 128) * (lp // 128 + 1) // 2
        flops = 2.0 * 128 * 128 * tiles * hp * b
        # three TF32 products per FP32 product, TF32 at half the BF16 rate
        peak, sustained = peaks["bf16_tflops"] / 6.0, peaks["bf16_tflops_sustained"] / 6.0
        kernel = f"ns_gemm_kernel<EpiFloat<float, gram>> B={b} 1024x1024 lower tiles (k=4096), 3 x TF32"
    else:
        raise SystemExit(f"unknown kernel {name}")
    for _ in range(3):
        launch()
    n = 10
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(n):
        launch()
    end.record()
    torch.cuda.synchronize()
    if int(status_word(dev).item()) != 0:
        raise SystemExit("a kernel reported a timed-out wait")
    seconds = start.elapsed_time(end) / 1e3 / n
    achieved = flops / seconds / 1e12
    return {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
            "frac_of_sustained_peak": achieved / sustained, "kernel": kernel, "flops_per_launch": flops,
            "ms_per_launch": seconds * 1e3,
            "peak_source": f"from bf16_tflops (burst) of MEASURED_PEAKS.json ({source}); INT8 taken as 2 x BF16, "
                           "3xTF32 as BF16 / 6"}


def reserve_sms_if_collective(args, stepper, dev, world):
    """With the collective gather the GEMMs leave `--reserve-sms` SMs to NCCL; peer copies need none."""
    from i8muon_b200 import native
    if world > 1 and stepper.gather == "collective" and args.reserve_sms > 0:
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        native.call("i8m_set_cta_limit", sms - args.reserve_sms)


def run_native(args):
    import torch.distributed as dist
    from i8muon_b200 import CutlassNSInt8, check_status, native, recommend_coefficients
    from i8muon_b200.optimizer import native_step_ops
    from i8muon_b200.sharding import ShardedMuonStep

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run for N > 1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # The persistent GEMM kernels own every SM they run on, so the all-gather (an SM kernel) gets
        # SMs of its own: the GEMMs launch on all but `--reserve-sms` SMs and NCCL is held to as many CTAs.
        if args.reserve_sms > 0:
            os.environ.setdefault("NCCL_MAX_CTAS", str(args.reserve_sms))
        dist.init_process_group("nccl", device_id=dev)

    shape_list = shapes(args.layers)
    total_flops = ns_flops_of(shape_list)
    coeffs = recommend_coefficients(NS_STEPS)
    engine = CutlassNSInt8(fp16_first=bool(args.fp16_first))
    ops = native_step_ops(engine, lr=LR, weight_decay=WD, momentum=MOMENTUM, ns_coefficients=coeffs,
                          adjust_lr_fn="match_rms_adamw", precision=args.precision, use_gram=False)
    gen = torch.Generator(device=dev).manual_seed(4000)  # same seed on every rank: replicated tensors
    params = [(torch.randn(s, device=dev, generator=gen) * 0.02).bfloat16() for s in shape_list]
    grads = [(torch.randn(s, device=dev, generator=gen) * 1e-3).bfloat16() for s in shape_list]
    stepper = ShardedMuonStep(params, NS_STEPS, ops, max_group_bytes=args.group_bytes,
                              adopt_parameters=bool(args.adopt), gather=args.gather)
    reserve_sms_if_collective(args, stepper, dev, world)
    buffers = {i: torch.zeros_like(grads[i]) for i in stepper.plan.owned(rank)}

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    host_issue = {}

    def timed(fn, count):
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        began = time.perf_counter()
        for _ in range(count):
            fn()
        host_issue["ms_per_step"] = (time.perf_counter() - began) / count * 1e3   # host time to queue a step
        end.record()
        barrier()
        ms = torch.tensor([start.elapsed_time(end)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item() / 1e3

    step = lambda: stepper.step(params, grads, buffers)  # noqa: E731
    for _ in range(args.warmup):
        step()
    check_status()
    sampler = ClockSampler(local) if rank == 0 else None
    launches_before = native.launch_count()
    seconds = timed(step, args.steps)
    issue_ms = host_issue["ms_per_step"]
    launches = native.launch_count() - launches_before
    clocks = sampler.stop() if sampler else None
    check_status()
    phase_table = None
    if args.phases:
        # one more step with a pair of CUDA events around every phase of every chunk (max over ranks)
        marks = []
        barrier()
        stepper.step(params, grads, buffers, phases=marks)
        totals, _ = ShardedMuonStep.phase_milliseconds(marks)
        names = sorted(totals)
        values = torch.tensor([totals[n] for n in names], device=dev)
        if world > 1:
            dist.all_reduce(values, op=dist.ReduceOp.MAX)
        phase_table = {n: round(v, 3) for n, v in zip(names, values.tolist())}

    # end to end: this step's gradients arrive from pinned host memory, a scalar comes back
    pinned = torch.empty(256 << 20, dtype=torch.bfloat16).pin_memory()
    pinned.normal_(0, 1e-3)
    result_host = torch.empty(1, dtype=torch.float32).pin_memory()
    h2d = sum(g.numel() * g.element_size() for g in grads)  # every matrix is copied by the one rank that owns it

    # every gradient's host source is a view of the same pinned region (14 GB are copied per step,
    # 512 MB are pinned); the step streams them in, chunk by chunk, under the kernels
    host_grads = [pinned[:g.numel()].view(g.shape) for g in grads]

    def e2e_step():
        stepper.step(params, grads, buffers, host_grads=host_grads)
        result_host.copy_(params[0].float().norm().reshape(1), non_blocking=True)
    e2e_steps = args.steps          # steady state: one untimed step fills the copy pipeline first
    e2e_step()
    e2e_seconds = timed(e2e_step, e2e_steps)
    check_status()

    launch_total = torch.tensor([float(launches)], device=dev)
    if world > 1:
        dist.all_reduce(launch_total)
    peaks, source = measured_peaks()
    roofline = dominant_kernel_roofline(dev, peaks, source) if rank == 0 else None
    drop_in = None
    if world == 1 and not args.no_drop_in:
        # the same step through the drop-in optimizer object, with its CUDA graphs
        del stepper, buffers
        from i8muon_b200 import Muon
        wrapped = [torch.nn.Parameter(p) for p in params]
        for p, g in zip(wrapped, grads):
            p.grad = g
        opt = Muon(wrapped, lr=LR, weight_decay=WD, momentum=MOMENTUM, ns_coefficients=coeffs,
                   adjust_lr_fn="match_rms_adamw", precision=args.precision, fp16_first=bool(args.fp16_first),
                   use_gram=False, use_cuda_graph=True)
        for _ in range(3):
            opt.step()
        check_status()
        before = native.launch_count()
        api_seconds = timed(opt.step, args.steps)
        check_status()
        drop_in = {"api": "Muon(params, precision=..., use_cuda_graph=True).step()",
                   "value": total_flops * args.steps / api_seconds / 1e12, "unit": "TFLOP/s",
                   "ms_per_step": api_seconds / args.steps * 1e3, "captured_graphs": len(opt._ns_graphs),
                   "launches_outside_graphs": native.launch_count() - before}
        del opt, wrapped
    cpu = time_cpu(1, 0) if (rank == 0 and world == 1 and not args.no_cpu) else None
    ref_gpu = reference_gpu_leg(args) if (rank == 0 and world == 1 and not args.no_reference_gpu) else None
    if rank == 0:
        value = total_flops * args.steps / seconds / 1e12
        line = {"metric": "muon_step_ns_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds / args.steps * 1e3,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "s8",
                "data": "synthetic", "config": config_dict(world, args.layers, args.precision, bool(args.fp16_first)),
                "algorithmic_flops_per_step": total_flops,
                "frac_of_int8_peak": value / world / (2.0 * peaks["bf16_tflops_sustained"]),
                "e2e": {"value": total_flops * e2e_steps / e2e_seconds / 1e12, "unit": "TFLOP/s",
                        "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                        "ms_per_step": e2e_seconds / e2e_steps * 1e3, "steps": e2e_steps},
                "gpu_launches": int(launch_total.item()), "clocks": clocks, "roofline": roofline}
        if cpu is not None:
            line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
        if phase_table is not None:
            line["phase_ms_max_over_ranks"] = phase_table
        line["host_issue_ms_per_step"] = issue_ms
        if world > 1:
            line["config"]["gather"] = stepper.gather
            line["config"]["reserve_sms"] = args.reserve_sms if stepper.gather == "collective" else 0
            line["config"]["adopted_parameters"] = bool(args.adopt)
        if drop_in is not None:
            line["drop_in_api"] = drop_in
        if ref_gpu is not None:
            line["reference_gpu"] = ref_gpu
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=3)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=("native", "reference", "reference-gpu"), default="native")
    parser.add_argument("--config", default="cfg4-int8bq",
                        choices=("cfg4-int8bq", "cfg4-fp8bq", "cfg1", "cfg2", "cfg2-gram", "cfg3", "cfg5"))
    parser.add_argument("--precision", default="int8_bq")
    parser.add_argument("--fp16-first", type=int, default=1)
    parser.add_argument("--layers", type=int, default=32, help="layers of the parameter set (32 = the full set)")
    parser.add_argument("--group-bytes", type=int, default=2 << 30)
    parser.add_argument("--reserve-sms", type=int, default=16,
                        help="N > 1: SMs left to the all-gather (the GEMMs launch on the others)")
    parser.add_argument("--gather", choices=("auto", "copy", "collective"), default="auto",
                        help="N > 1: how updated parameters reach the other ranks (peer copies over CUDA IPC, "
                             "or NCCL all-gather on reserved SMs; auto = copies when IPC works)")
    parser.add_argument("--adopt", type=int, default=1,
                        help="N > 1: parameters live in the all-gather buffers and only their owner updates them")
    parser.add_argument("--phases", action="store_true", help="add per-phase device times of one step to the line")
    parser.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    parser.add_argument("--no-drop-in", action="store_true", help="skip the Muon(...).step() leg")
    parser.add_argument("--no-reference-gpu", action="store_true",
                        help="skip timing the reference's own kernels on this GPU (oracle/_ref, when present)")
    parser.add_argument("--only-fp16", type=int, default=0, metavar="B",
                        help="only time the FP16 first-iteration update GEMM on B matrices (small case for ncu)")
    parser.add_argument("--only-roofline", type=int, default=0, metavar="B",
                        help="only time the dominant GEMM on B matrices of 4096x14336 (small case for ncu)")
    parser.add_argument("--wholek-variant", type=int, default=0,
                        help="with --only-fp16: whole-K kernel (0 units of 128x256, 1 two streams of 128x128 tiles, "
                             "2 one CTA per tile)")
    parser.add_argument("--only-kernel", choices=("bq_gram", "bq_poly", "bq_final", "float_to_bq", "i8_gram", "i8_square", "i8_update", "fp32_gram"), default=None,
                        help="only time this GEMM kernel alone (small case for ncu); --kernel-batch matrices")
    parser.add_argument("--kernel-batch", type=int, default=1)
    args = parser.parse_args()
    if args.only_kernel:
        torch.cuda.set_device(0)
        peaks, source = measured_peaks()
        print(json.dumps(single_kernel(torch.device("cuda", 0), peaks, source, args.only_kernel, args.kernel_batch)))
        return
    if args.only_fp16:
        torch.cuda.set_device(0)
        peaks, source = measured_peaks()
        print(json.dumps(fp16_first_iteration_gemm(torch.device("cuda", 0), peaks, source, args.only_fp16,
                                                   args.wholek_variant)))
        return
    if args.only_roofline:
        torch.cuda.set_device(0)
        peaks, source = measured_peaks()
        print(json.dumps(dominant_kernel_roofline(torch.device("cuda", 0), peaks, source, args.only_roofline)))
        return
    if args.config == "cfg4-fp8bq":
        args.precision = "fp8_bq"
    if args.impl == "native" and not args.config.startswith("cfg4"):
        run_other_config(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.impl == "reference-gpu":
        run_reference_gpu(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
