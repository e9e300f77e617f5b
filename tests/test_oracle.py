"""The CPU oracle: internal consistency, mathematical anchors, and the pieces
that CAN be pinned to the reference's own code (its muon_step arithmetic)."""
import numpy as np
import pytest
import torch

from i8muon_b200 import recommend_coefficients
from oracle import ns_oracle as o

C5 = recommend_coefficients(5)


def rel(a, b):
    a, b = a.double(), b.double()
    return ((a - b).norm() / b.norm().clamp_min(1e-30)).item()


def sigma(y):
    s = torch.linalg.svdvals(y.double().reshape(-1, *y.shape[-2:]))
    return s.min().item(), s.max().item(), s.mean().item()


@pytest.fixture(scope="module")
def x():
    g = torch.Generator().manual_seed(7)
    return torch.randn(2, 128, 512, generator=g)


def test_fp32_oracle_equals_plain_torch_newton_schulz(x):
    # tolerance 1e-5: the FP32 bar stated for this path
    assert rel(o.ns_float(x, C5, precision="float32"), o.ns_fp32_torch(x, C5)) < 1e-5


def test_singular_value_anchors(x):
    # int8_safe x5 maps a Gaussian matrix into the band [0.823, 1.191]
    lo, hi, _ = sigma(o.ns_fp32_torch(x, C5))
    assert abs(lo - 0.823) < 5e-3 and abs(hi - 1.191) < 5e-3
    # Polar Express x8 converges to singular values of 1
    lo, hi, mean = sigma(o.ns_fp32_torch(x, recommend_coefficients(8, method="polar_express")))
    assert abs(lo - 1) < 2e-3 and abs(hi - 1) < 2e-3 and abs(mean - 1) < 1e-3


@pytest.mark.parametrize("name,fn,tol", [
    ("bf16", lambda x: o.ns_float(x.bfloat16(), C5, precision="bfloat16"), 2e-2),
    ("fp16", lambda x: o.ns_float(x.half(), C5, precision="float16"), 5e-3),
    ("gram", lambda x: o.ns_float(x.half(), C5, precision="float16", gram=True), 1e-2),
    ("int8", lambda x: o.ns_int8(x, C5, fp16_first=False), 5e-2),
    ("int8-fp16first", lambda x: o.ns_int8(x, C5, fp16_first=True), 5e-2),
    ("bq", lambda x: o.ns_bq(x, C5, fp16_first=False), 1.2e-1),
    ("bq-fp16first", lambda x: o.ns_bq(x, C5, fp16_first=True), 1.2e-1),
    ("fp8", lambda x: o.ns_bq(x, C5, fp8=True), 1.2e-1),
])
def test_every_path_orthogonalises(x, name, fn, tol):
    y = fn(x)
    truth = o.ns_fp32_torch(x, C5)
    assert y.shape == x.shape
    assert rel(y.float(), truth) < tol
    lo, hi, _ = sigma(y.float())
    assert 0.78 < lo and hi < 1.23


def test_shapes_transpose_and_batch_folding():
    g = torch.Generator().manual_seed(8)
    tall = torch.randn(3, 2, 200, 48, generator=g)
    for fn in (lambda v: o.ns_float(v, C5, precision="float32"), lambda v: o.ns_int8(v, C5),
               lambda v: o.ns_bq(v, C5)):
        y = fn(tall)
        assert y.shape == tall.shape
        # each batch entry is independent, and X -> NS(X) commutes with transposition
        single = fn(tall[1, 0].mT.contiguous())
        assert rel(single.mT.float(), y[1, 0].float()) < 1e-6
    zero = torch.zeros(1, 16, 32)
    assert o.ns_float(zero, C5, precision="float16").abs().max() == 0
    assert o.ns_bq(zero, C5).abs().max() == 0
    one_row = o.ns_float(tall[0], C5[:1], precision="float16")
    assert one_row.shape == tall[0].shape


def test_exact_integer_and_fma_helpers():
    rng = np.random.default_rng(0)
    a = rng.integers(-127, 128, (37, 300)).astype(np.int8)
    b = rng.integers(-127, 128, (21, 300)).astype(np.int8)
    assert np.array_equal(o.i8_gemm_nt(a, b), o.i8_gemm_nt_exact(a, b))
    assert np.array_equal(o.i8_gemm_nt(a, b), a.astype(np.int64) @ b.astype(np.int64).T)
    total = rng.standard_normal(1000).astype(np.float32)
    part = rng.integers(-2_000_000, 2_000_000, 1000).astype(np.float32)
    scale = (rng.standard_normal(1000) * 1e-6).astype(np.float32)
    expect = (part.astype(np.float64) * scale.astype(np.float64) + total.astype(np.float64))
    got = total.copy()
    o.fma_accumulate(got, part, scale)
    assert np.max(np.abs(got.astype(np.float64) - expect) / np.maximum(np.abs(expect), 1e-30)) < 6.1e-8


def test_quantisers():
    v = np.array([0.5, 1.5, 2.5, -0.5, -1.5, 126.6, 127.5, -300.0], dtype=np.float32)
    assert o.quant_rn(v, 1.0).tolist() == [0, 2, 2, 0, -2, 127, 127, -127]  # ties to even, clamp
    blk = np.zeros((128, 128), dtype=np.float32)
    blk[0, 0], blk[0, 1], blk[1, 0] = 2.0, -1.999, 0.0157
    q, s = o.bq_quantise_blocks(blk, fp8=False)
    assert q[0, 0] == 127 and q[0, 1] == -126 and q[1, 0] == 0  # truncation toward zero
    assert np.float32(1.0) / (np.float32(127.0) / np.float32(2.0)) == s[0, 0]
    q8, s8 = o.bq_quantise_blocks(blk, fp8=True)
    assert q8[0, 0] == 448 and s8.shape == (1, 1)
    assert o.e4m3_round(np.array([500.0, -1e9, 17.0, 0.003, 0.0009], dtype=np.float32)).tolist() == [448.0, -448.0, 16.0, 0.00390625, 0.0]


def test_step_arithmetic_matches_reference_muon_step(host_golden, step_golden):
    """momentum_update + apply_update reproduce the reference's muon_step bit for bit
    (fixtures were produced by running the reference's own Python on CPU tensors)."""
    for case in host_golden["muon_step_cases"]:
        key = case["key"]
        p = step_golden[key + ".param0"].clone()
        b = step_golden[key + ".buf0"].clone()
        for s in range(2):
            g = step_golden[f"{key}.grad{s}"]
            u = o.momentum_update(g, b, case["momentum"])
            u = (u.float() * 3.0).to(u.dtype)  # the fixtures' stand-in for Newton-Schulz
            o.apply_update(p, u, lr=case["lr"], adjusted_lr=o.adjust_lr(case["lr"], case["adjust"], p.shape),
                           weight_decay=case["wd"], weight_decay_mode=case["mode"])
            assert torch.equal(p, step_golden[f"{key}.param{s + 1}"]), key
            assert torch.equal(b, step_golden[f"{key}.buf{s + 1}"]), key


def test_adamw_restatement_follows_torch_adamw():
    """The AdamW statements used by the fused companion kernel, against torch.optim.AdamW on CPU."""
    g = torch.Generator().manual_seed(3)
    p0 = torch.randn(257, generator=g) * 0.1
    grads = [torch.randn(257, generator=g) * 0.01 for _ in range(5)]
    kw = dict(lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ref = p0.clone().requires_grad_()
    opt = torch.optim.AdamW([ref], foreach=False, **kw)
    p = p0.numpy().copy()
    m, v = np.zeros_like(p), np.zeros_like(p)
    for step, gr in enumerate(grads, 1):
        ref.grad = gr.clone()
        opt.step()
        p = o.adamw_update(p, gr.numpy(), m, v, step, **kw)
    np.testing.assert_allclose(p, ref.detach().numpy(), rtol=2e-6, atol=2e-8)
    np.testing.assert_allclose(m, opt.state[ref]["exp_avg"].numpy(), rtol=2e-6, atol=1e-10)


def test_factored_rows_and_grouped_cubics_restate_their_polynomials():
    """c((G + pI)^2 + qI) is the quintic (c(p^2 + q), 2cp, c): the two INT8 restatements agree to
    quantisation noise, and grouped cubics followed by a quintic track the same maps in FP32."""
    g = torch.Generator().manual_seed(1)
    x = torch.randn((1, 48, 80), generator=g)
    rows = [(c, b / (2 * c), a / c - (b / (2 * c)) ** 2) for a, b, c in C5[:2]]
    factored = o.ns_int8(x, rows, fp16_first=False, factored=True)
    plain = o.ns_int8(x, C5[:2], fp16_first=False)
    assert float((factored - plain).norm() / plain.norm()) < 2e-2
    first16 = o.ns_int8(x, rows, fp16_first=True, factored=True)
    assert float((first16 - plain).norm() / plain.norm()) < 5e-2
    abc = (3.4445, -4.775, 2.0315)
    cubic = o.ns_int8_grouped_cubic(x, 1.0, [1.5, 1.5], abc)
    t = x[0] / x[0].norm()
    eye = torch.eye(48)
    for gain in (1.5, 1.5):
        t = -gain * ((t @ t.mT) - eye) @ t
    gram = t @ t.mT
    t = (abc[0] * eye + abc[1] * gram + abc[2] * gram @ gram) @ t
    assert float((cubic[0] - t).norm() / t.norm()) < 3e-2
