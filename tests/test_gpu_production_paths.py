"""Bit-exact checks of the kernel paths that the benchmarked step actually runs.

The small stage tests give every persistent CTA at most one tile.  Here every launch has more tiles
than the GPU has SMs and several K blocks per tile, so the tile loops of ``bq_persistent_kernel``
(scale ring parity, the prefetched scale factors, buffer state carried across tiles, the
four-K-block fast path) and both tile streams of ``wholek_persistent_kernel`` run, and every integer
artefact is compared bit for bit with the CPU oracle on the same inputs, stage by stage, through the
C ABI.  The oracle's integer products go through float64 BLAS (exact), so these sizes take seconds.
"""
import numpy as np
import pytest
import torch

import gpu_helpers as H
from i8muon_b200 import CutlassNSInt8, recommend_coefficients
from oracle import ns_oracle as o

pytestmark = pytest.mark.gpu
C5 = recommend_coefficients(5)
C6 = recommend_coefficients(6)
PE8 = recommend_coefficients(8, method="polar_express")
F32 = np.float32


def npy(t):
    return t.detach().cpu().numpy()


def rel(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return ((a - b).norm() / b.norm()).item()


def seeded(shape, dtype, seed, std=1e-3, outliers=False):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g) * std
    if outliers:
        x = x * torch.where(torch.rand(shape, generator=g) < 0.01, 50.0, 1.0)
    return x.to(dtype)


def bq_iteration_bit_exact(dev, x, coeffs, fp8=False):
    """One block-quantised iteration, every stage against the oracle fed the same operands."""
    b, rows, cols = x.shape
    l, h, lp, hp, tr = H.geometry(rows, cols, 128)
    norm, _ = H.stats(x)
    a, at, sa = H.bq_quant(x, norm, fp8)
    gq, _, sg, dg = H.bq_gemm(fp8, 0, a, sa, a, sa, lm=l, ln=l)
    pq, _, sp, dp = H.bq_gemm(fp8, 1, gq, sg, gq, sg, da=dg, lm=l, ln=l, coeffs=coeffs)
    y, yt, sy, _ = H.bq_gemm(fp8, 2, pq, sp, at, sa, da=dp, row_b=a, lm=l, ln=h)
    yfin, *_ = H.bq_gemm(fp8, 2, pq, sp, at, sa, da=dp, row_b=a, lm=l, ln=h, final=True, transpose=bool(tr),
                         out_dtype=torch.float32)
    assert H.status_ok(dev) == 0
    for i in range(b):
        aq = npy(H.decode_q(a[i], fp8))
        w_gq, w_sg, w_dg = o.bq_gram(aq, npy(sa[i]), l, fp8)
        assert np.array_equal(npy(H.decode_q(gq[i], fp8)), w_gq), "gram codes"
        assert np.array_equal(npy(sg[i]), w_sg) and np.array_equal(npy(dg[i]), w_dg), "gram scales / diagonal"
        w_pq, w_sp, w_dp = o.bq_poly(w_gq, w_sg, w_dg, coeffs, l, fp8)
        assert np.array_equal(npy(H.decode_q(pq[i], fp8)), w_pq), "polynomial codes"
        assert np.array_equal(npy(sp[i]), w_sp) and np.array_equal(npy(dp[i]), w_dp), "polynomial scales / diagonal"
        w_y = o.bq_update(w_pq, w_sp, w_dp, aq, npy(sa[i]), l, h, fp8)
        w_next, w_snext = o.bq_quantise_blocks(w_y, fp8)
        assert np.array_equal(npy(H.decode_q(y[i], fp8)), w_next), "update codes"
        assert np.array_equal(npy(H.decode_q(yt[i], fp8)), w_next.T), "transposed update codes"
        assert np.array_equal(npy(sy[i]), w_snext), "update scales"
        want = w_y[:l, :h].T if tr else w_y[:l, :h]
        assert np.array_equal(npy(yfin[i]), want), "final FP32 tile"


@pytest.fixture(params=[0, 1, 2], ids=["split-tail", "fused-tail-6-stages", "fused-tail-4-stages"])
def bq_variant(request):
    """Every kernel variant of the block-quantised GEMMs that the tuner may choose."""
    from i8muon_b200 import native
    native.call("i8m_set_variant", b"bq_gemm", request.param)
    yield request.param
    native.call("i8m_set_variant", b"bq_gemm", 0)


@pytest.mark.parametrize("shape", [(1, 1536, 2048), (1, 2100, 1500), (2, 1024, 4096)],
                         ids=["1536x2048", "2100x1500-ragged-tall", "k-v-1024x4096-b2"])
def test_int8_bq_iteration_bit_exact_beyond_one_tile_per_cta(cuda_device, bq_variant, shape):
    """1536 x 2048: 192 update tiles on 148 CTAs, K = 1536 = 12 K blocks (tile loop it >= 1, scale ring
    parity, the (nkb & 3) == 0 fast path in the polynomial and the update).  2100 x 1500: rows > cols with
    ragged edges in both dimensions (lp = 1536, hp = 2176; the Gram runs K = 2176 = 17 K blocks, the
    general loop).  1024 x 4096 x 2: the k/v shape of the Llama-shaped set, two matrices."""
    x = seeded(shape, torch.bfloat16, 71).to(cuda_device)
    bq_iteration_bit_exact(cuda_device, x, C5[1])


def test_e4m3_bq_iteration_beyond_one_tile_per_cta(cuda_device, bq_variant):
    """E4M3 at 1536 x 2048 on every kernel variant: the variants must agree with each other bit for bit
    (same tensor-core instructions in the same order), and with the oracle within one E4M3 step on the
    few codes that sit on a rounding edge (the tensor core's accumulation order is its own)."""
    dev = cuda_device
    x = seeded((1, 1536, 2048), torch.bfloat16, 76).to(dev)
    norm, _ = H.stats(x)
    a, at, sa = H.bq_quant(x, norm, True)
    gq, _, sg, dg = H.bq_gemm(True, 0, a, sa, a, sa, lm=1536, ln=1536)
    pq, _, sp, dp = H.bq_gemm(True, 1, gq, sg, gq, sg, da=dg, lm=1536, ln=1536, coeffs=C5[1])
    y, yt, sy, _ = H.bq_gemm(True, 2, pq, sp, at, sa, da=dp, row_b=a, lm=1536, ln=2048)
    assert H.status_ok(dev) == 0
    got = [t.cpu() for t in (gq, sg, dg, pq, sp, dp, y, yt, sy)]
    if not hasattr(test_e4m3_bq_iteration_beyond_one_tile_per_cta, "first"):
        test_e4m3_bq_iteration_beyond_one_tile_per_cta.first = got
    for p, q in zip(test_e4m3_bq_iteration_beyond_one_tile_per_cta.first, got):
        assert torch.equal(p, q)
    w_gq, w_sg, w_dg = o.bq_gram(npy(H.decode_q(a[0], True)), npy(sa[0]), 1536, True)
    differ = npy(H.decode_q(gq[0], True)) != w_gq
    assert differ.mean() < 0.02 and np.allclose(npy(sg[0]), w_sg, rtol=2e-5) and np.allclose(npy(dg[0]), w_dg, rtol=2e-5)
    assert torch.equal(yt[0], y[0].mT)


def test_int8_bq_iteration_bit_exact_on_the_gate_projection_shape(cuda_device):
    """The benchmark's dominant shape at full K: 4096 x 14336, one matrix, one iteration (Gram K = 14336 =
    112 K blocks, 528 triangular tiles; update 3584 tiles of K = 4096)."""
    x = seeded((1, 4096, 14336), torch.bfloat16, 72).to(cuda_device)
    bq_iteration_bit_exact(cuda_device, x, C5[1])


def int8_iteration_bit_exact(dev, x, coeffs):
    b, rows, cols = x.shape
    l, h, lp, hp, tr = H.geometry(rows, cols, 16)
    norm, amax = H.stats(x)
    a8, a8t, a_scale = H.input_quant(x, amax, norm)
    ca, cb, cc = coeffs
    g32, gmax = H.i8_gemm(0, a8, a8, lm=l, ln=l)
    g8, g_scale, g_diag = H.symmetric_quant(g32, gmax, a_scale, None, False)
    p32, pmax = H.i8_gemm(1, g8, g8, a_scale=g_scale, diag=g_diag, lm=l, ln=l, alpha=cb, beta=cc)
    p8, p_scale, p_diag = H.symmetric_quant(p32, pmax, g_scale, g_diag, True, (ca, cb, cc))
    y, ymax = H.i8_gemm(2, p8, a8t, row_b=a8, a_scale=p_scale, b_scale=a_scale, diag=p_diag, lm=l, ln=h)
    n8, n8t, n_scale = H.output_quant(y, ymax)
    assert H.status_ok(dev) == 0
    blk = np.arange(lp) // 128
    lower = (blk[:, None] >= blk[None, :])[:l, :l]
    for i in range(b):
        a8_i = npy(a8[i, :l, :h])
        w_g32, w_gmax = o.i8_gram(a8_i)
        assert np.array_equal(npy(g32[i, :l, :l])[lower], w_g32[lower]) and int(gmax[i]) == w_gmax
        w_g8, w_gs, w_gd = o.i8_gram_quant(w_g32, w_gmax, npy(a_scale)[i])
        assert np.array_equal(npy(g8[i, :l, :l]), w_g8) and npy(g_scale)[i] == w_gs
        assert np.array_equal(npy(g_diag[i, :l]), w_gd)
        w_p32, w_pmax = o.i8_square(w_g8, w_gs, w_gd, cb, cc)
        assert np.array_equal(npy(p32[i, :l, :l])[lower], w_p32[lower]) and npy(pmax)[i] == w_pmax
        w_p8, w_ps, w_pd = o.i8_poly_quant(w_p32, w_pmax, w_gd, ca, cb, cc)
        assert np.array_equal(npy(p8[i, :l, :l]), w_p8) and npy(p_scale)[i] == w_ps
        assert np.array_equal(npy(p_diag[i, :l]), w_pd)
        w_y = o.i8_update(w_p8, w_ps, w_pd, a8_i, npy(a_scale)[i])
        assert np.array_equal(npy(y[i, :l, :h]), w_y)
        w_n8, w_ns, w_ymax = o.i8_output_quant(w_y)
        assert npy(ymax)[i] == w_ymax and npy(n_scale)[i] == w_ns
        assert np.array_equal(npy(n8[i, :l, :h]), w_n8) and np.array_equal(npy(n8t[i, :h, :l]), w_n8.T)


@pytest.mark.parametrize("shape", [(1, 2048, 2048), (1, 4096, 4096), (1, 3000, 1400)],
                         ids=["2048x2048", "4096x4096", "3000x1400-ragged-tall"])
def test_global_int8_iteration_bit_exact_beyond_one_tile_per_cta(cuda_device, shape):
    """2048^2: 136 Gram tiles and 256 update tiles through both streams of the whole-K persistent
    kernel; 4096^2 is the shape of the global-INT8 benchmark configuration (528 Gram tiles, 32 K
    blocks of 128); 3000 x 1400 has ragged edges and rows > cols."""
    x = seeded(shape, torch.float32, 73, outliers=True).to(cuda_device)
    int8_iteration_bit_exact(cuda_device, x, C6[1])


def test_fp16_gram_polar_express_on_the_2048x8192_shape(cuda_device, monkeypatch):
    """The FP16 Gram + Polar Express x8 configuration at its own shape.  With the alternating restart
    order the iteration is well conditioned and is held to 2e-2 of the oracle; with the default order
    00100 it is not (the reference's own kernel is 0.12 from the exact iteration on the recorded
    fixture), so there it is held to the oracle's distance from the exact FP32 iteration."""
    dev = cuda_device
    x = seeded((1, 2048, 8192), torch.bfloat16, 74)
    truth = o.ns_fp32_torch(x, PE8)
    engine = CutlassNSInt8()
    monkeypatch.setenv("I8MUON_GRAM_RESET", "01010101")
    y = engine._gram_prec(x.to(dev), PE8, 1e-7, True, "float16")
    norm, _ = H.stats(x.to(dev))
    want = o.ns_float(x, PE8, 1e-7, "float16", gram=True, order="01010101", norm=npy(norm))
    assert rel(y.float(), want.float()) <= 2e-2
    sv = torch.linalg.svdvals(y.float())
    assert 0.95 < sv.min().item() and sv.max().item() < 1.05
    monkeypatch.setenv("I8MUON_GRAM_RESET", "00100")
    y = engine._gram_prec(x.to(dev), PE8, 1e-7, True, "float16")
    want = o.ns_float(x, PE8, 1e-7, "float16", gram=True, order="00100", norm=npy(norm))
    assert H.status_ok(dev) == 0
    assert torch.isfinite(y).all()
    assert rel(y.float(), truth.float()) <= 1.5 * rel(want.float(), truth.float()) + 1e-2


def test_bf16_regular_on_the_768x3072_shape_with_more_tiles_than_sms(cuda_device):
    """B = 4 of 768 x 3072: 576 update tiles, so both tile streams of every CTA run several tiles."""
    dev = cuda_device
    x = seeded((4, 768, 3072), torch.bfloat16, 75, std=0.02)
    y = CutlassNSInt8()._regular_prec(x.to(dev), C5, 1e-7, True, "bfloat16")
    norm, _ = H.stats(x.to(dev))
    want = o.ns_float(x, C5, 1e-7, "bfloat16", norm=npy(norm))
    assert H.status_ok(dev) == 0
    assert rel(y.float(), want.float()) <= 2e-2
