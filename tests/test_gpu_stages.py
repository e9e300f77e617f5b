"""Stage-wise parity of the CUDA kernels against the CPU oracle, through the C ABI.

Integer artefacts (quantised operands, int32 accumulators, maxima, scales,
diagonals) must match bit for bit when the oracle is given the same inputs.
Floating tensor-core accumulations are compared with a stated tolerance.
Each case runs with the tensor-core path and, for the small shapes, with the
debug core that replaces TMA/tcgen05 by plain dot products.
"""
import numpy as np
import pytest
import torch

from i8muon_b200 import native, recommend_coefficients
from oracle import ns_oracle as o
import gpu_helpers as H

pytestmark = pytest.mark.gpu
C5 = recommend_coefficients(5)
F32 = np.float32


def npy(t):
    return t.detach().cpu().numpy()


@pytest.fixture(params=[0, 1], ids=["tensorcore", "debugcore"])
def core(request, cuda_device):
    native.call("i8m_set_debug_core", request.param)
    yield request.param
    native.call("i8m_set_debug_core", 0)
    assert H.status_ok(cuda_device) == 0


def make_input(shape, dtype, seed, outliers=False):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g) * 0.02
    if outliers:
        x = x * torch.where(torch.rand(shape, generator=g) < 0.01, 50.0, 1.0)
    return x.to(dtype)


# ------------------------------------------------------------------ passes
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_stats(cuda_device, dtype):
    x = make_input((3, 211, 517), dtype, 1, outliers=True).to(cuda_device)
    norm, amax = H.stats(x)
    ref = x.float().norm(dim=(1, 2))
    assert torch.allclose(norm, ref, rtol=2e-6, atol=0)        # FP32 summation order differs
    assert torch.equal(amax, x.float().abs().amax(dim=(1, 2)))   # a maximum is order independent
    zero = torch.zeros((2, 8, 8), device=cuda_device, dtype=dtype)
    norm, amax = H.stats(zero)
    assert norm.abs().max() == 0 and amax.abs().max() == 0


@pytest.mark.parametrize("shape", [(2, 48, 112), (2, 112, 48), (1, 37, 75), (1, 75, 37), (2, 200, 328), (1, 328, 200)])
@pytest.mark.parametrize("compute", [torch.float16, torch.bfloat16, torch.float32])
def test_normalize(cuda_device, shape, compute):
    # widths that are multiples of eight take the vectorised kernel (16-bit compute types),
    # the others and FP32 compute the scalar one
    x = make_input(shape, torch.float16 if shape[1] == 200 else torch.bfloat16, 2).to(cuda_device)
    norm, _ = H.stats(x)
    a, at, alo, atlo = H.normalize(x, norm, compute)
    inv = o._inv_norm(npy(norm), 1e-7)
    wide = o.to_wide(npy(x.float())) * inv[:, None, None]
    l, h = wide.shape[1:]
    got = a.float() + (alo if alo is not None else 0)
    got_t = at.float() + (atlo if atlo is not None else 0)
    ref = torch.zeros_like(got.cpu())
    ref[:, :l, :h] = torch.from_numpy(o.round_to(wide.astype(F32), str(compute)[6:]))
    if compute == torch.float32:
        # two TF32 planes carry 22 significant bits
        assert (got.cpu() - ref).abs().max() <= 2.0 ** -21 * ref.abs().max(), (got.cpu() - ref).abs().max()
        assert torch.equal(got_t.cpu(), got.cpu().mT)
        assert torch.equal(a.view(torch.int32) & 0x1fff, torch.zeros_like(a, dtype=torch.int32))
    else:
        assert torch.equal(got.cpu(), ref)
        assert torch.equal(got_t.cpu(), ref.mT)


@pytest.mark.parametrize("shape", [(2, 64, 160), (2, 160, 64), (1, 45, 91), (1, 91, 45)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_input_quant_bit_exact(cuda_device, shape, dtype):
    x = make_input(shape, dtype, 3, outliers=True).to(cuda_device)
    norm, amax = H.stats(x)
    a8, a8t, scale = H.input_quant(x, amax, norm)
    wide = o.to_wide(npy(x.float()))
    for b in range(shape[0]):
        ref8, ref_scale = o.input_quant(wide[b], npy(amax)[b], npy(norm)[b], 1e-7, True)
        l, h = ref8.shape
        assert np.array_equal(npy(a8[b, :l, :h]), ref8)
        assert np.array_equal(npy(a8t[b, :h, :l]), ref8.T)
        assert npy(scale)[b] == ref_scale
    pad = torch.cat([a8[:, l:].reshape(-1), a8[:, :, h:].reshape(-1), a8t[:, h:].reshape(-1)])
    assert pad.numel() == 0 or int(pad.abs().max()) == 0  # zero padding
    # without normalisation the scale is amax / 127
    _, _, scale1 = H.input_quant(x, amax, None)
    assert np.array_equal(npy(scale1), npy(amax) / F32(127.0))


# ------------------------------------------------------------------ global INT8 iteration
@pytest.mark.parametrize("l,h", [(144, 400), (48, 80), (257, 300)])
def test_int8_iteration_stagewise_bit_exact(cuda_device, core, l, h):
    if core == 1 and l > 200:
        pytest.skip("debug core only on small shapes")
    dev = cuda_device
    x = make_input((2, l, h), torch.float32, 4, outliers=True).to(dev)
    norm, amax = H.stats(x)
    a8, a8t, a_scale = H.input_quant(x, amax, norm)
    lp, hp = a8.shape[1:]
    ca, cb, cc = C5[0]
    g32, gmax = H.i8_gemm(0, a8, a8, lm=l, ln=l)
    g8, g_scale, g_diag = H.symmetric_quant(g32, gmax, a_scale, None, False)
    p32, pmax = H.i8_gemm(1, g8, g8, a_scale=g_scale, diag=g_diag, lm=l, ln=l, alpha=cb, beta=cc)
    p8, p_scale, p_diag = H.symmetric_quant(p32, pmax, g_scale, g_diag, True, (ca, cb, cc))
    y, ymax = H.i8_gemm(2, p8, a8t, row_b=a8, a_scale=p_scale, b_scale=a_scale, diag=p_diag, lm=l, ln=h)
    n8, n8t, n_scale = H.output_quant(y, ymax)
    yfin, _ = H.i8_gemm(2, p8, a8t, row_b=a8, a_scale=p_scale, b_scale=a_scale, diag=p_diag, lm=l, ln=h,
                        final=True, out_dtype=torch.bfloat16)
    assert H.status_ok(dev) == 0
    blk = np.arange(lp) // 128
    lower_tiles = blk[:, None] >= blk[None, :]
    for b in range(2):
        st = o.int8_iteration(npy(a8[b, :l, :h]), npy(a_scale)[b], C5[0], final=False)
        lt = lower_tiles[:l, :l]
        assert np.array_equal(npy(g32[b, :l, :l])[lt], st.g32[lt])
        assert int(gmax[b]) == st.gmax
        assert np.array_equal(npy(g8[b, :l, :l]), st.g8)
        assert npy(g_scale)[b] == st.g_scale
        assert np.array_equal(npy(g_diag[b, :l]), st.g_diag)
        assert np.array_equal(npy(p32[b, :l, :l])[lt], st.p32[lt])
        assert npy(pmax)[b] == st.pmax
        assert np.array_equal(npy(p8[b, :l, :l]), st.p8)
        assert npy(p_scale)[b] == st.p_scale
        assert np.array_equal(npy(p_diag[b, :l]), st.p_diag)
        assert np.array_equal(npy(y[b, :l, :h]), st.y)
        assert npy(ymax)[b] == st.ymax
        assert np.array_equal(npy(n8[b, :l, :h]), st.a8_next)
        assert np.array_equal(npy(n8t[b, :h, :l]), st.a8_next.T)
        assert npy(n_scale)[b] == st.a_scale_next
        assert torch.equal(yfin[b].cpu(), torch.from_numpy(st.y).to(torch.bfloat16))
    # padding of the symmetric operands stays zero
    assert lp == l or int(g8[:, l:].abs().max()) == 0


# ------------------------------------------------------------------ block-quantised iteration
@pytest.mark.parametrize("fp8", [False, True], ids=["int8", "e4m3"])
@pytest.mark.parametrize("shape,dtype", [((2, 144, 400), torch.bfloat16), ((1, 400, 144), torch.bfloat16),
                                         ((1, 256, 512), torch.float16), ((1, 130, 203), torch.bfloat16),
                                         ((1, 203, 130), torch.float16), ((1, 144, 400), torch.float32)])
def test_bq_quant_bit_exact(cuda_device, fp8, shape, dtype):
    """Rows of whole 16-byte vectors of a 16-bit type take the vectorised kernel, odd widths and
    FP32 inputs the scalar one; both must reproduce the oracle's codes, transposes and scales."""
    x = make_input(shape, dtype, 5, outliers=True).to(cuda_device)
    norm, _ = H.stats(x)
    a, at, sa = H.bq_quant(x, norm, fp8)
    inv = o._inv_norm(npy(norm), 1e-7)
    wide = o.to_wide(npy(x.float()))
    b, l, h = wide.shape
    lp, hp = a.shape[1:]
    for i in range(b):
        v = np.zeros((lp, hp), dtype=F32)
        v[:l, :h] = (wide[i] * inv[i]).astype(F32)
        q, s = o.bq_quantise_blocks(v, fp8)
        assert np.array_equal(npy(H.decode_q(a[i], fp8)), q)
        assert np.array_equal(npy(H.decode_q(at[i], fp8)), q.T)
        assert np.array_equal(npy(sa[i]), s)


@pytest.mark.parametrize("fp8", [False, True], ids=["int8", "e4m3"])
@pytest.mark.parametrize("l,h", [(144, 400), (256, 640)])
def test_bq_iteration_stagewise(cuda_device, core, fp8, l, h):
    if core == 1 and l > 200:
        pytest.skip("debug core only on small shapes")
    dev = cuda_device
    x = make_input((2, l, h), torch.bfloat16, 6).to(dev)
    norm, _ = H.stats(x)
    a, at, sa = H.bq_quant(x, norm, fp8)
    ca, cb, cc = C5[0]
    gq, _, sg, dg = H.bq_gemm(fp8, 0, a, sa, a, sa, lm=l, ln=l)
    pq, _, sp, dp = H.bq_gemm(fp8, 1, gq, sg, gq, sg, da=dg, lm=l, ln=l, coeffs=(ca, cb, cc))
    y, yt, sy, _ = H.bq_gemm(fp8, 2, pq, sp, at, sa, da=dp, row_b=a, lm=l, ln=h)
    yfin, *_ = H.bq_gemm(fp8, 2, pq, sp, at, sa, da=dp, row_b=a, lm=l, ln=h, final=True,
                         out_dtype=torch.float32)
    assert H.status_ok(dev) == 0
    for b in range(2):
        st = o.bq_iteration(npy(H.decode_q(a[b], fp8)), npy(sa[b]), C5[0], l, h, fp8, final=False)
        got = dict(gq=npy(H.decode_q(gq[b], fp8)), sg=npy(sg[b]), dg=npy(dg[b]),
                   pq=npy(H.decode_q(pq[b], fp8)), sp=npy(sp[b]), dp=npy(dp[b]),
                   y=npy(yfin[b]), aq_next=npy(H.decode_q(y[b], fp8)), sa_next=npy(sy[b]))
        assert np.array_equal(npy(H.decode_q(yt[b], fp8)), got["aq_next"].T)
        if not fp8:
            # int32 partials are exact and the promotion order is fixed: everything is bit-exact
            for key, value in got.items():
                ref = getattr(st, key)
                ref = ref[:l, :h] if key == "y" else ref
                assert np.array_equal(value, ref), key
        else:
            # E4M3 partials are accumulated inside the tensor core in an unspecified
            # order: scales and diagonals to 1e-5 relative, dequantised tiles to one
            # E4M3 step (2^-3 relative) on the few entries that sit on a rounding edge.
            for key in ("sg", "dg", "sp", "dp", "sa_next"):
                assert np.allclose(got[key], getattr(st, key), rtol=2e-5, atol=1e-9), key
            for key, scale_key in (("gq", "sg"), ("pq", "sp"), ("aq_next", "sa_next")):
                ref = getattr(st, key)
                differ = got[key] != ref
                assert differ.mean() < 0.02, key
                assert np.all(np.abs(got[key] - ref)[differ] <= 0.126 * np.abs(ref)[differ] + 2 ** -9), key
            assert np.allclose(got["y"], st.y[:l, :h], rtol=1e-4, atol=1e-6)


# ------------------------------------------------------------------ floating GEMM modes
@pytest.mark.parametrize("dtype,tol", [(torch.float16, 2 ** -10), (torch.bfloat16, 2 ** -7), (torch.float32, 4e-6)])
def test_float_gemm_modes(cuda_device, core, dtype, tol):
    dev = cuda_device
    g = torch.Generator().manual_seed(9)
    b, m, n, k, l = 2, 208, 336, 176, 200
    if core == 1 and dtype == torch.float32:
        pytest.skip("the debug core multiplies only the high TF32 plane")

    def planes(t):
        if dtype != torch.float32:
            return t.to(dtype).to(dev), None
        t = t.to(dev)
        hi = (t.view(torch.int32) + 0xfff + ((t.view(torch.int32) >> 13) & 1) & ~0x1fff).view(torch.float32)
        lo = t - hi
        lo = (lo.view(torch.int32) + 0xfff + ((lo.view(torch.int32) >> 13) & 1) & ~0x1fff).view(torch.float32)
        return hi, lo

    a_full = torch.randn(b, m, k, generator=g) * 0.3
    a_full[:, l:] = 0
    bt_full = torch.randn(b, n, k, generator=g) * 0.3
    a, a_lo = planes(a_full)
    bt, bt_lo = planes(bt_full)
    av = (a + (a_lo if a_lo is not None else 0)).double()
    bv = (bt + (bt_lo if bt_lo is not None else 0)).double()

    def close(got, ref):
        # relative to the entry, with a floor of the typical entry for sums that cancel
        got, ref = got.double().cpu(), ref.double().cpu()
        return bool(((got - ref).abs() <= tol * (ref.abs() + ref.abs().mean())).all())

    # plain, with transposed copy
    out, out_t, lo, lo_t = H.float_gemm(a, bt, lm=l, ln=n, want_t=True, left_lo=a_lo, right_lo=bt_lo)
    ref = av @ bv.mT
    ref[:, l:] = 0
    assert close(out.float() + (lo if lo is not None else 0), ref)
    assert close(out_t.float() + (lo_t if lo_t is not None else 0), ref.mT)
    # symmetric Gram with mirror
    gram, _, glo, _ = H.float_gemm(a, a, sym=True, lm=l, ln=l, left_lo=a_lo, right_lo=a_lo)
    gv = gram.float() + (glo if glo is not None else 0)
    assert close(gv, av @ av.mT)
    assert torch.equal(gv, gv.mT.contiguous())
    # polynomial epilogue on the symmetric operand
    ca, cb, cc = C5[1]
    poly, _, plo, _ = H.float_gemm(gram, gram, mode=1, sym=True, lm=l, ln=l, coeffs=(ca, cb, cc), left_lo=glo,
                                   right_lo=glo)
    gd = gv.double()
    refp = cb * gd + cc * (gd @ gd.mT) + ca * torch.eye(m, device=dev, dtype=torch.double)
    refp[:, l:] = 0
    refp[:, :, l:] = 0
    pv = poly.float() + (plo if plo is not None else 0)
    assert bool(((pv.double() - refp).abs() <= 4 * tol * (cb * gd).abs() + 4 * tol * (cc * (gd @ gd.mT)).abs() + 1e-5).all())
    # final stores: un-padded, both orientations, all user dtypes
    for out_dtype in (torch.float32, torch.float16, torch.bfloat16):
        for tr in (False, True):
            fin, *_ = H.float_gemm(a, bt, final=True, transpose=tr, out_dtype=out_dtype, lm=l, ln=n - 5,
                                   left_lo=a_lo, right_lo=bt_lo)
            want = (av @ bv.mT)[:, :l, :n - 5]
            want = want.mT if tr else want
            step = max(tol, {torch.float32: 0, torch.float16: 2 ** -10, torch.bfloat16: 2 ** -7}[out_dtype])
            assert bool(((fin.double() - want).abs() <= 2 * step * want.abs() + 1e-6).all())


# ------------------------------------------------------------------ bounded waits
@pytest.mark.parametrize("variant", [0, 1], ids=["split-tail", "fused-tail"])
def test_bounded_waits_run_out_and_report_when_the_producer_issues_nothing(cuda_device, variant):
    """The failure path of the block-quantised GEMM kernels, made on purpose in the one way that leaves nothing in
    flight: a host-set flag lets the producers return without issuing a copy (one tile, one CTA).  The issuers'
    wait for operands runs out after its two-second limit, sets the abort flag, the fold and tail warps leave at
    their next poll, tensor memory is freed, and the status word holds a timeout code.  The same launch without
    the flag is then correct, on the same context."""
    dev = cuda_device
    x = make_input((1, 128, 256), torch.bfloat16, 8).to(dev)
    norm, _ = H.stats(x)
    a, at, sa = H.bq_quant(x, norm, False)
    native.call("i8m_set_variant", b"bq_gemm", variant)
    try:
        want = H.bq_gemm(False, 0, a, sa, a, sa, lm=128, ln=128)
        assert H.status_ok(dev) == 0
        native.call("i8m_set_debug_core", 2)
        H.bq_gemm(False, 0, a, sa, a, sa, lm=128, ln=128)
        code = H.status_ok(dev)            # synchronises: about two seconds
        assert code & 0xf00 in (0x100, 0x200, 0x300, 0x400) and code != 0
        native.call("i8m_set_debug_core", 0)
        again = H.bq_gemm(False, 0, a, sa, a, sa, lm=128, ln=128)
        assert H.status_ok(dev) == 0
        for p, q in zip(want, again):
            if isinstance(p, torch.Tensor):
                assert torch.equal(p, q)
    finally:
        native.call("i8m_set_debug_core", 0)
        native.call("i8m_set_variant", b"bq_gemm", 0)


def shifted(t):
    """The same values at an address that is 4 bytes past a 16-byte boundary: the library then takes its
    general kernels (32 x 32 tiles, scalar accesses) instead of the vectorised ones."""
    flat = torch.empty(t.numel() + 4, dtype=t.dtype, device=t.device)
    view = flat[1:1 + t.numel()].view(t.shape)
    view.copy_(t)
    assert view.data_ptr() % 16 != 0
    return view


@pytest.mark.parametrize("b,m,n", [(2, 256, 384), (1, 384, 256), (1, 128, 128)])
def test_tiled_requantisers_match_the_general_kernels_bit_for_bit(cuda_device, b, m, n):
    """The 128 x 128-tile kernels of the global-INT8 route (input, symmetric and output quantisers) against the
    general kernels on the same values: codes, transposed / mirrored codes, scales and diagonals are identical."""
    dev = cuda_device
    g = torch.Generator().manual_seed(41)
    # output quantiser: FP32 (m x n) -> int8, int8^T, scale
    y = (torch.randn((b, m, n), generator=g) * 3).to(dev)
    mx = y.abs().amax(dim=(1, 2)).contiguous()
    fast, slow = H.output_quant(y, mx), H.output_quant(shifted(y), mx)
    for p, q in zip(fast, slow):
        assert torch.equal(p, q)
    # input quantiser: x -> int8, int8^T, scale (with and without the norm in the scale)
    x = make_input((b, m, n), torch.float32, 42, outliers=True).to(dev)
    norm, amax = H.stats(x)
    for nrm in (norm, None):
        fast, slow = H.input_quant(x, amax, nrm), H.input_quant(shifted(x), amax, nrm)
        for p, q in zip(fast, slow):
            assert torch.equal(p, q)
    # symmetric quantisers: int32 Gram (lower tiles valid) and FP32 polynomial with its diagonal formula
    gram = torch.randint(-90000, 90000, (b, m, m), generator=g, dtype=torch.int32)
    gram = torch.tril(gram) + torch.tril(gram, -1).transpose(1, 2)
    gram = gram.to(dev)
    off = gram.clone()
    off.diagonal(dim1=1, dim2=2).zero_()
    gmax = off.abs().amax(dim=(1, 2)).to(torch.int32).contiguous()
    scale = torch.rand(b, generator=g).to(dev) * 1e-3 + 1e-4
    fast, slow = H.symmetric_quant(gram, gmax, scale, None, 0), H.symmetric_quant(shifted(gram), gmax, scale, None, 0)
    for p, q in zip(fast, slow):
        assert torch.equal(p, q)
    poly = torch.tril(torch.randn((b, m, m), generator=g)).to(dev)       # only the lower tiles are read
    pmax = poly.abs().amax(dim=(1, 2)).contiguous()
    diag = torch.rand((b, m), generator=g).to(dev)
    coeffs = (0.7, -1.3, 0.4)
    fast = H.symmetric_quant(poly, pmax, scale, diag, 1, coeffs)
    slow = H.symmetric_quant(shifted(poly), pmax, scale, diag, 1, coeffs)
    for p, q in zip(fast, slow):
        assert torch.equal(p, q)


def test_bounded_waits_of_the_whole_k_kernel_run_out_and_report(cuda_device):
    """The same failure path in the whole-K kernel (128 x 256 units): with the producer issuing nothing, the
    issuer's wait for operands runs out, the epilogue warps leave at their next poll, tensor memory is freed and
    the status word holds a timeout code; the next launch on the same context is correct."""
    dev = cuda_device
    a = (make_input((1, 128, 256), torch.float32, 9) * 50).half().to(dev)
    try:
        want = H.float_gemm(a, a)[0]
        assert H.status_ok(dev) == 0
        native.call("i8m_set_debug_core", 2)
        H.float_gemm(a, a)
        code = H.status_ok(dev)            # synchronises: about two seconds
        assert code & 0xf00 in (0x100, 0x200, 0x300) and code != 0
        native.call("i8m_set_debug_core", 0)
        again = H.float_gemm(a, a)[0]
        assert H.status_ok(dev) == 0
        assert torch.equal(want, again) and torch.isfinite(again).all()
    finally:
        native.call("i8m_set_debug_core", 0)


# ------------------------------------------------------------------ fused first row of an fp16-first call
@pytest.mark.parametrize("b,l,h", [(2, 144, 400), (1, 200, 330), (1, 1536, 2048)])
@pytest.mark.parametrize("user", [torch.bfloat16, torch.float16, torch.float32])
def test_float_update_that_quantises_its_own_result_matches_the_two_kernel_sequence(cuda_device, b, l, h, user):
    """``i8m_float_gemm_to_bq`` (the FP16 first row's update product whose epilogue is the block quantiser)
    against the sequence it replaces: the floating route's final store in the caller's dtype followed by the
    standalone quantisation pass without normalisation.  Codes, transposed codes and scales are bit-identical."""
    dev = cuda_device
    g = torch.Generator().manual_seed(12)
    lp16, hp16 = -(-l // 16) * 16, -(-h // 16) * 16
    lp, hp = -(-l // 128) * 128, -(-h // 128) * 128
    q0 = torch.zeros((b, lp16, lp16), dtype=torch.float16)
    q0[:, :l, :l] = (torch.randn((b, l, l), generator=g) * 0.05).half()
    at = torch.zeros((b, hp16, lp16), dtype=torch.float16)
    at[:, :h, :l] = (torch.randn((b, h, l), generator=g) * 0.05).half()
    q0, at = q0.to(dev), at.to(dev)
    first, *_ = H.float_gemm(q0, at, final=True, transpose=False, out_dtype=user, lm=l, ln=h)   # (b, l, h)
    want_a, want_at, want_sa = H.bq_quant(first, None, False)
    a = torch.full((b, lp, hp), 77, device=dev, dtype=torch.uint8)
    a_t = torch.full((b, hp, lp), 77, device=dev, dtype=torch.uint8)
    sa = torch.empty((b, lp // 128, hp // 128), device=dev)
    native.call("i8m_float_gemm_to_bq", q0.data_ptr(), at.data_ptr(), a.data_ptr(), a_t.data_ptr(), sa.data_ptr(),
                native.F16, H.DT[user], b, lp16, hp16, lp16, l, h, lp, hp, H.status_word(dev).data_ptr(), H._stream())
    assert H.status_ok(dev) == 0
    assert torch.equal(a, want_a) and torch.equal(a_t, want_at) and torch.equal(sa, want_sa)
