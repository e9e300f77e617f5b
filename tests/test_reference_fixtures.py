"""The CPU oracle against tensors recorded from the REFERENCE'S OWN CUDA KERNELS (CPU test).

``tests/golden/reference_ns_*.npz`` were written on a B200 by ``tests/golden/make_ns_golden.py``:
the reference (i8muon 0.2.0), imported unmodified, its ``csrc/{int8,prec,bq}.cu`` built for sm_100a,
ran on seeded inputs while every native call of its drivers was recorded.  Each stage of the oracle is
fed the reference's own inputs of that stage ("teacher forcing"), so one differing element cannot
cascade, and must reproduce the reference's outputs of that stage:

  * global INT8 (int8.cu): input quantisation, int32 Gram and its integer maximum, the int8 Gram /
    scale / FP32 diagonal, the polynomial's int8 operand / scale / diagonal, the FP32 update, its maximum
    and the re-quantised operands: bit for bit.  The FP32 polynomial tile P32 is the one place where
    the reference's binary is not one formula (two contraction variants, 1 ulp apart, by unrolled
    instance): every element must equal one of the two, and the share of the canonical one is reported.
  * block-quantised INT8 (bq.cu): every quantised operand, block scale, diagonal and the final
    result: bit for bit.  E4M3: codes, scales and the result bit for bit on these fixtures; the FP32
    diagonals (raw tensor-core sums of another accumulation order) to 1e-5 relative.
  * floating routes (prec.cu): the result within 1e-5 (FP32) / 2e-2 (BF16, FP16) relative Frobenius.
"""
import numpy as np
import pytest
import torch

import ref_fixtures as rf
from oracle import ns_oracle as o

F32 = np.float32
Q = 128


def rel(a, b):
    a, b = a.double(), b.double()
    return ((a - b).norm() / b.norm()).item()


def npy(t):
    if t is None:
        return None
    if t.dtype in (torch.float8_e4m3fn, torch.bfloat16, torch.float16):
        return t.float().numpy()      # exact widening
    return t.numpy()


def test_fixture_set_is_complete():
    expected = {"i8_staged_wide", "i8_staged_tall", "bq_int8_staged", "bq_int8_staged_tall", "bq_fp8_staged",
                "float_regular_float32", "float_regular_bfloat16", "float_regular_float16",
                "gram_bf16_00100", "gram_fp16_pe8_default", "i8_fp16first", "bq_int8_fp16first"}
    assert expected <= set(rf.names())


# ------------------------------------------------------------------------------------------- global INT8
@pytest.mark.parametrize("name", ["i8_staged_wide", "i8_staged_tall"])
def test_int8_stages_match_the_reference_kernels(name):
    case = rf.Case(name)
    x = case.x
    xw = o.to_wide(o.fold(x).float().numpy())
    batch, l, h = xw.shape
    canonical = other = 0
    seen = {op: 0 for op in ("stats", "input_quant", "aat", "symmetric_quant", "square", "update", "output_quant")}
    final_seen = False
    for call in case.calls:
        op, a = call["op"], [npy(t) if isinstance(t, torch.Tensor) else t for t in case.args(call)]
        seen[op] += 1
        if op == "stats":
            assert np.array_equal(a[1][0], np.abs(xw).reshape(batch, -1).max(1))
        elif op == "input_quant":
            _, maxima, norm, a8, a8t, a_scale = a[:6]
            # the norm the reference fed its quantiser (torch's CUDA reduction) is part of the fixture
            assert np.allclose(norm, o.frobenius_norm(x), rtol=2e-6, atol=0)
            for b in range(batch):
                want8, want_scale = o.input_quant(xw[b], maxima[0][b], norm[b], a[8], True)
                assert np.array_equal(a8[b, :l, :h], want8) and np.array_equal(a8t[b, :h, :l], want8.T)
                assert a_scale[b] == want_scale
        elif op == "aat":
            a8, g32, maxima, lm, _, slot = a
            blk = np.arange(a8.shape[1]) // 128
            computed = blk[:, None] >= blk[None, :]          # the reference fills lower 128-tiles only
            for b in range(batch):
                want, gmax = o.i8_gram(a8[b, :lm])
                assert np.array_equal(g32[b][computed], want[computed])
                assert int(maxima[slot].view(np.int32)[b]) == gmax
        elif op == "symmetric_quant":
            inp, maxima, oscale, odiag, out8, scale, diag, quad, c0, c1, c2, slot = a
            for b in range(batch):
                if not quad:
                    low = np.tril(inp[b], -1)
                    g32 = low + low.T + np.diag(np.diag(inp[b]))
                    g8, g_scale, g_diag = o.i8_gram_quant(g32, int(maxima[slot].view(np.int32)[b]), oscale[b], c0)
                    assert np.array_equal(out8[b], g8) and scale[b] == g_scale and np.array_equal(diag[b], g_diag)
                else:
                    p8, p_scale, p_diag = o.i8_poly_quant(inp[b], maxima[slot][b], odiag[b], c0, c1, c2)
                    assert np.array_equal(out8[b], p8) and scale[b] == p_scale and np.array_equal(diag[b], p_diag)
        elif op == "square":
            g8, gs, gd, p32, maxima, lm, cb, cc, _, slot = a
            blk = np.arange(g8.shape[1]) // 128
            computed = blk[:, None] >= blk[None, :]
            off = computed & ~np.eye(g8.shape[1], dtype=bool)
            for b in range(batch):
                v0, _ = o.i8_square(g8[b], gs[b], gd[b], cb, cc, variant=0)
                v1, _ = o.i8_square(g8[b], gs[b], gd[b], cb, cc, variant=1)
                got = p32[b]
                is0, is1 = got == v0, got == v1
                assert bool((is0 | is1)[computed].all()), "an element equals neither contraction variant"
                canonical += int(is0[computed].sum())
                other += int((~is0)[computed].sum())
                assert maxima[slot][b] == np.abs(got[off]).max()      # the maximum of what was stored
        elif op == "update":
            p8, ps, pd, _, as_, out, maxima, lm, hm, final, tr, _, a8, slot = a
            for b in range(batch):
                y = o.i8_update(p8[b], ps[b], pd[b], a8[b], as_[b])
                if final:
                    got = o.fold(case.y)[b]
                    want = o.cast_output(y[:lm, :hm].T if tr else y[:lm, :hm], case.y.dtype)
                    assert torch.equal(got, want)
                    final_seen = True
                else:
                    assert np.array_equal(out[b][:lm, :hm], y[:lm, :hm])
                    assert maxima[slot][b] == np.abs(y[:lm, :hm]).max()
        elif op == "output_quant":
            inp, maxima, o8, o8t, scale, slot = a
            for b in range(batch):
                want8, want_scale, _ = o.i8_output_quant(inp[b], maxima[slot][b])
                assert np.array_equal(o8[b], want8) and np.array_equal(o8t[b], want8.T) and scale[b] == want_scale
    assert final_seen and all(seen.values())
    share = canonical / (canonical + other)
    print(f"{name}: P32 elements in the canonical contraction variant: {share:.3f} ({other} of {canonical + other} in the other)")
    assert share > 0.5


# ------------------------------------------------------------------------------------------ block quantised
@pytest.mark.parametrize("name", ["bq_int8_staged", "bq_int8_staged_tall", "bq_fp8_staged"])
def test_bq_stages_match_the_reference_kernels(name):
    case = rf.Case(name)
    fp8 = "fp8" in name
    x = case.x
    xw = o.to_wide(o.fold(x).float().numpy())
    batch, l, h = xw.shape
    modes = []

    def close(got, want):
        if not fp8:
            return np.array_equal(got, want)
        return np.allclose(got, want, rtol=1e-5, atol=1e-7)   # raw FP32 tensor-core sums, other order

    for call in case.calls:
        a = [npy(t) if isinstance(t, torch.Tensor) else t for t in case.args(call)]
        if call["op"] == "quant":
            _, norm, out, out_t, scale, _, eps = a
            assert np.allclose(norm, o.frobenius_norm(x), rtol=3e-6, atol=0)
            inv = o._inv_norm(norm, eps)
            lp, hp = out.shape[1:]
            for b in range(batch):
                v = np.zeros((lp, hp), dtype=F32)
                v[:l, :h] = (xw[b] * inv[b]).astype(F32)
                q, s = o.bq_quantise_blocks(v, fp8)
                assert np.array_equal(out[b].astype(F32), q) and np.array_equal(out_t[b], out[b].T)
                assert np.array_equal(scale[b], s)
            continue
        A, sa, da, B, sb, rb, out, ot, so, dout, mode, lm, ln, ca, cb, cc, final, tr, _ = a
        modes.append((mode, bool(final)))
        for b in range(batch):
            if mode == 0:
                gq, sg, dg = o.bq_gram(A[b].astype(F32), sa[b], lm, fp8)
                assert np.array_equal(out[b].astype(F32), gq) and np.array_equal(so[b], sg) and close(dout[b], dg)
            elif mode == 1:
                pq, sp, dp = o.bq_poly(A[b].astype(F32), sa[b], da[b], (ca, cb, cc), lm, fp8)
                assert np.array_equal(out[b].astype(F32), pq) and np.array_equal(so[b], sp) and close(dout[b], dp)
            else:
                y = o.bq_update(A[b].astype(F32), sa[b], da[b], rb[b].astype(F32), sb[b], lm, ln, fp8)
                if final:
                    got = o.fold(case.y)[b]
                    want = o.cast_output(y[:lm, :ln].T if tr else y[:lm, :ln], case.y.dtype)
                    assert torch.equal(got, want)
                else:
                    q, s = o.bq_quantise_blocks(y, fp8)
                    assert np.array_equal(out[b].astype(F32), q) and np.array_equal(ot[b], out[b].T)
                    assert np.array_equal(so[b], s)
    assert modes[-1] == (2, True) and {m for m, _ in modes} == {0, 1, 2}


# ------------------------------------------------------------------------------------------ whole entry points
def _norm_of(case):
    return npy(case.ops("normalize")[0][1])


FLOAT_CASES = [("float_regular_float32", 1e-5), ("float_regular_bfloat16", 2e-2), ("float_regular_float16", 2e-2),
               ("float_regular_tall_bf16", 2e-2), ("float_first_row_fp16_of_fp32", 2e-2),
               ("gram_bf16_00100", 2e-2), ("gram_fp16_00100", 2e-2), ("gram_fp32_00100", 1e-5),
               ("gram_fp16_pe8_01010101", 2e-2), ("gram_fp16_0010010", 2e-2)]


@pytest.mark.parametrize("name,tolerance", FLOAT_CASES)
def test_floating_routes_against_the_reference_kernels(name, tolerance):
    case = rf.Case(name)
    m = case.manifest
    kwargs = dict(gram=True, order=m["env"].get("I8MUON_GRAM_RESET", "00100")) if m["entry"] == "_gram_prec" else {}
    y = o.ns_float(case.x, case.coeffs, case.eps, m["precision"], norm=_norm_of(case), **kwargs)
    assert rel(y.float(), case.y.float()) <= tolerance


def test_polar_express_default_order_is_ill_conditioned_in_the_reference_too():
    """FP16 Gram + Polar Express x8 with the default restart order ``00100``: the reference's own kernel
    output is 0.12 away from the exact FP32 iteration and 0.18 away from a restatement of the same
    arithmetic that only accumulates differently, while with order ``01010101`` both agree to 3e-3.
    This fixture is the evidence for comparing that configuration by distance to the exact iteration."""
    case = rf.Case("gram_fp16_pe8_default")
    truth = o.ns_fp32_torch(case.x, case.coeffs)
    y = o.ns_float(case.x, case.coeffs, case.eps, "float16", norm=_norm_of(case), gram=True, order="00100")
    ref_to_truth, ours_to_truth = rel(case.y.float(), truth.float()), rel(y.float(), truth.float())
    assert 2e-2 < ref_to_truth < 0.3 and ours_to_truth < 1.5 * ref_to_truth + 1e-2
    assert rel(y.float(), case.y.float()) > 2e-2          # not a 2e-2 configuration, by the reference's own output


def test_fp16_first_entry_points_against_the_reference_kernels():
    """The reference's default engine setting: first row in FP16, its result rounded to the input dtype,
    then the quantised rows without re-normalising (_cutlass.py:137-142).  The quantised rows are
    discontinuous in their input (one flipped code moves the result by ~1e-2), so they are checked from
    the reference's own first-row result, which the fixtures hold as the input of its quantiser; the
    first row itself is checked against the oracle's FP16 iteration."""
    for name, quantiser, fn in (("i8_fp16first", "stats", o.ns_int8), ("bq_int8_fp16first", "quant", o.ns_bq),
                                ("bq_int8_fp16first_512x1024", "quant", o.ns_bq)):
        case = rf.Case(name)
        first = case.ops(quantiser)[0][0].reshape(case.x.shape)
        mine = o.ns_float(case.x, case.coeffs[:1], case.eps, "float16", norm=_norm_of(case))
        assert rel(mine.float(), first.float()) <= 2e-2, name
        y = fn(case.x, case.coeffs, case.eps, fp16_first=True, first=first)
        if fn is o.ns_bq:
            assert torch.equal(y, case.y), f"{name}: INT8-BQ rows from the same first row are bit-identical"
        else:
            assert rel(y.float(), case.y.float()) <= 2e-2, name
    for name, fp8 in (("bq_int8_5rows", False), ("bq_fp8_5rows", True)):
        case = rf.Case(name)
        norm = npy(case.ops("quant")[0][1])
        y = o.ns_bq(case.x, case.coeffs, case.eps, fp8=fp8, norm=norm)
        if fp8:
            assert rel(y.float(), case.y.float()) <= 2e-2
        else:
            assert torch.equal(y, case.y), "INT8-BQ from the same norm is bit-identical end to end"
