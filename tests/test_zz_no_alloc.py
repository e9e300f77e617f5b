"""The allocation-free statistics entry point, for callers that cannot reach an
allocator (a fixed memory budget set by the host framework, a latency-critical
thread where cudaMalloc's implicit synchronisation is forbidden, a foreign thread).

It keeps the partial sums of the two-pass reduction in an array inside the
library image instead of caller scratch.  Checked here through the C ABI against
the ordinary entry point: both launch the same kernels, so the results must be
identical, on two calls in a row (the array keeps the previous call's contents)
and on shapes that leave stale partials behind.  The size limit must be refused
with a clear error instead of overrunning the array.
"""
import ctypes

import pytest
import torch

from i8muon_b200 import native

pytestmark = pytest.mark.gpu
DT = {torch.float32: native.F32, torch.float16: native.F16, torch.bfloat16: native.BF16}


def stats_with_scratch(x):
    b, count = x.shape[0], x[0].numel()
    nbytes = native.stats_scratch_bytes(b, count)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    norm, amax = torch.empty(b, device=x.device), torch.empty(b, device=x.device)
    native.call("i8m_stats", x.data_ptr(), DT[x.dtype], b, count, scratch.data_ptr(), nbytes, norm.data_ptr(),
                amax.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return norm, amax


def stats_static(x):
    b, count = x.shape[0], x[0].numel()
    norm = torch.full((b,), float("nan"), device=x.device)
    amax = torch.full((b,), float("nan"), device=x.device)
    native.call("i8m_stats_static", x.data_ptr(), DT[x.dtype], b, count, norm.data_ptr(), amax.data_ptr(),
                torch.cuda.current_stream().cuda_stream)
    return norm, amax


def test_static_scratch_matches_caller_scratch_twice_in_a_row(cuda_device):
    gen = torch.Generator().manual_seed(99)
    big = (torch.randn((5, 300, 1000), generator=gen) * 3).to(torch.bfloat16).to(cuda_device)
    small = torch.randn((2, 17, 33), generator=gen).to(cuda_device)   # leaves stale partials of `big` behind
    for x in (big, big, small, big):
        want_norm, want_amax = stats_with_scratch(x)
        got_norm, got_amax = stats_static(x)
        torch.cuda.synchronize()
        assert torch.equal(got_norm, want_norm)   # same kernels, same order: identical, tolerance zero
        assert torch.equal(got_amax, want_amax)
        assert torch.allclose(got_norm, x.float().norm(dim=(1, 2)), rtol=2e-6)
    # either output may be omitted
    norm = torch.empty(5, device=cuda_device)
    native.call("i8m_stats_static", big.data_ptr(), native.BF16, 5, 300 * 1000, norm.data_ptr(), None,
                torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert torch.equal(norm, stats_with_scratch(big)[0])


def test_static_scratch_refuses_oversized_requests(cuda_device):
    x = torch.zeros(8, device=cuda_device)
    lib = native.library()
    # 65535 matrices of 8192 * 9 elements need 589815 partial pairs > 524288
    code = lib.i8m_stats_static(x.data_ptr(), native.F32, 65535, 8192 * 9, None, None, None)
    assert code == -4
    assert b"exceeds the built-in scratch" in lib.i8m_last_error()
    with pytest.raises(native.NativeError):
        native.call("i8m_stats_static", None, native.F32, 1, 8, None, None, None)
