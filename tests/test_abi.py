"""The C-ABI library loads without a GPU, exports every symbol the header
declares, and rejects bad arguments with error codes instead of crashing."""
import ctypes
import re
from pathlib import Path

import pytest

from i8muon_b200 import native
from i8muon_b200.build import LIBRARY, build

HEADER = Path(__file__).resolve().parents[1] / "include" / "i8muon_b200.h"


@pytest.fixture(scope="module")
def lib():
    build()
    return native.library()


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(i8m_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    names = declared_symbols()
    assert len(names) >= 18
    raw = ctypes.CDLL(str(LIBRARY))
    for name in names:
        assert hasattr(raw, name), f"{name} declared in the header but not exported"
    assert sorted(native.EXPORTED_SYMBOLS) == names


def test_build_info_and_version(lib):
    assert lib.i8m_version() >= 100
    info = native.build_info()
    assert "sm_100a" in info and "tcgen05" in info


def test_workspace_queries(lib):
    small = native.ns_workspace_bytes(native.ROUTE_FLOAT, 1, 64, 256, native.F32, native.F16, 5, 0)
    large = native.ns_workspace_bytes(native.ROUTE_FLOAT, 4, 64, 256, native.F32, native.F16, 5, 0)
    assert 0 < small < large and small % 256 == 0
    # fp16_first needs the floating stage's buffers on top of the quantised ones
    plain = native.ns_workspace_bytes(native.ROUTE_BQ_INT8, 2, 512, 1024, native.BF16, native.F16, 5, 0)
    first = native.ns_workspace_bytes(native.ROUTE_BQ_INT8, 2, 512, 1024, native.BF16, native.F16, 5, 1)
    assert first > plain
    # fp32 compute keeps two planes per matrix
    f16 = native.ns_workspace_bytes(native.ROUTE_GRAM, 2, 128, 1024, native.F32, native.F16, 5, 0)
    f32 = native.ns_workspace_bytes(native.ROUTE_GRAM, 2, 128, 1024, native.F32, native.F32, 5, 0)
    assert f32 > 3 * f16
    assert native.stats_scratch_bytes(3, 8193) == 2 * 3 * 2 * 4


def test_argument_errors_are_codes_not_crashes(lib):
    size = ctypes.c_size_t(0)
    for args in ((99, 1, 8, 8, 0, 1, 5, 0), (0, 0, 8, 8, 0, 1, 5, 0), (0, 70000, 8, 8, 0, 1, 5, 0),
                 (0, 1, 0, 8, 0, 1, 5, 0), (0, 1, 8, 8, 7, 1, 5, 0), (0, 1, 8, 8, 0, 1, 0, 0)):
        assert lib.i8m_ns_workspace_bytes(*args, ctypes.byref(size)) == -1
        assert lib.i8m_last_error()
    with pytest.raises(native.NativeError, match="null"):
        native.call("i8m_ns_run", 0, None, None, 0, 1, 8, 8, 1, None, 5, 1e-7, 0, 1, -1, None, None, None, 0, None, None)
    with pytest.raises(native.NativeError):
        native.call("i8m_momentum", None, None, 0, None, 0, 0, 0.0, 0.0, 0, None, None)
    with pytest.raises(native.NativeError):
        native.call("i8m_bq_gemm", 0, 0, 1, 1, None, 1, 1, None, 1, None, None, None, 1, 100, 128, 128, 100,
                    128, 0.0, 0.0, 0.0, 0, 0, 0, None, None)
