"""The shared library loads without a GPU and exports every symbol the public header declares."""
import os
import re

from quant_cast_bench_b200 import build as qbuild
from quant_cast_bench_b200.quant_cast_cuda import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "quant_cast_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(qcc_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_header_symbols():
    qbuild.build()
    lib = L.load()
    syms = declared_symbols()
    assert len(syms) >= 12
    for s in syms:
        assert hasattr(lib, s), f"{s} declared in include/quant_cast_cuda.h but not exported"
        assert s in L.SIGNATURES, f"{s} has no ctypes signature"
    assert lib.qcc_version() >= 100
    assert lib.qcc_amax_workspace_bytes() > 0


def test_header_constants_match_binding():
    text = open(os.path.join(ROOT, "include", "quant_cast_cuda.h")).read()
    consts = dict(re.findall(r"#define\s+(QCC_[A-Z0-9_]+)\s+(-?\d+)", text))
    assert int(consts["QCC_ROWWISE"]) == L.ROWWISE and int(consts["QCC_COLWISE"]) == L.COLWISE
    assert int(consts["QCC_SWIZZLE"]) == L.SWIZZLE and int(consts["QCC_FLOOR"]) == L.FLOOR and int(consts["QCC_SR"]) == L.SR
    assert int(consts["QCC_FMT_E5M2"]) == L.FMT_E5M2 and int(consts["QCC_AMAX_NVFP4_SCALE"]) == L.AMAX_NVFP4_SCALE
    for code in (-1, -2, -3, -4, -5):
        assert code in L.ERRORS


def test_no_cpu_path():
    import pytest
    import torch
    from quant_cast_bench_b200 import quant_cast_cuda as Q
    x = torch.zeros(32, 32, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        Q.mxfp8_cuda(x)


def test_opt_in_device_check_raises_on_a_recorded_error(monkeypatch):
    """QCC_CHECK_DEVICE=1: after every call the recipe layer reads the device error word and raises when a kernel gave
    up a bounded wait (host logic only: the library is replaced by a stand-in that reports code 19)."""
    import pytest

    class Recorded:
        def qcc_device_error(self, ref):
            ref._obj.value = 19
            return 0

    monkeypatch.setattr(L, "_lib", Recorded())
    monkeypatch.setattr(L, "CHECK_DEVICE", True)
    with pytest.raises(RuntimeError, match="device error 19"):
        L.check(0, "some cast")
    monkeypatch.setattr(L, "CHECK_DEVICE", False)
    L.check(0, "some cast")                      # off by default: no synchronisation, no raise
    with pytest.raises(ValueError):
        L.check(-1, "some cast")
