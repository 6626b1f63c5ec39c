"""The C-ABI library loads on a CPU-only host and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "flaggems_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fg_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    assert "fg_scaled_mm_fp8" in syms and "fg_act_quant_bf16_e4m3" in syms and len(syms) >= 12


def test_library_exports_every_declared_symbol():
    from flaggems_b200 import _cabi
    from flaggems_b200.build import build

    build()
    handle = ctypes.CDLL(_cabi.LIB_PATH)
    for s in declared_symbols():
        assert hasattr(handle, s), f"{s} declared in include/flaggems_b200.h but not exported"
    for s in _cabi.EXPORTED_SYMBOLS:
        assert s in declared_symbols(), f"{s} bound in _cabi.py but not declared in the header"
    assert _cabi.lib().fg_version() >= 100


def test_host_rejects_cpu_tensors_loudly():
    import torch

    import flag_gems
    from flaggems_b200._cabi import FlagGemsB200Error

    x = torch.randn(4, 128).bfloat16()
    with pytest.raises(FlagGemsB200Error):
        flag_gems.act_quant_triton(x)
    with pytest.raises(FlagGemsB200Error):
        flag_gems.per_token_group_quant_fp8(x, 128)
    with pytest.raises(AssertionError):
        flag_gems.act_quant_triton(x[:, :100].contiguous(), 128)


def test_missing_library_fails_loudly(monkeypatch):
    from flaggems_b200 import _cabi

    monkeypatch.setattr(_cabi, "_lib", None)
    monkeypatch.setattr(_cabi, "LIB_PATH", "/nonexistent/libflaggems_b200.so")
    with pytest.raises(_cabi.FlagGemsB200Error):
        _cabi.lib()
