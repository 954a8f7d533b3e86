"""CPU: the C-ABI library builds, loads, and exports every symbol include/b200moe.h declares."""
import ctypes
import os
import re

import pytest

from tests.conftest import ROOT, load_pkg


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200moe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200moe_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    pkg = load_pkg()
    path = pkg.build()
    handle = ctypes.CDLL(path)
    declared = _declared_symbols()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(handle, name), f"{name} declared in include/b200moe.h but not exported"
    assert sorted(pkg.EXPORTED) == declared, "ctypes signature table and header disagree"


def test_host_only_entry_points():
    pkg = load_pkg()
    lib = pkg.lib()
    assert b"sm_100a" in lib.b200moe_version()
    assert lib.b200moe_padded_rows_cap(98304, 64) == (98304 // 256 + 64) * 256
    assert lib.b200moe_padded_rows_cap(1, 1) == 512
    assert lib.b200moe_permute_ws_bytes(98304, 64) >= 98304 // 512 * 64 * 4
    assert b"expert index" in lib.b200moe_status_string(5)


def test_argument_errors_are_python_exceptions():
    """Bad shapes are rejected on the host before anything is launched (no GPU needed)."""
    pkg = load_pkg()
    lib = pkg.lib()
    from importlib import import_module
    L = import_module(pkg.__name__ + "._lib")
    rc = lib.b200moe_router_topk_fwd(1, 0, None, 4, 300, 2, 1, 1.0, 1, 1, None, None)   # E too large
    assert rc == -3
    with pytest.raises(ValueError, match="E = 300"):
        L.check(rc)
    rc = lib.b200moe_gemm_nt(16, 16, 16, 8, 12, 64, None, None)                          # N % 8 != 0
    assert rc == -1
    with pytest.raises(ValueError):
        L.check(rc)
    assert lib.b200moe_combine(None, None, None, 4, 2, 64, None, None) == -6


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    pkg = load_pkg()
    from importlib import import_module
    L = import_module(pkg.__name__ + "._lib")
    monkeypatch.setattr(L, "_lib", None)
    monkeypatch.setattr(L, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no fallback"):
        L.lib()


def test_cpu_tensors_are_rejected():
    import torch
    pkg = load_pkg()
    x = torch.zeros(4, 64, dtype=torch.bfloat16)
    idx = torch.zeros(4, 2, dtype=torch.int64)
    w = torch.zeros(4, 2)
    gu = torch.zeros(2, 32, 64, dtype=torch.bfloat16)
    dn = torch.zeros(2, 64, 16, dtype=torch.bfloat16)
    codes = torch.zeros(2, dtype=torch.int32)
    with pytest.raises(ValueError, match="CUDA"):
        pkg.moe(x, idx, w, gu, dn, codes)
    with pytest.raises(ValueError, match="unknown act code 9"):
        pkg.moe(x, idx, w, gu, dn, torch.tensor([0, 9], dtype=torch.int32))
    with pytest.raises(ValueError, match="must precede"):
        pkg.moe(x, idx, w, gu, dn, torch.tensor([3, 0, 1], dtype=torch.int32))
