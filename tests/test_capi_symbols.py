"""The C-ABI library builds for sm_100a, loads without a GPU and exports every function that
include/syncopate_b200.h declares (no compute call is made here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "syncopate_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b(syn_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_the_expected_entry_points():
    names = _declared_functions()
    for must in ("syn_gemm", "syn_ag_gemm", "syn_gemm_rs", "syn_ctx_create", "syn_symm_alloc", "syn_barrier",
                 "syn_strerror"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from syncopate_b200 import build

    path = build.build()
    lib = ctypes.CDLL(path)
    missing = [n for n in _declared_functions() if not hasattr(lib, n)]
    assert not missing, f"declared in the header but not exported: {missing}"
    lib.syn_version.restype = ctypes.c_char_p
    assert b"sm_100a" in lib.syn_version()
    lib.syn_strerror.restype = ctypes.c_char_p
    assert lib.syn_strerror(-4) == b"device wait on a signal flag timed out"


def test_argument_errors_are_reported_without_a_gpu():
    from syncopate_b200 import _lib as L

    lib = L.lib()
    assert lib.syn_gemm(None, None, None, None) == -1
    assert lib.syn_gemm_pick_block_n(8192, 3584, 148) == 224
    assert lib.syn_gemm_pick_block_n(8192, 8192, 148) == 256
    assert lib.syn_gemm_pick_block_n(0, 8, 148) == -1
    out = ctypes.c_void_p()
    assert lib.syn_ctx_create(3, 2, 0, b"/tmp/x", ctypes.byref(out)) == -1  # rank >= world


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from syncopate_b200 import _lib as L

    monkeypatch.setattr(L, "_lib", None)
    monkeypatch.setattr(L, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        L.lib()
