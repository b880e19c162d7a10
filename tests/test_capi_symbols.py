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


def test_attention_plan_balances_causal_units_without_a_gpu():
    """The ownership planner is host code: for the per-rank Ulysses shape (4 heads, 32768 causal
    tokens, 148 CTAs) every unit is owned exactly once and the heaviest CTA carries at most 8 %
    more key blocks than the average."""
    from syncopate_b200 import _lib as L

    a = L.AttnArgs()
    a.Z, a.Hq, a.Hkv, a.Sq, a.Skv, a.D = 1, 4, 4, 32768, 32768, 128
    a.causal, a.dtype, a.num_sms = 1, L.SYN_DTYPE_BF16, 148
    sched, keep = L.make_schedule([[0, 0, 0, 0]], [[1, 4, 32768, 32768]], None, ndim=4)
    plan = L.AttnPlan()
    assert L.lib().syn_attention_plan(ctypes.byref(a), ctypes.byref(sched), None, None, ctypes.byref(plan)) == 0
    assert (plan.grid, plan.unit_rows, plan.num_units) == (148, 256, 512)
    owned = sorted(plan.units[i] for i in range(plan.start[148]))
    assert owned == list(range(512))
    blocks = lambda u: min(2 * (u % 128) + 2, 256)  # noqa: E731  key blocks a causal tile pair visits
    loads = [sum(blocks(plan.units[i]) for i in range(plan.start[c], plan.start[c + 1])) for c in range(148)]
    assert max(loads) <= 1.08 * sum(loads) / 148
    a.Hq = a.Hkv = 64  # 8192 units: more than a plan holds
    assert L.lib().syn_attention_plan(ctypes.byref(a), ctypes.byref(sched), None, None, ctypes.byref(plan)) == L.SYN_ERR_TOO_LARGE
