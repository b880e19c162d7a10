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
    assert lib.syn_flag_wait_stream(None, 1, None) == -1
    assert lib.syn_attention_plan(None, None, None, None, None) == -1
    assert lib.syn_gemm_rs(None, None, None, None) == -1


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


def test_attention_plan_with_zigzag_positions_and_waves():
    """Context-parallel shape (rank 3 of 8, 8192 local queries, eight KV waves of 8192 keys, zigzag
    positions): the planner weighs a unit by the key blocks its tiles really see in every wave, so the
    late half of the local queries (which sees nearly everything) is spread over all CTAs."""
    from syncopate_b200 import _lib as L
    from syncopate_b200.computation.attn.plan import zigzag_tables

    world, rank, S, H = 8, 3, 65536, 8
    local = S // world
    q_pos, kv_pos = zigzag_tables(world, rank, S)
    a = L.AttnArgs()
    a.Z, a.Hq, a.Hkv, a.Sq, a.Skv, a.D = 1, H, 1, local, S, 128
    a.causal, a.dtype, a.num_sms = 1, L.SYN_DTYPE_BF16, 148
    a.q_pos, a.kv_pos = 1, 1  # device pointers are not touched by the planner; non-NULL marks "tables given"
    offs = [[0, 0, 0, ((rank + i) % world) * local] for i in range(world)]
    sizes = [[1, H, local, local]] * world
    sched, keep = L.make_schedule(offs, sizes, None, ndim=4)
    qh = (ctypes.c_int32 * len(q_pos))(*q_pos)
    kh = (ctypes.c_int32 * len(kv_pos))(*kv_pos)
    plan = L.AttnPlan()
    assert L.lib().syn_attention_plan(ctypes.byref(a), ctypes.byref(sched), qh, kh, ctypes.byref(plan)) == 0
    per_head = local // 256
    assert plan.num_units == H * per_head and sorted(plan.units[i] for i in range(plan.start[148])) == list(range(H * per_head))

    def weight(u):  # key blocks (of any wave) that the two tiles of unit u see
        seen = 0
        for kb, kp in enumerate(kv_pos):
            seen += any(kp <= q_pos[2 * u + x] + 127 for x in range(2))
        return seen

    w = [weight(u) for u in range(per_head)]
    loads = [sum(w[plan.units[i] % per_head] for i in range(plan.start[c], plan.start[c + 1])) for c in range(148)]
    assert max(loads) <= 1.25 * sum(loads) / 148   # 256 units of very different length on 148 CTAs
    # tables must be given on both sides or on neither
    assert L.lib().syn_attention_plan(ctypes.byref(a), ctypes.byref(sched), None, kh, ctypes.byref(plan)) == -1
