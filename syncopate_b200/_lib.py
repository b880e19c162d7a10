"""ctypes binding of ``libsyncopate_b200.so`` (the C ABI declared in ``include/syncopate_b200.h``).

The shared library is built in-tree by :mod:`syncopate_b200.build` (``nvcc`` for sm_100a).  There is
no fallback of any kind: when the library is missing, :func:`lib` raises ``RuntimeError``.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence

_HERE = os.path.dirname(os.path.abspath(__file__))
# SYNCOPATE_B200_LIB points at another build of the same library (tuning experiments).
LIB_PATH = os.environ.get("SYNCOPATE_B200_LIB") or os.path.join(_HERE, "libsyncopate_b200.so")

SYN_MAX_WORLD = 8
SYN_DTYPE_F16 = 0
SYN_DTYPE_BF16 = 1
SYN_ERR_TOO_LARGE = -9

ERRORS = {
    0: "SYN_OK",
    -1: "SYN_ERR_INVALID",
    -2: "SYN_ERR_SHAPE",
    -3: "SYN_ERR_CUDA",
    -4: "SYN_ERR_TIMEOUT_FLAG",
    -5: "SYN_ERR_TIMEOUT_MBAR",
    -6: "SYN_ERR_TIMEOUT_COUNTER",
    -7: "SYN_ERR_RENDEZVOUS",
    -8: "SYN_ERR_UNSUPPORTED",
    -9: "SYN_ERR_TOO_LARGE",
}


class SynError(RuntimeError):
    """A C-ABI call returned a negative code."""

    def __init__(self, code: int, where: str, detail: str = ""):
        self.code = code
        name = ERRORS.get(code, str(code))
        msg = f"{where}: {name}"
        if detail:
            msg += f" ({detail})"
        super().__init__(msg)


class Schedule(C.Structure):
    """``syn_schedule``."""

    _fields_ = [
        ("num_waves", C.c_int32),
        ("ndim", C.c_int32),
        ("offsets", C.POINTER(C.c_int32)),
        ("shapes", C.POINTER(C.c_int32)),
        ("signals", C.POINTER(C.c_int32)),
        ("target_ranks", C.POINTER(C.c_int32)),
        ("dst_offsets", C.POINTER(C.c_int32)),
    ]


class GemmArgs(C.Structure):
    """``syn_gemm_args``."""

    _fields_ = [
        ("a", C.c_void_p),
        ("b", C.c_void_p),
        ("c", C.c_void_p),
        ("M", C.c_int32),
        ("N", C.c_int32),
        ("K", C.c_int32),
        ("lda", C.c_int32),
        ("ldb", C.c_int32),
        ("ldc", C.c_int32),
        ("dtype", C.c_int32),
        ("block_m", C.c_int32),
        ("block_n", C.c_int32),
        ("block_k", C.c_int32),
        ("group_size_m", C.c_int32),
        ("num_sms", C.c_int32),
        ("consumer_signal_ptr", C.c_void_p),
        ("producer_signal_ptr", C.c_void_p),
        ("producer_counter_ptr", C.c_void_p),
        ("signal_value", C.c_uint64),
        ("timeout_ns", C.c_uint64),
        ("status", C.c_void_p),
        ("sched_counter", C.c_void_p),
        ("trace", C.c_void_p),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
    ]


class Symm(C.Structure):
    """``syn_symm``: all ranks' pointers of one symmetric buffer."""

    _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("ptrs", C.c_void_p * SYN_MAX_WORLD)]

    @classmethod
    def of(cls, rank: int, ptrs: Sequence[int]) -> "Symm":
        s = cls()
        s.world = len(ptrs)
        s.rank = rank
        for i, p in enumerate(ptrs):
            s.ptrs[i] = p
        return s


class AgGemmArgs(C.Structure):
    """``syn_ag_gemm_args``."""

    _fields_ = [("gemm", GemmArgs), ("a", Symm), ("counters", C.c_void_p)]


class GemmRsArgs(C.Structure):
    """``syn_gemm_rs_args``."""

    _fields_ = [
        ("gemm", GemmArgs),
        ("stage", Symm),
        ("recv_flags", Symm),
        ("remote_signals", C.POINTER(C.c_int32)),
        ("out", C.c_void_p),
        ("ldo", C.c_int32),
        ("counters", C.c_void_p),
        ("send_buf", C.c_void_p),
        ("send_flags", C.c_void_p),
        ("out_flags", C.c_void_p),
        ("reduce_pass", C.c_int32),
        ("reserved", C.c_int32),
    ]


class CeStep(C.Structure):
    """``syn_ce_step``: wait for a flag, copy, raise a flag - on one of the caller's streams."""

    _fields_ = [
        ("wait_flag", C.c_void_p),
        ("dst", C.c_void_p),
        ("src", C.c_void_p),
        ("bytes", C.c_size_t),
        ("set_flag", C.c_void_p),
        ("stream", C.c_int32),
        ("reserved", C.c_int32),
    ]


def make_ce_program(steps):
    """ctypes array of ``syn_ce_step`` from ``(wait_flag, dst, src, nbytes, set_flag, stream)`` tuples
    (addresses as integers, 0 / None = absent)."""
    arr = (CeStep * max(len(steps), 1))()
    for i, (wait, dst, src, nbytes, flag, stream) in enumerate(steps):
        arr[i].wait_flag = wait or None
        arr[i].dst = dst or None
        arr[i].src = src or None
        arr[i].bytes = int(nbytes)
        arr[i].set_flag = flag or None
        arr[i].stream = int(stream)
    return arr


def ce_run(program, num_steps: int, streams, value: int, flag_stream=None) -> None:
    """Issues a copy-engine program (``make_ce_program``) on ``streams`` (torch streams); with
    ``flag_stream`` the flag writes go there, each behind an event recorded after its copy."""
    ptrs = (C.c_void_p * len(streams))(*[s.cuda_stream or None for s in streams])
    fs = flag_stream.cuda_stream if flag_stream is not None else None
    check(lib().syn_ce_run(program, num_steps, ptrs, len(streams), fs, value), "syn_ce_run")


class AttnArgs(C.Structure):
    """``syn_attn_args``."""

    _fields_ = [
        ("q", C.c_void_p),
        ("k", C.c_void_p),
        ("v", C.c_void_p),
        ("o", C.c_void_p),
        ("lse", C.c_void_p),
        ("visit", C.c_void_p),
        ("Z", C.c_int32),
        ("Hq", C.c_int32),
        ("Hkv", C.c_int32),
        ("Sq", C.c_int32),
        ("Skv", C.c_int32),
        ("D", C.c_int32),
        ("q_strides", C.c_int64 * 3),
        ("k_strides", C.c_int64 * 3),
        ("v_strides", C.c_int64 * 3),
        ("o_strides", C.c_int64 * 3),
        ("sm_scale", C.c_float),
        ("causal", C.c_int32),
        ("q_pos", C.c_void_p),
        ("kv_pos", C.c_void_p),
        ("dtype", C.c_int32),
        ("num_sms", C.c_int32),
        ("epoch", C.c_int32),
        ("signal_ptr", C.c_void_p),
        ("signal_value", C.c_uint64),
        ("timeout_ns", C.c_uint64),
        ("status", C.c_void_p),
        ("plan", C.c_void_p),
        ("push", C.c_void_p),
    ]


class AttnPushSlab(C.Structure):
    """``syn_attn_push_slab``."""

    _fields_ = [("q_begin", C.c_int32), ("q_rows", C.c_int32), ("dst_rank", C.c_int32), ("dst_row0", C.c_int32),
                ("flag", C.c_int32)]


class AttnPush(C.Structure):
    """``syn_attn_push``: the attention kernel's producer role."""

    _fields_ = [
        ("num_slabs", C.c_int32),
        ("slabs", C.POINTER(AttnPushSlab)),
        ("dst", Symm),
        ("dst_strides", C.c_int64 * 3),
        ("dst_rows", C.c_int32),
        ("dst_heads", C.c_int32),
        ("head_offset", C.c_int32),
        ("flags", Symm),
        ("counters", C.c_void_p),
    ]


ATTN_PLAN_MAX_GRID = 160
ATTN_PLAN_MAX_UNITS = 2048


class AttnPlan(C.Structure):
    """``syn_attn_plan``."""

    _fields_ = [
        ("grid", C.c_int32),
        ("unit_rows", C.c_int32),
        ("num_units", C.c_int32),
        ("start", C.c_uint16 * (ATTN_PLAN_MAX_GRID + 1)),
        ("units", C.c_uint16 * ATTN_PLAN_MAX_UNITS),
        ("visits", C.c_uint8 * (2 * ATTN_PLAN_MAX_UNITS)),
    ]


class CopyOp(C.Structure):
    """``syn_copy_op``."""

    _fields_ = [
        ("src_rank", C.c_int32),
        ("dst_rank", C.c_int32),
        ("src_buf", C.c_int32),
        ("dst_buf", C.c_int32),
        ("src_offset", C.c_uint64),
        ("dst_offset", C.c_uint64),
        ("src_pitch", C.c_uint64),
        ("dst_pitch", C.c_uint64),
        ("rows", C.c_uint32),
        ("row_bytes", C.c_uint32),
        ("flag_rank", C.c_int32),
        ("flag", C.c_int32),
        ("reduce", C.c_int32),
        ("dtype", C.c_int32),
    ]


class AttnComm(C.Structure):
    """``syn_attn_comm``."""

    _fields_ = [
        ("num_ops", C.c_int32),
        ("ops", C.POINTER(CopyOp)),
        ("num_bufs", C.c_int32),
        ("bufs", Symm * 4),
        ("flags", Symm),
        ("counters", C.c_void_p),
    ]


_lib: Optional[C.CDLL] = None


def lib() -> C.CDLL:
    """Loads the shared library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m syncopate_b200.build` "
                "(nvcc, sm_100a). There is no CPU or PyTorch fallback."
            )
        _lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
        _declare(_lib)
    return _lib


def _declare(l: C.CDLL) -> None:
    l.syn_strerror.restype = C.c_char_p
    l.syn_strerror.argtypes = [C.c_int]
    l.syn_last_cuda_error.restype = C.c_char_p
    l.syn_version.restype = C.c_char_p
    l.syn_gemm.restype = C.c_int
    l.syn_gemm.argtypes = [C.POINTER(GemmArgs), C.POINTER(Schedule), C.POINTER(Schedule), C.c_void_p]
    l.syn_gemm_noalloc.restype = C.c_int
    l.syn_gemm_noalloc.argtypes = [C.POINTER(GemmArgs), C.POINTER(Schedule), C.POINTER(Schedule), C.c_void_p]
    l.syn_gemm_mod1d.restype = C.c_int
    l.syn_gemm_mod1d.argtypes = [C.POINTER(GemmArgs), C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    l.syn_gemm_pick_block_n.restype = C.c_int
    l.syn_gemm_pick_block_n.argtypes = [C.c_int, C.c_int, C.c_int]
    l.syn_ctx_create.restype = C.c_int
    l.syn_ctx_create.argtypes = [C.c_int, C.c_int, C.c_int, C.c_char_p, C.POINTER(C.c_void_p)]
    l.syn_ctx_destroy.restype = C.c_int
    l.syn_ctx_destroy.argtypes = [C.c_void_p]
    l.syn_symm_alloc.restype = C.c_int
    l.syn_symm_alloc.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.POINTER(Symm)]
    l.syn_symm_free.restype = C.c_int
    l.syn_symm_free.argtypes = [C.c_void_p, C.c_void_p]
    l.syn_preload.restype = C.c_int
    l.syn_preload.argtypes = []
    l.syn_barrier.restype = C.c_int
    l.syn_barrier.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64]
    l.syn_ctx_status_ptr.restype = C.c_void_p
    l.syn_ctx_status_ptr.argtypes = [C.c_void_p]
    l.syn_ctx_status.restype = C.c_int
    l.syn_ctx_status.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_int32)]
    l.syn_memcpy_async.restype = C.c_int
    l.syn_memcpy_async.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    l.syn_flag_set.restype = C.c_int
    l.syn_flag_set.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p]
    l.syn_flag_wait.restype = C.c_int
    l.syn_flag_wait.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_void_p, C.c_int, C.c_void_p]
    l.syn_flag_wait_stream.restype = C.c_int
    l.syn_flag_wait_stream.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p]
    l.syn_ce_run.restype = C.c_int
    l.syn_ce_run.argtypes = [C.POINTER(CeStep), C.c_int, C.POINTER(C.c_void_p), C.c_int, C.c_void_p, C.c_uint64]
    l.syn_ag_gemm.restype = C.c_int
    l.syn_ag_gemm.argtypes = [C.POINTER(AgGemmArgs), C.POINTER(Schedule), C.c_void_p]
    l.syn_copy.restype = C.c_int
    l.syn_copy.argtypes = [C.POINTER(AttnComm), C.c_int, C.c_uint64, C.c_uint64, C.c_void_p, C.c_void_p]
    l.syn_attention.restype = C.c_int
    l.syn_attention.argtypes = [C.POINTER(AttnArgs), C.POINTER(Schedule), C.POINTER(AttnComm), C.c_void_p]
    l.syn_attention_plan.restype = C.c_int
    l.syn_attention_plan.argtypes = [C.POINTER(AttnArgs), C.POINTER(Schedule), C.c_void_p, C.c_void_p,
                                     C.POINTER(AttnPlan)]
    l.syn_gemm_rs.restype = C.c_int
    l.syn_gemm_rs.argtypes = [C.POINTER(GemmRsArgs), C.POINTER(Schedule), C.POINTER(Schedule), C.c_void_p]


def check(code: int, where: str) -> None:
    if code != 0:
        detail = ""
        if code == -3:
            detail = lib().syn_last_cuda_error().decode()
        raise SynError(code, where, detail)


def int32_array(values: Optional[Sequence[int]]):
    """Host int32 array (kept alive by the caller) or a NULL pointer."""
    if values is None:
        return None, C.POINTER(C.c_int32)()
    flat = [int(v) for v in values]
    arr = (C.c_int32 * max(len(flat), 1))(*flat)
    return arr, C.cast(arr, C.POINTER(C.c_int32))


def make_schedule(offsets, shapes, signals=None, target_ranks=None, dst_offsets=None, ndim: int = 2):
    """Builds a ``syn_schedule`` from nested Python lists (the ``RawSchedule.gen_*`` outputs).

    Returns ``(struct, keepalive)``; keep ``keepalive`` referenced until the call returns.
    """

    def flat(x):
        if x is None:
            return None
        out = []
        for row in x:
            if isinstance(row, (list, tuple)):
                out.extend(int(v) for v in row)
            else:
                out.append(int(row))
        return out

    offs, shp = flat(offsets), flat(shapes)
    nw = len(shp) // ndim
    keep = []
    s = Schedule()
    s.num_waves = nw
    s.ndim = ndim
    for name, vals in (
        ("offsets", offs),
        ("shapes", shp),
        ("signals", flat(signals)),
        ("target_ranks", flat(target_ranks)),
        ("dst_offsets", flat(dst_offsets)),
    ):
        arr, ptr = int32_array(vals)
        keep.append(arr)
        setattr(s, name, ptr)
    return s, keep


def make_attn_comm(ops, bufs, flags, counters_ptr):
    """``syn_attn_comm`` from a list of CopyOp, a list of Symm buffer tables, the flag table and the
    device pointer of the counters.  Returns ``(struct, keepalive)``."""
    arr = (CopyOp * max(len(ops), 1))(*ops)
    c = AttnComm()
    c.num_ops = len(ops)
    c.ops = C.cast(arr, C.POINTER(CopyOp))
    c.num_bufs = len(bufs)
    for i, b in enumerate(bufs):
        c.bufs[i] = b
    c.flags = flags
    c.counters = counters_ptr
    return c, arr
