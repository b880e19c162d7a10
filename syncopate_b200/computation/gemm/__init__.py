"""Host-side entry points of the GEMM kernels, mirroring the argument conventions of the
reference's generated kernels (syncopate/computation/transform/transformer.py:1125-1178; used as in
tests/test_ag_gemm_gen.py:57-76, tests/test_gemm_rs_transform.py:141-158):

* ``gemm``     — persistent GEMM with wave schedule, consumer wait flags and producer flags,
* ``ag_gemm``  — all-gather + GEMM with the gather done by the kernel's comm warps,
* ``gemm_rs``  — GEMM + reduce-scatter with the scatter done by the kernel's epilogue.

``b`` is ``[N, K]`` (K-major, as in the reference).  Schedules are the ``RawSchedule.gen_*`` lists:
Python lists, CPU tensors or CUDA tensors (the latter are copied to the host, which synchronises).
Every call goes through the C ABI of ``libsyncopate_b200.so``; there is no fallback.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from syncopate_b200 import _lib as L

_DTYPES = {torch.float16: L.SYN_DTYPE_F16, torch.bfloat16: L.SYN_DTYPE_BF16}


def _to_list(x):
    if x is None:
        return None
    if isinstance(x, torch.Tensor):
        return x.detach().cpu().tolist()
    return x


def _ptr(t) -> Optional[int]:
    if t is None:
        return None
    if isinstance(t, int):
        return t
    return t.data_ptr()


def _stream_ptr(stream) -> Optional[int]:
    if stream is None:
        stream = torch.cuda.current_stream()
    return stream.cuda_stream or None


def _check_mat(name: str, t: torch.Tensor) -> None:
    if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be a 2-D CUDA tensor with unit inner stride")
    if t.dtype not in _DTYPES:
        raise ValueError(f"{name}: unsupported dtype {t.dtype} (fp16 and bf16 only)")


_WORKSPACES = {}


def tail_workspace(device, stream_ptr=None) -> torch.Tensor:
    """Zeroed scratch (one per device and stream, kept zero by the kernel) that lets the CTA-pair
    GEMM split the tiles left over after the last full persistent round along K.  Launches that
    share a scratch must not overlap on the GPU (its counters and partial tiles belong to one
    launch at a time), which stream order guarantees for one stream; every stream gets its own."""
    index = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    key = (index, stream_ptr or 0)
    ws = _WORKSPACES.get(key)
    if ws is None:
        ws = torch.zeros(256 + 74 * 256 * 256 * 4, dtype=torch.uint8, device=torch.device("cuda", index))
        _WORKSPACES[key] = ws
    return ws


def _gemm_args(a, b, c, num_sms, block_n, group_m, signal_value, timeout_ns, status, stream=None) -> L.GemmArgs:
    _check_mat("a", a)
    _check_mat("b", b)
    if a.dtype != b.dtype or a.shape[1] != b.shape[1]:
        raise ValueError("a [M,K] and b [N,K] must agree in dtype and K")
    g = L.GemmArgs()
    g.a, g.b = a.data_ptr(), b.data_ptr()
    g.M, g.N, g.K = a.shape[0], b.shape[0], a.shape[1]
    g.lda, g.ldb = a.stride(0), b.stride(0)
    if c is not None:
        _check_mat("c", c)
        if c.dtype != a.dtype or tuple(c.shape) != (g.M, g.N):
            raise ValueError("c must be [M, N] of the input dtype")
        g.c, g.ldc = c.data_ptr(), c.stride(0)
    g.dtype = _DTYPES[a.dtype]
    g.block_m, g.block_n, g.block_k = 128, int(block_n or 0), 64
    g.group_size_m = int(group_m or 8)
    g.num_sms = int(num_sms or 0)
    g.signal_value = int(signal_value or 1)
    g.timeout_ns = int(timeout_ns or 0)
    g.status = _ptr(status)
    ws = tail_workspace(a.device, _stream_ptr(stream))
    g.workspace, g.workspace_bytes = ws.data_ptr(), ws.numel()
    return g


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    c: torch.Tensor,
    world_size: int = 1,
    num_gemm_sms: int = 0,
    BLOCK_SIZE_M: int = 128,
    BLOCK_SIZE_N: int = 0,
    BLOCK_SIZE_K: int = 64,
    GROUP_SIZE_M: int = 8,
    STAGES: int = 0,
    *,
    cur_wave_sizes=None,
    wave_offsets=None,
    signal_ptr=None,
    signal_offsets=None,
    producer_signal_ptr=None,
    producer_signal_offsets=None,
    counter_ptr=None,
    cum_tiles: int = 0,
    signal_value: int = 1,
    timeout_ns: int = 0,
    status=None,
    sched_counter=None,
    trace=None,
    stream=None,
) -> torch.Tensor:
    """``c = a @ b.T`` with fp32 accumulation.

    ``cur_wave_sizes`` / ``wave_offsets`` (``[W, 2]``, elements) give the wave order (``[W, 3]`` rows
    are waves over (M, N, K): every wave all of C and one range of K, the consumer form of
    all-to-all + GEMM, as tests/test_all2all_gemm.py:83-110 of the reference builds them);
    ``signal_ptr`` + ``signal_offsets`` make each wave wait for its flag (consumer role);
    ``producer_signal_ptr`` + ``producer_signal_offsets`` + ``counter_ptr`` make each wave raise its
    flag after its last tile (producer role).  ``BLOCK_SIZE_N = 0`` lets the library choose the tile
    width; ``STAGES`` and ``cum_tiles`` are accepted for signature compatibility (the pipeline
    depth is fixed by the shared-memory budget, the tile count follows from the waves).
    """
    if BLOCK_SIZE_M not in (0, 128) or BLOCK_SIZE_K not in (0, 64):
        raise ValueError("this backend uses 128 x N x 64 tiles")
    g = _gemm_args(a, b, c, num_gemm_sms, BLOCK_SIZE_N, GROUP_SIZE_M, signal_value, timeout_ns, status, stream)
    g.sched_counter = _ptr(sched_counter)  # uint32[2], zero: dynamic tile scheduling
    g.trace = _ptr(trace)                  # uint64[2 + 3 * waves] timer stamps (see the header)
    keep = []
    cons = prod = None
    sizes, offs = _to_list(cur_wave_sizes), _to_list(wave_offsets)
    if sizes is not None:
        # rows of three numbers are waves over (M, N, K): ranges of K that arrive separately
        ndim = len(sizes[0]) if len(sizes) and isinstance(sizes[0], (list, tuple)) else 2
        s, k = L.make_schedule(offs, sizes, _to_list(signal_offsets), ndim=ndim)
        keep.append(k)
        cons = s
        g.consumer_signal_ptr = _ptr(signal_ptr)
        if producer_signal_ptr is not None:
            ps, k2 = L.make_schedule(offs, sizes, _to_list(producer_signal_offsets))
            keep.append(k2)
            prod = ps
            g.producer_signal_ptr = _ptr(producer_signal_ptr)
            g.producer_counter_ptr = _ptr(counter_ptr)
    rc = L.lib().syn_gemm(
        C.byref(g), C.byref(cons) if cons is not None else None, C.byref(prod) if prod is not None else None,
        _stream_ptr(stream),
    )
    L.check(rc, "syn_gemm")
    return c


def gemm_mod1d(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, schedule, signal_ptr, *, signal_value: int = 1,
               num_sms: int = 0, block_n: int = 0, timeout_ns: int = 0, status=None, stream=None) -> torch.Tensor:
    """Flag-gated GEMM whose wave schedule is given in closed form: ``schedule`` is a
    ``Mod1DSchedule`` (what ``SimplifiedSchedule(raw).simplify()`` finds for ring and swizzled direct
    all-gathers, syncopate/interface/tile_schedule.py:178-266) or a tuple ``(num_waves, stride,
    starting_offset, axis)``.  No schedule arrays cross the boundary; the library expands the form."""
    if hasattr(schedule, "num_waves"):
        form = (schedule.num_waves, schedule.stride, schedule.starting_offset, schedule.schedule_axis)
    else:
        form = tuple(int(x) for x in schedule)
    g = _gemm_args(a, b, c, num_sms, block_n, 8, signal_value, timeout_ns, status, stream)
    g.consumer_signal_ptr = _ptr(signal_ptr)
    L.check(L.lib().syn_gemm_mod1d(C.byref(g), form[0], form[1], form[2], form[3], _stream_ptr(stream)), "syn_gemm_mod1d")
    return c


def ag_gemm(
    a_symm: L.Symm,
    a_local: torch.Tensor,
    b: torch.Tensor,
    c: torch.Tensor,
    schedule,
    recv_flags,
    counters,
    *,
    epoch: int,
    num_sms: int = 0,
    block_n: int = 0,
    group_size_m: int = 8,
    timeout_ns: int = 0,
    status=None,
    trace=None,
    stream=None,
) -> torch.Tensor:
    """All-gather + GEMM.  ``a_local`` ``[M, K]`` is this rank's copy of the gathered buffer (own
    shard in place) and ``a_symm`` its symmetric table; ``schedule`` is the lowered ``RawSchedule``
    of that buffer (or a tuple ``(offsets, shapes, signals, target_ranks, dst_offsets)``)."""
    g = _gemm_args(a_local, b, c, num_sms, block_n, group_size_m, epoch, timeout_ns, status, stream)
    g.consumer_signal_ptr = _ptr(recv_flags)
    g.trace = _ptr(trace)
    args = L.AgGemmArgs()
    args.gemm = g
    args.a = a_symm
    args.counters = _ptr(counters)
    s, keep = _schedule_struct(schedule)
    rc = L.lib().syn_ag_gemm(C.byref(args), C.byref(s), _stream_ptr(stream))
    L.check(rc, "syn_ag_gemm")
    return c


def gemm_rs(
    a: torch.Tensor,
    b: torch.Tensor,
    out: torch.Tensor,
    src_schedule,
    dst_schedule,
    remote_signals: Sequence[int],
    stage: L.Symm,
    recv_flags: L.Symm,
    counters,
    *,
    epoch: int,
    num_sms: int = 0,
    block_n: int = 0,
    group_size_m: int = 8,
    timeout_ns: int = 0,
    status=None,
    stream=None,
    send_buf: Optional[torch.Tensor] = None,
    send_flags: Optional[torch.Tensor] = None,
    trace=None,
    out_flags: Optional[torch.Tensor] = None,
    reduce_pass: bool = False,
) -> torch.Tensor:
    """GEMM + reduce-scatter.  ``a`` ``[M, K_local]``, ``b`` ``[N, K_local]``; ``out``
    ``[M / world, N]`` receives the fp32 sum over ranks of this rank's row slab.  With ``send_buf``
    ``[world, M / world, N]`` and ``send_flags`` (int64, one word per wave of ``src_schedule``) the
    kernel stores the rows for other ranks locally and raises the local flag of each wave; moving
    them is the caller's job.  ``reduce_pass``: the kernel stores this rank's own partial sum and a
    coalesced pass launched behind it adds the staged ones (instead of the epilogue of the own tiles)."""
    g = _gemm_args(a, b, None, num_sms, block_n, group_size_m, epoch, timeout_ns, status, stream)
    _check_mat("out", out)
    g.trace = _ptr(trace)
    args = L.GemmRsArgs()
    args.gemm = g
    args.stage = stage
    args.recv_flags = recv_flags
    rs_arr, rs_ptr = L.int32_array(list(remote_signals))
    args.remote_signals = rs_ptr
    args.out = out.data_ptr()
    args.ldo = out.stride(0)
    args.counters = _ptr(counters)
    if send_buf is not None:
        args.send_buf = send_buf.data_ptr()
        args.send_flags = send_flags.data_ptr()
    if out_flags is not None:
        args.out_flags = out_flags.data_ptr()  # int64, one word per row piece of the slab kept here
    args.reduce_pass = 1 if reduce_pass else 0
    s, keep1 = _schedule_struct(src_schedule)
    d, keep2 = _schedule_struct(dst_schedule)
    rc = L.lib().syn_gemm_rs(C.byref(args), C.byref(s), C.byref(d), _stream_ptr(stream))
    L.check(rc, "syn_gemm_rs")
    return out


def _schedule_struct(schedule, ndim: int = 2):
    """``syn_schedule`` from a RawSchedule-like object or a tuple of the five ``gen_*`` lists."""
    if hasattr(schedule, "gen_block_offset_lists"):
        parts = (
            schedule.gen_block_offset_lists(),
            schedule.gen_block_shape_lists(),
            schedule.gen_signal_lists(),
            schedule.gen_target_rank_list(),
            schedule.gen_dst_offset_lists(),
        )
    else:
        parts = tuple(_to_list(x) for x in schedule)
        parts = parts + (None,) * (5 - len(parts))
    if parts[0] and isinstance(parts[0][0], (list, tuple)):
        ndim = len(parts[0][0])
    return L.make_schedule(parts[0], parts[1], parts[2], parts[3], parts[4], ndim=ndim)


__all__ = ["gemm", "gemm_mod1d", "ag_gemm", "gemm_rs"]
