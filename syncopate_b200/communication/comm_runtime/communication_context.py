"""``CommContext``: symmetric buffers, signal flags and the interpreter of a rank's op program.

Same constructor, attributes and methods as the reference's
syncopate/communication/comm_runtime/communication_context.py (:15-305), on a different substrate:
buffers and flag arrays are CUDA-IPC symmetric allocations (``syncopate_b200.runtime``) instead of
NVSHMEM tensors; copy-engine ops are peer ``cudaMemcpyAsync`` calls; SM copies (plain and reducing)
run on the ``syn_copy`` kernel; flag sets are stream memory operations and flag waits bounded
one-thread kernels (or stream memory operations with ``stream_waits=True``).  Flags carry
``signal_value`` (1 after ``reset_signals``; ``next_epoch()`` raises it so that a loop needs neither
a reset nor a barrier per iteration).

``CommContext(rank, info)`` allocates from the process's symmetric context
(``syncopate_b200.runtime.current_context()``, opened by ``init_from_env``), as the reference
allocates from the process-wide NVSHMEM heap; ``symmetric=`` names another one (tests that emulate
several ranks in one process).

The fused kernels (``syncopate_b200.computation``) move data themselves; ``execute()`` is the
un-fused path: ``CodeGenOptions(copy_engine=True)`` programs, or SM box copies run by ``syn_copy``.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional

import torch

from syncopate_b200 import _lib as L
from syncopate_b200.communication.comm_runtime.operations import (
    CollectiveComm,
    CommInfo,
    CopyEngineOp,
    IntraNodeSignal,
    SMCopyOp,
    WaitIntraNodeSignal,
)
from syncopate_b200.communication.descriptor import CollectiveOp, SignalType
from syncopate_b200.computation.attn.plan import box_copy_ops
from syncopate_b200.runtime import SymmetricTensor, current_context

SIGNAL_DTYPE = torch.int64  # 64-bit flag words (NVSHMEM_SIGNAL_DTYPE in the reference is uint64)
_SYN_DTYPES = {torch.float16: L.SYN_DTYPE_F16, torch.bfloat16: L.SYN_DTYPE_BF16}
_COPY_MAX_OPS = 64  # pieces one syn_copy launch takes


class CommContext:
    """Runtime state of one rank for one ``CommInfo``."""

    def __init__(self, rank: int, info: CommInfo, multi_info: bool = False, *, symmetric=None, timeout_ns: int = 0,
                 stream_waits: bool = False):
        """``stream_waits``: run ``WaitIntraNodeSignal`` as a stream memory operation (needs no SM, so a
        persistent kernel that fills the GPU cannot starve it; it has no time bound of its own, so
        use it only for flags that a bounded kernel raises on every path).  Default: a one-thread
        kernel whose wait is bounded by ``timeout_ns``."""
        if symmetric is None:
            symmetric = current_context()
        if info.local_world_size == 0:
            info.local_world_size = info.world_size
        self.rank = rank
        self.local_rank = rank % info.local_world_size
        self.node_id = rank // info.local_world_size
        self.info = info
        self.symmetric = symmetric
        self.timeout_ns = timeout_ns
        self.stream_waits = stream_waits
        self.signal_value = 1
        extra = 100 if multi_info else 0  # head-room for later infos, as the reference leaves

        def flags(count: int) -> Optional[SymmetricTensor]:
            return symmetric.alloc((count + extra,), SIGNAL_DTYPE) if count > 0 else None

        self._recv = flags(info.recv_signal_num)
        self._transit = flags(info.transit_signal_num)
        self._compute = flags(info.compute_signal_num)
        self.recv_signal_bufs: List[torch.Tensor] = self._recv.peers if self._recv else []
        self.transit_signal_bufs: List[torch.Tensor] = self._transit.peers if self._transit else []
        self.compute_signal_bufs: List[torch.Tensor] = self._compute.peers if self._compute else []
        self._buffers: Dict[str, SymmetricTensor] = {}
        self.comm_buffers: Dict[str, List[torch.Tensor]] = {}
        for name, (shape, dtype) in info.comm_buffer_sizes.items():
            t = symmetric.alloc(tuple(shape), dtype)
            self._buffers[name] = t
            self.comm_buffers[name] = t.peers
        self.streams: List[torch.cuda.Stream] = []
        self.compute_stream: Optional[torch.cuda.Stream] = None
        self._copy_cache: Dict[int, tuple] = {}
        self._make_streams()

    def _make_streams(self) -> None:
        self.streams = [torch.cuda.Stream(device=self.symmetric.device) for _ in range(len(self.info.operations[self.rank]))]
        self.compute_stream = None

    # ---- symmetric tables for the fused kernels
    def symm(self, name: str) -> L.Symm:
        return self._buffers[name].symm

    @property
    def recv_symm(self) -> Optional[L.Symm]:
        return self._recv.symm if self._recv else None

    @property
    def compute_symm(self) -> Optional[L.Symm]:
        return self._compute.symm if self._compute else None

    # ---- flags
    def reset_signals(self):
        """Zeroes this rank's flag arrays (callers then barrier, as with the reference)."""
        for t in (self._recv, self._transit, self._compute):
            if t is not None:
                t.local.fill_(0)
        self.signal_value = 1

    def next_epoch(self) -> int:
        """Flags are compared with ``>=``: raising the value replaces reset + barrier."""
        self.signal_value += 1
        return self.signal_value

    # ---- stream wiring
    def start_after(self, stream: Optional[torch.cuda.Stream] = None):
        stream = stream or torch.cuda.current_stream()
        for s in self.streams:
            s.wait_stream(stream)

    def end_before(self, stream: Optional[torch.cuda.Stream] = None):
        stream = stream or torch.cuda.current_stream()
        for s in self.streams:
            stream.wait_stream(s)

    # ---- interpreter
    def _flag_array(self, kind: SignalType, rank: int) -> torch.Tensor:
        if kind == SignalType.COMPUTE_DONE:
            return self.compute_signal_bufs[rank % self.info.local_world_size]
        if kind == SignalType.RECEIVE_DATA:
            return self.recv_signal_bufs[rank % self.info.local_world_size]
        raise NotImplementedError(f"Signal type {kind} not implemented yet.")

    def _sm_copy(self, op: SMCopyOp, sp) -> None:
        """One ``SMCopyOp`` (an N-D box, optionally reducing) on the SM copy kernel: the box is cut
        into 2-D strided pieces and handed to ``syn_copy``, at most 64 pieces per launch."""
        lib = L.lib()
        status = self.symmetric.status.data_ptr()
        n_sms = self.info.num_copy_sms if getattr(self.info, "num_copy_sms", 0) else 0
        cached = self._copy_cache.get(id(op))
        if cached is not None:  # the program is static: its boxes are cut into pieces once
            for comm, _keep in cached[1]:
                L.check(lib.syn_copy(C.byref(comm), n_sms, self.signal_value, self.timeout_ns, status, sp), "syn_copy")
            return
        src_t, dst_t = self._buffers[op.src], self._buffers[op.dst]
        elem = src_t.dtype.itemsize
        src_off = [a.start for a in op.src_slice]
        dst_off = [a.start for a in op.dst_slice]
        extent_s = [a.end - a.start for a in op.src_slice]
        extent_d = [a.end - a.start for a in op.dst_slice]
        if extent_s != extent_d:
            # same bytes, different box shapes (a reshaping copy): fall back on the flat view of both
            if _numel(extent_s) != _numel(extent_d):
                raise ValueError("source and destination boxes of an SM copy differ in size")
            raise NotImplementedError("SM copies between boxes of different shape are not supported")
        reduce = 0
        if op.reduce_op is not None:
            if src_t.dtype not in _SYN_DTYPES or dst_t.dtype != src_t.dtype:
                raise NotImplementedError("reducing SM copies take fp16 / bf16 buffers of one type")
            reduce = 1
        pieces = box_copy_ops(src_t.shape, src_off, dst_t.shape, dst_off, extent_s, elem)
        launches = []
        self._copy_cache[id(op)] = (op, launches)  # (the op is kept so that its id stays unique)
        for first in range(0, len(pieces), _COPY_MAX_OPS):
            ops = []
            for so, do, rows, row_bytes, spitch, dpitch in pieces[first:first + _COPY_MAX_OPS]:
                c = L.CopyOp()
                c.src_rank, c.dst_rank = op.src_rank % self.info.local_world_size, op.dst_rank % self.info.local_world_size
                c.src_buf, c.dst_buf = 0, 1
                c.src_offset, c.dst_offset = so, do
                c.src_pitch, c.dst_pitch = spitch, dpitch
                c.rows, c.row_bytes = rows, row_bytes
                c.flag_rank, c.flag = 0, -1
                c.reduce = reduce
                c.dtype = _SYN_DTYPES.get(src_t.dtype, 0)
                ops.append(c)
            comm, keep = L.make_attn_comm(ops, [src_t.symm, dst_t.symm], src_t.symm, None)
            launches.append((comm, keep))
            L.check(lib.syn_copy(C.byref(comm), n_sms, self.signal_value, self.timeout_ns, status, sp), "syn_copy")

    def execute(self, neglect_local: bool = False):
        """Issues this rank's op program on the communication streams."""
        lib = L.lib()
        lws = self.info.local_world_size
        status = self.symmetric.status.data_ptr()
        for stream, ops in zip(self.streams, self.info.operations[self.rank]):
            sp = stream.cuda_stream or None
            with torch.cuda.stream(stream):
                for op in ops:
                    if isinstance(op, CopyEngineOp):
                        assert op.src_rank == self.rank or op.dst_rank == self.rank
                        assert op.src_rank // lws == op.dst_rank // lws
                        if neglect_local and op.src_rank == op.dst_rank:
                            continue
                        src = self.comm_buffers[op.src][op.src_rank % lws]
                        dst = self.comm_buffers[op.dst][op.dst_rank % lws]
                        L.check(lib.syn_memcpy_async(dst.data_ptr() + op.dst_offset, src.data_ptr() + op.src_offset,
                                                     op.size, sp), "syn_memcpy_async")
                    elif isinstance(op, IntraNodeSignal):
                        assert op.signal_type == SignalType.RECEIVE_DATA
                        assert op.rank // lws == self.node_id
                        flag = self._flag_array(op.signal_type, op.rank)
                        L.check(lib.syn_flag_set(flag.data_ptr() + 8 * op.offset, self.signal_value, sp), "syn_flag_set")
                    elif isinstance(op, WaitIntraNodeSignal):
                        assert op.rank // lws == self.node_id
                        flag = self._flag_array(op.signal_type, op.rank)
                        if self.stream_waits:
                            L.check(lib.syn_flag_wait_stream(flag.data_ptr() + 8 * op.offset, self.signal_value, sp),
                                    "syn_flag_wait_stream")
                        else:
                            L.check(lib.syn_flag_wait(flag.data_ptr() + 8 * op.offset, self.signal_value,
                                                      self.timeout_ns, status, op.offset, sp), "syn_flag_wait")
                    elif isinstance(op, SMCopyOp):
                        assert op.src_rank == self.rank or op.dst_rank == self.rank
                        if neglect_local and op.src_rank == op.dst_rank:
                            continue
                        self._sm_copy(op, sp)
                    elif isinstance(op, CollectiveComm):
                        self._collective(op)
                    else:  # pragma: no cover
                        raise NotImplementedError(f"unknown op {op}")

    def _collective(self, op: CollectiveComm) -> None:
        import torch.distributed as dist

        src = self.comm_buffers[op.src][self.local_rank][tuple(slice(a.start, a.end) for a in op.src_slice)]
        dst = self.comm_buffers[op.dst][self.local_rank][tuple(slice(a.start, a.end) for a in op.dst_slice)]
        if op.op == CollectiveOp.REDUCE_SCATTER:
            tmp = dst if dst.is_contiguous() else torch.empty_like(dst)
            dist.reduce_scatter_tensor(tmp, src.contiguous())
            if tmp is not dst:
                dst.copy_(tmp)
        elif op.op == CollectiveOp.ALL_REDUCE:
            if op.src != op.dst:
                raise ValueError("NCCL all-reduce currently requires src and dst to be the same buffer.")
            tmp = src if src.is_contiguous() else src.contiguous()
            dist.all_reduce(tmp)
            if tmp is not src:
                dst.copy_(tmp)
        else:
            raise NotImplementedError(f"Collective operation {op.op} not implemented yet.")

    def get_comm_sms(self) -> int:
        return self.info.num_copy_sms

    def get_graph(self) -> torch.cuda.CUDAGraph:
        """Captures start_after / execute / end_before into a CUDA graph for replay.  The flag value
        is captured with the graph: replay it with the same ``signal_value`` (``reset_signals``
        between replays, as the reference's drivers do)."""
        L.lib()  # resolve the library (and its driver entry points) outside the capture
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.start_after(torch.cuda.current_stream())
            self.execute()
            self.end_before(torch.cuda.current_stream())
        return graph

    def update_comm_info(self, info: CommInfo):
        """Switches to another op program over the same buffers."""
        if info.local_world_size == 0:
            info.local_world_size = info.world_size
        self.info = info
        self._copy_cache = {}
        self._make_streams()


def _numel(extent) -> int:
    n = 1
    for e in extent:
        n *= int(e)
    return n
