"""Records of the per-rank communication program produced by the code generator
(cf. syncopate/communication/comm_runtime/operations.py:6-106).  Plain attribute bags: the
generator fills them, the runtime and the fused kernels' host code read them."""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..descriptor import AxisSlice, CollectiveOp, ReduceOp, SignalType


def _show(obj, names) -> str:
    body = ", ".join(f"{n}={getattr(obj, n)}" for n in names)
    return f"{type(obj).__name__}({body})"


class CopyEngineOp:
    """One contiguous byte copy for a DMA engine."""

    src: str
    dst: str
    src_rank: int
    dst_rank: int
    src_offset: int
    dst_offset: int
    size: int

    def __str__(self) -> str:
        return _show(self, ("src_rank", "dst_rank", "src_offset", "dst_offset", "size"))


class SMCopyOp:
    """One N-D box copy (optionally a reduction) executed by SMs."""

    src: str
    dst: str
    src_rank: int
    dst_rank: int
    src_slice: Tuple[AxisSlice, ...]
    dst_slice: Tuple[AxisSlice, ...]
    reduce_op: Optional[ReduceOp] = None
    use_tma: bool = True

    def __str__(self) -> str:
        return _show(self, ("src_rank", "dst_rank", "src_slice", "dst_slice", "reduce_op"))


class CollectiveComm:
    """One library collective over a box of ``src`` into a box of ``dst``."""

    op: CollectiveOp
    src: str
    dst: str
    src_slice: Tuple[AxisSlice, ...]
    dst_slice: Tuple[AxisSlice, ...]

    def __str__(self) -> str:
        return _show(self, ("op", "src", "dst", "src_slice", "dst_slice"))


class IntraNodeSignal:
    """Raise flag ``offset`` of ``rank``'s array for ``signal_type``."""

    signal_type: SignalType
    offset: int
    rank: int

    def __str__(self) -> str:
        return f"IntraNodeSignal(type={self.signal_type}, offset={self.offset}, rank={self.rank})"


class WaitIntraNodeSignal:
    """Wait until flag ``offset`` of ``rank``'s array for ``signal_type`` is raised."""

    signal_type: SignalType
    offset: int
    rank: int

    def __str__(self) -> str:
        return f"WaitIntraNodeSignal(type={self.signal_type}, offset={self.offset}, rank={self.rank})"


class CommInfo:
    """Everything a rank needs to run its communication: flag counts, buffers, op program."""

    world_size: int
    local_world_size: int
    recv_signal_num: int
    transit_signal_num: int
    compute_signal_num: int
    comm_buffer_sizes: Dict[str, Tuple[torch.Size, torch.dtype]]
    operations: List[List[List]]  # [rank][stream][op]
    num_copy_sms: int
    need_green_ctx: bool

    def __init__(self) -> None:
        self.world_size = 0
        self.local_world_size = 0
        self.recv_signal_num = 0
        self.transit_signal_num = 0
        self.comm_buffer_sizes = {}
        self.operations = []
        self.num_copy_sms = 0
        self.need_green_ctx = False

    def __str__(self) -> str:
        out = [
            f"world_size={self.world_size}",
            f"local_world_size={self.local_world_size}",
            f"recv_signal_num={self.recv_signal_num}",
            f"transit_signal_num={self.transit_signal_num}",
            f"compute_signal_num={self.compute_signal_num}",
        ]
        if self.comm_buffer_sizes:
            out.append("comm_buffers:")
            out += [f"  {n}: shape={tuple(s)} dtype={d}" for n, (s, d) in self.comm_buffer_sizes.items()]
        else:
            out.append("comm_buffers: none")
        for rank, streams in enumerate(self.operations):
            out.append(f"rank {rank}:")
            for s, ops in enumerate(streams):
                out.append(f"  stream {s}:")
                out += [f"    {op}" for op in ops]
        return "\n".join(out)
