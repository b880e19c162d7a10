"""Host logic that joins the front end's outputs (CommInfo op program + lowered RawSchedules) into
the per-wave arguments of the fused GEMM kernels."""
from __future__ import annotations

from typing import Dict, List, Sequence


def push_completion_signals(comm_info, rank: int) -> Dict[int, List[int]]:
    """For the op program of ``rank``: first-axis start of every pushed / copied source box ->
    ``[dst_rank, flag index raised on dst_rank]``, read off the copy op and the signal ops that
    follow it (the order ``generate_code_for_plan`` emits: waits, body, signals)."""
    out: Dict[int, List[int]] = {}
    for stream in comm_info.operations[rank]:
        pending = None
        for op in stream:
            kind = type(op).__name__
            if kind == "SMCopyOp":
                pending = (op.src_slice[0].start, op.dst_rank)
            elif kind == "CopyEngineOp":
                if pending is None or pending[1] != op.dst_rank or pending[2:] != ("ce",):
                    pending = (op.src_offset, op.dst_rank, "ce")
            elif kind == "IntraNodeSignal" and pending is not None:
                if op.rank == pending[1] and pending[0] not in out:
                    out[pending[0]] = [op.rank, op.offset]
                pending = None
            elif kind == "WaitIntraNodeSignal":
                pending = None
    return out


def rs_remote_signals(comm_info, rank: int, src_schedule) -> List[int]:
    """Per wave of the partial-C schedule: the flag index to raise on the wave's target rank
    (-1 for the wave kept locally)."""
    table = push_completion_signals(comm_info, rank)
    offsets = src_schedule.gen_block_offset_lists()
    targets = src_schedule.gen_target_rank_list()
    out = []
    for off, tgt in zip(offsets, targets):
        hit = table.get(off[0])
        if tgt < 0 or tgt == rank or hit is None or hit[0] != tgt:
            out.append(-1)
        else:
            out.append(hit[1])
    return out


__all__ = ["push_completion_signals", "rs_remote_signals"]
