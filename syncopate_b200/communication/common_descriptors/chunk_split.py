"""Chunk-size tuning for plans whose lowered schedules drive a kernel.

``DevicePlan.split_xfers`` (syncopate/communication/descriptor.py:718) cuts every transfer by BYTES:
the pieces are flat segment lists, which the copy-engine code generator can execute but which
``lower_comm_plan_to_raw_schedules`` rejects ("inconsistent dimensionality"), in the reference as
here.  A fused kernel needs pieces that are still boxes, so that each piece lowers to one wave with
a flag of its own.  ``split_transfers_along_axis`` therefore cuts every push / pull of a plan into
``num_splits`` boxes along one axis (``BufferRegion.split(n, axis)``,
syncopate/communication/descriptor.py:254-335) and keeps everything else (op kind, peer, reduce
op, what the transfer depends on, local copies, resident regions) as it is.  Call it on every rank's plan before
``CommGenerator.plan_signals``: smaller chunks raise their flags earlier, which shortens the
non-overlapped head and tail of a fused operator at the price of more flags and waves.
"""
from __future__ import annotations

import copy

from ..descriptor import DevicePlan, Transfer, TransferOp


def split_transfers_along_axis(plan: DevicePlan, num_splits: int, axis: int = 0) -> DevicePlan:
    """A copy of ``plan`` in which every push / pull is ``num_splits`` box-shaped pieces along
    ``axis`` (of both its source and its destination region), in order."""
    if num_splits < 1:
        raise ValueError("num_splits must be at least 1")
    streams = []
    for ops in plan.xfer:
        out = []
        for op in ops:
            remote = isinstance(op, Transfer) and op.op in (TransferOp.PUSH, TransferOp.PULL)
            if not remote or num_splits == 1:
                out.append(copy.deepcopy(op))
                continue
            if op.src_region is None or op.dst_region is None:
                raise ValueError("cannot split a transfer with dynamic regions")
            if op.set_signals:
                raise ValueError("split the plan before signals are planned")
            src_parts = op.src_region.split(num_splits, axis)
            dst_parts = op.dst_region.split(num_splits, axis)
            if len(src_parts) != len(dst_parts):
                raise ValueError("source and destination splits differ in count")
            for i, (src, dst) in enumerate(zip(src_parts, dst_parts)):
                out.append(Transfer(op=op.op, src_buf=op.src_buf, src_region=src, dst_buf=op.dst_buf, dst_region=dst,
                                    chunk_idx=op.chunk_idx * num_splits + i, peer=op.peer, reduce_op=op.reduce_op,
                                    dependency=copy.deepcopy(op.dependency)))
        streams.append(out)
    return DevicePlan(dev=plan.dev, xfer=streams, local_regions=copy.deepcopy(plan.local_regions),
                      transit_signals=copy.deepcopy(plan.transit_signals),
                      tensors_involved=copy.deepcopy(plan.tensors_involved))


__all__ = ["split_transfers_along_axis"]
