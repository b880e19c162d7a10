"""Code generator: a signal-planned CommPlan -> per-rank op programs (``CommInfo``).

Same classes and outputs as syncopate/communication/code_gen.py (``CodeGenOptions`` :7-30,
``CommGenerator.generate_code_for_plan`` :36-181, buffer table :184-199).  For each op, in order:
one wait per dependency, then the body (one ``CollectiveComm`` per box pair, or one
``CopyEngineOp`` per contiguous span, or one ``SMCopyOp`` per box pair), then one signal per
planned completion flag.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple

from .comm_runtime.operations import (
    CollectiveComm,
    CommInfo,
    CopyEngineOp,
    IntraNodeSignal,
    SMCopyOp,
    WaitIntraNodeSignal,
)
from .descriptor import (
    AxisSlice,
    BufferRegion,
    Collective,
    CollectiveOp,
    CommPlan,
    ComputeDependency,
    SignalType,
    Transfer,
    TransferOp,
    XferDependency,
)


@dataclass
class CodeGenOptions:
    copy_engine: bool = True
    low_latency: bool = False
    use_tma: bool = True
    fuse_with_compute_intra: bool = False
    fuse_with_compute_inter: bool = False

    def __init__(
        self,
        copy_engine: bool = True,
        low_latency: bool = False,
        use_tma: bool = True,
        fuse_with_compute_intra: bool = False,
        fuse_with_compute_inter: bool = False,
    ):
        self.copy_engine = copy_engine
        self.low_latency = low_latency
        self.use_tma = use_tma
        self.fuse_with_compute_intra = fuse_with_compute_intra
        self.fuse_with_compute_inter = fuse_with_compute_inter

    def validate(self):
        if self.low_latency:
            raise NotImplementedError("low_latency codegen is not implemented yet")
        if self.copy_engine and self.fuse_with_compute_intra:
            raise ValueError("copy_engine and fuse_with_compute_intra cannot be both enabled")
        if self.fuse_with_compute_inter and not self.fuse_with_compute_intra:
            raise ValueError("fuse_with_compute_inter requires fuse_with_compute_intra to be enabled")


def _boxes_in_buffer_coords(region: BufferRegion, purpose: str) -> List[Tuple[AxisSlice, ...]]:
    """Boxes of ``region`` with its byte ``base_offset`` folded back into per-axis index shifts."""
    shifts = [0] * len(region.strides)
    if region.base_offset != 0:
        if region.base_offset % region.elem_size != 0:
            raise ValueError("base_offset must align with elem_size for TMA copy")
        rest = region.base_offset // region.elem_size
        for i, stride in enumerate(region.strides):
            shifts[i], rest = divmod(rest, stride)
        if rest != 0:
            raise ValueError("base_offset not representable by strides for TMA copy")
    return [tuple(AxisSlice(a.start + shifts[i], a.end + shifts[i]) for i, a in enumerate(box)) for box in region.regions]


def _endpoints(transfer: Transfer, dev: int) -> Tuple[int, int]:
    """(src_rank, dst_rank) of a transfer issued by ``dev``."""
    if transfer.op == TransferOp.LOCAL_COPY:
        return dev, dev
    assert transfer.peer is not None
    return (dev, transfer.peer) if transfer.op == TransferOp.PUSH else (transfer.peer, dev)


class CommGenerator(CommPlan):
    """Turns the plan into op programs for the B200 runtime (peer-mapped buffers + flags)."""

    options: CodeGenOptions

    def generate_code_for_plan(self, options: CodeGenOptions = CodeGenOptions()) -> CommInfo:
        options.validate()
        info = CommInfo()
        info.world_size = len(self.device_plans)
        (info.recv_signal_num, info.transit_signal_num, info.compute_signal_num, info.comm_buffer_sizes) = (
            self._get_buffer_info()
        )
        for dev, dev_plan in self.device_plans.items():
            info.operations.append([])
            for ops in dev_plan.xfer:
                program: List = []
                info.operations[dev].append(program)
                for op in ops:
                    program.extend(self._waits_for(op))
                    if isinstance(op, Collective):
                        program.extend(self._collective_body(op))
                    elif isinstance(op, Transfer):
                        program.extend(self._transfer_body(op, dev_plan.dev, options))
                    for sig in op.set_signals:
                        # intra-node only: a plain flag write on the destination rank
                        assert sig.type == SignalType.RECEIVE_DATA
                        raise_op = IntraNodeSignal()
                        raise_op.signal_type = sig.type
                        raise_op.offset = sig.dst_offset
                        raise_op.rank = sig.dst_rank
                        program.append(raise_op)
        return info

    @staticmethod
    def _waits_for(op) -> List[WaitIntraNodeSignal]:
        waits = []
        for dep in op.dependency:
            if isinstance(dep, ComputeDependency):
                assert dep.signal is not None
                kind = SignalType.COMPUTE_DONE
            elif isinstance(dep, XferDependency):
                if dep.signal is None:
                    raise ValueError("XferDependency requires planned signals before codegen")
                kind = dep.signal.type
            else:
                raise NotImplementedError("dependency handling is not implemented yet")
            w = WaitIntraNodeSignal()
            w.signal_type = kind
            w.offset = dep.signal.dst_offset
            w.rank = dep.signal.dst_rank
            waits.append(w)
        return waits

    @staticmethod
    def _collective_body(op: Collective) -> List[CollectiveComm]:
        if op.src_region is None or op.dst_region is None:
            raise ValueError("Collective requires materialized regions.")
        if op.op == CollectiveOp.ALL_REDUCE and op.src_buf != op.dst_buf:
            raise ValueError("ALL_REDUCE must use the same buffer for src and dst.")
        src_boxes = _boxes_in_buffer_coords(op.src_region, "collective")
        dst_boxes = _boxes_in_buffer_coords(op.dst_region, "collective")
        if len(src_boxes) != len(dst_boxes):
            raise ValueError("source and destination region counts differ for collective")
        body = []
        for s, d in zip(src_boxes, dst_boxes):
            c = CollectiveComm()
            c.op, c.src, c.dst, c.src_slice, c.dst_slice = op.op, op.src_buf, op.dst_buf, s, d
            body.append(c)
        return body

    @staticmethod
    def _transfer_body(op: Transfer, dev: int, options: CodeGenOptions) -> List:
        src_rank, dst_rank = _endpoints(op, dev)
        body: List = []
        if options.copy_engine:
            if op.reduce_op is not None:
                raise ValueError("Copy engine transfer cannot do reduction.")
            for src_off, dst_off, nbytes in op.to_memcpys():
                c = CopyEngineOp()
                c.src_rank, c.dst_rank = src_rank, dst_rank
                c.src, c.dst = op.src_buf, op.dst_buf
                c.src_offset, c.dst_offset, c.size = src_off, dst_off, nbytes
                body.append(c)
            return body
        assert op.src_region is not None and op.dst_region is not None
        src_boxes = _boxes_in_buffer_coords(op.src_region, "copy")
        dst_boxes = _boxes_in_buffer_coords(op.dst_region, "copy")
        if len(src_boxes) != len(dst_boxes):
            raise ValueError("source and destination region counts differ for TMA copy")
        for s, d in zip(src_boxes, dst_boxes):
            c = SMCopyOp()
            c.use_tma = options.use_tma
            c.src_rank, c.dst_rank = src_rank, dst_rank
            c.src, c.dst = op.src_buf, op.dst_buf
            c.src_slice, c.dst_slice = s, d
            c.reduce_op = op.reduce_op
            body.append(c)
        return body

    def _get_buffer_info(self) -> Tuple[int, int, int, dict]:
        """Flag-array sizes (largest per-device counter) and the merged buffer table."""

        def peak(table) -> int:
            return max(table.values()) if table else 0

        buffers: dict = {}
        for dev_plan in self.device_plans.values():
            for name, (size, dtype) in dev_plan.tensors_involved.items():
                if name not in buffers:
                    buffers[name] = (size, dtype)
                elif buffers[name] != (size, dtype):
                    raise ValueError(f"Buffer {name} has inconsistent size or dtype across devices.")
        return (
            peak(self.receive_signal_counters),
            peak(self.transit_signal_counters),
            peak(self.compute_signal_counters),
            buffers,
        )

    def _generate_nic_code(self):
        """Inter-node transfers are out of scope (single NVSwitch box)."""
        pass
