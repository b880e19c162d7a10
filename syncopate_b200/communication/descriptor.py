"""Communication IR of the front end: buffer regions, transfers, device plans, signal planning.

API-compatible restatement of Syncopate's ``syncopate/communication/descriptor.py`` (class names,
fields, defaults, error types and printed text are the contract; the implementation is this
project's own).  Reference anchors:

* ``BufferRegion`` and its byte-segment view — descriptor.py:61-358
* ``Transfer`` / ``to_memcpys`` — descriptor.py:435-590
* ``DevicePlan`` — descriptor.py:643-745
* ``CommPlan.plan_signals`` — descriptor.py:860-988, ``estimate_period`` — :990-1061

Every list a plan produces (segments, signal offsets, start times) is pinned bit-exact against
the reference by ``tests/test_frontend_parity.py`` and the fixtures in ``tests/golden``.
"""
from __future__ import annotations

import copy
import itertools
from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Dict, Iterable, List, Optional, Sequence, Tuple, Union

import torch


def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


# --------------------------------------------------------------------------- small value types
@dataclass
class Period:
    """Time interval of an operation in abstract units (start is filled by estimate_period)."""

    start: Optional[float] = None
    duration: float = 1.0

    def split(self, num_splits: int) -> "Period":
        assert self.start is None, "Cannot split a Period with known start time."
        if num_splits <= 1:
            return self
        return Period(start=None, duration=self.duration / num_splits)


@dataclass(frozen=True)
class MemorySegment:
    """Contiguous byte span within a logical buffer."""

    offset: int
    nbytes: int

    def __post_init__(self) -> None:
        if self.offset < 0:
            raise ValueError("segment offset must be non-negative")
        if self.nbytes < 0:
            raise ValueError("segment nbytes must be non-negative")

    @property
    def end(self) -> int:
        return self.offset + self.nbytes


@dataclass(frozen=True)
class AxisSlice:
    """Half-open index range along one axis."""

    start: int
    end: int

    def __post_init__(self) -> None:
        if self.start < 0:
            raise ValueError("axis slice start must be non-negative")
        if self.end < self.start:
            raise ValueError("axis slice end must be >= start")

    def length(self) -> int:
        return self.end - self.start


SliceSpec = Union[AxisSlice, slice, Tuple[int, int]]


def _coalesce(sorted_segments: Sequence[MemorySegment]) -> Tuple[MemorySegment, ...]:
    """Joins segments that touch end-to-start (input sorted by offset)."""
    out: List[MemorySegment] = []
    for seg in sorted_segments:
        if out and out[-1].end == seg.offset:
            out[-1] = MemorySegment(out[-1].offset, out[-1].nbytes + seg.nbytes)
        else:
            out.append(seg)
    return tuple(out)


# --------------------------------------------------------------------------- BufferRegion
@dataclass
class BufferRegion:
    """Union of axis-aligned boxes inside a strided buffer, with its byte-segment view."""

    regions: Tuple[Tuple[AxisSlice, ...], ...]
    elem_size: int
    strides: Tuple[int, ...]
    base_offset: int = 0
    _segments: Tuple[MemorySegment, ...] = field(init=False, repr=False)

    def __post_init__(self) -> None:
        if not self.regions:
            raise ValueError("BufferRegion requires at least one region")
        if self.elem_size <= 0:
            raise ValueError("elem_size must be positive")
        if self.base_offset < 0:
            raise ValueError("base_offset must be non-negative")
        rank = len(self.regions[0])
        if len(self.strides) != rank:
            raise ValueError("strides length must match number of axes")
        if any(len(box) != rank for box in self.regions):
            raise ValueError("all regions must have the same number of axes")
        spans: List[MemorySegment] = []
        for box in self.regions:
            spans.extend(self._box_segments(box))
        spans.sort(key=lambda s: s.offset)
        self._segments = _coalesce(spans)

    # ---- constructors
    @classmethod
    def contiguous(cls, offset: int, nbytes: int) -> "BufferRegion":
        return cls.from_segments([(offset, nbytes)])

    @classmethod
    def from_segments(cls, segments: Iterable[Union[MemorySegment, Tuple[int, int]]]) -> "BufferRegion":
        segs = [s if isinstance(s, MemorySegment) else MemorySegment(s[0], s[1]) for s in segments]
        if not segs:
            raise ValueError("from_segments expects at least one segment")
        boxes = tuple((AxisSlice(s.offset, s.end),) for s in segs)
        return cls(regions=boxes, elem_size=1, strides=(1,), base_offset=0)

    @classmethod
    def from_slices(
        cls, *, elem_size: int, strides: Sequence[int], slices: Sequence[SliceSpec], base_offset: int = 0
    ) -> "BufferRegion":
        return cls(
            regions=(cls._normalize_region(slices),),
            elem_size=elem_size,
            strides=tuple(strides),
            base_offset=base_offset,
        )

    @classmethod
    def from_multi_slices(
        cls,
        *,
        elem_size: int,
        strides: Sequence[int],
        regions: Sequence[Sequence[SliceSpec]],
        base_offset: int = 0,
    ) -> "BufferRegion":
        boxes = tuple(cls._normalize_region(r) for r in regions)
        if not boxes:
            raise ValueError("from_multi_slices expects at least one region")
        return cls(regions=boxes, elem_size=elem_size, strides=tuple(strides), base_offset=base_offset)

    @classmethod
    def strided(cls, base_offset: int, segment_bytes: int, stride: int, count: int) -> "BufferRegion":
        if count <= 0:
            raise ValueError("count must be positive for strided region")
        if segment_bytes <= 0:
            raise ValueError("segment_bytes must be positive")
        if stride < 0:
            raise ValueError("stride must be non-negative")
        return cls.from_segments([MemorySegment(base_offset + i * stride, segment_bytes) for i in range(count)])

    @staticmethod
    def _normalize_region(slices: Sequence[SliceSpec]) -> Tuple[AxisSlice, ...]:
        out: List[AxisSlice] = []
        for spec in slices:
            if isinstance(spec, AxisSlice):
                out.append(spec)
            elif isinstance(spec, slice):
                if spec.step not in (None, 1):
                    raise ValueError("slice step other than 1 is not supported")
                if spec.stop is None:
                    raise ValueError("slice stop must be provided")
                out.append(AxisSlice(spec.start or 0, spec.stop))
            else:
                lo, hi = spec
                out.append(AxisSlice(lo, hi))
        return tuple(out)

    # ---- byte view
    def _box_segments(self, box: Tuple[AxisSlice, ...]) -> List[MemorySegment]:
        """Byte runs of one box.

        Trailing axes are folded into one run for as long as an axis' byte stride equals the run
        length accumulated so far; the remaining leading axes are enumerated in row-major order.
        """
        if any(ax.length() == 0 for ax in box):
            return []
        es = self.elem_size
        run = es
        outer = len(box)  # number of leading axes that are enumerated
        while outer > 0 and self.strides[outer - 1] * es == run:
            run *= box[outer - 1].length()
            outer -= 1
        tail = sum(box[i].start * self.strides[i] * es for i in range(outer, len(box)))
        if outer == 0:
            return [MemorySegment(self.base_offset + tail, run)]
        bases = [self.base_offset + tail]
        for i in range(outer):
            step = self.strides[i] * es
            ax = box[i]
            bases = [b + k * step for b in bases for k in range(ax.start, ax.end)]
        return [MemorySegment(b, run) for b in bases]

    def to_segments(self) -> Tuple[MemorySegment, ...]:
        return self._segments

    def total_nbytes(self) -> int:
        return sum(s.nbytes for s in self._segments)

    def is_contiguous(self) -> bool:
        return len(self._segments) == 1

    def as_slice(self) -> Optional[slice]:
        flat = (
            len(self.regions) == 1
            and len(self.regions[0]) == 1
            and self.strides == (1,)
            and self.elem_size == 1
            and self.base_offset == 0
        )
        if not flat:
            return None
        ax = self.regions[0][0]
        return slice(ax.start, ax.end)

    # ---- splitting
    def split(self, num_splits: int, axis: Optional[int] = None) -> List["BufferRegion"]:
        if num_splits <= 1:
            return [self]
        return self._split_by_bytes(num_splits) if axis is None else self._split_along_axis(num_splits, axis)

    def _split_by_bytes(self, num_splits: int) -> List["BufferRegion"]:
        total = self.total_nbytes()
        if total == 0:
            return [self]
        quota = _ceil_div(total, num_splits)
        parts: List[BufferRegion] = []
        pending = deque((s.offset, s.nbytes) for s in self._segments)
        left = total
        for _ in range(num_splits):
            want = min(quota, left)
            if want <= 0:
                break
            taken: List[MemorySegment] = []
            while want > 0:
                if not pending:
                    raise RuntimeError("not enough data to satisfy split request")
                off, n = pending.popleft()
                use = min(want, n)
                taken.append(MemorySegment(off, use))
                if use < n:
                    pending.appendleft((off + use, n - use))
                want -= use
                left -= use
            parts.append(BufferRegion.from_segments(taken))
        return parts

    def _split_along_axis(self, num_splits: int, axis: int) -> List["BufferRegion"]:
        if not self.regions:
            return [self]
        rank = len(self.strides)
        if axis < 0:
            axis += rank
        if not 0 <= axis < rank:
            raise IndexError(f"axis {axis} out of range for BufferRegion with {rank} dims")
        if len(self.regions) != 1:
            raise NotImplementedError(
                "Axis-aligned splitting currently supports regions with a single contiguous block"
            )
        box = self.regions[0]
        span = box[axis]
        if span.length() == 0:
            return [self]
        step = _ceil_div(span.length(), num_splits)
        if step <= 0:
            return [self]
        parts: List[BufferRegion] = []
        lo = span.start
        while lo < span.end and len(parts) < num_splits:
            hi = min(span.end, lo + step)
            piece = box[:axis] + (AxisSlice(lo, hi),) + box[axis + 1 :]
            parts.append(
                BufferRegion(
                    regions=(piece,), elem_size=self.elem_size, strides=self.strides, base_offset=self.base_offset
                )
            )
            lo = hi
        return parts or [self]

    def describe(self) -> str:
        def one(box: Tuple[AxisSlice, ...]) -> str:
            return "[" + ", ".join(f"{a.start}:{a.end}" for a in box) + "]" if box else "[]"

        if len(self.regions) == 1:
            return one(self.regions[0])
        return "{" + ", ".join(one(b) for b in self.regions) + "}"


# --------------------------------------------------------------------------- high-level descriptor
@dataclass
class DataPlacement:
    """Where one datum lives (rank and, optionally, region)."""

    rank: int
    region: Optional[BufferRegion] = None


@dataclass
class CommDescriptor:
    """Placement of data before and after a collective; carries no scheduling."""

    data_info: dict[int, Optional[int]]
    before_placement: dict[int, DataPlacement]
    after_placement: dict[int, DataPlacement]


# --------------------------------------------------------------------------- transfers and signals
class TransferOp(Enum):
    PUSH = "push"
    PULL = "pull"
    LOCAL_COPY = "local_copy"


class SignalType(Enum):
    RECEIVE_DATA = "receive_data"
    COMPUTE_DONE = "compute_done"
    REMOTE_DATA_READY = "remote_data_ready"


class ReduceOp(Enum):
    SUM = 1
    MAX = 2


class CollectiveOp(Enum):
    REDUCE_SCATTER = "reduce_scatter"
    ALL_REDUCE = "all_reduce"
    ALL_GATHER = "all_gather"
    ALL_REDUCE_NVSHARP = "all_reduce_nvsharp"


@dataclass
class Signal:
    """Flag raised when an operation completes: slot ``dst_offset`` of ``dst_rank``'s flag array."""

    dst_rank: int
    dst_offset: int
    type: SignalType
    period: Period = field(default_factory=Period)


@dataclass
class XferDependency:
    """This op may start only after op ``(depend_rank, depend_xfer_stream, depend_xfer_idx)`` is done."""

    depend_rank: int
    depend_xfer_stream: int
    depend_xfer_idx: int
    signal: Optional[Signal] = None


@dataclass
class ComputeDependency:
    """This op may start only after compute on ``compute_rank`` has produced ``src_region``."""

    compute_rank: int
    src_region: Optional[BufferRegion]
    signal: Optional[Signal] = None

    def __post_init__(self):
        if self.signal is not None:
            assert self.signal.type == SignalType.COMPUTE_DONE


Dependency = Union[XferDependency, ComputeDependency]


@dataclass
class Transfer:
    """One push / pull / local copy between (possibly strided) regions."""

    op: TransferOp
    src_buf: str
    src_region: Optional[BufferRegion]
    dst_buf: str
    dst_region: Optional[BufferRegion]
    chunk_idx: int
    dependency: List[Dependency] = field(default_factory=list)
    set_signals: List[Signal] = field(default_factory=list)
    peer: Optional[int] = None
    period: Period = field(default_factory=Period)
    reduce_op: Optional[ReduceOp] = None

    def __post_init__(self):
        if self.op in (TransferOp.PULL, TransferOp.PUSH):
            assert self.peer is not None
        else:
            assert self.peer is None

    def _both_single_run(self) -> bool:
        return (
            self.src_region is not None
            and self.dst_region is not None
            and self.src_region.is_contiguous()
            and self.dst_region.is_contiguous()
        )

    @property
    def nbytes(self) -> Optional[int]:
        if not self._both_single_run():
            return None
        n_src, n_dst = self.src_region.total_nbytes(), self.dst_region.total_nbytes()
        if n_src != n_dst:
            raise ValueError("source and destination regions disagree on total bytes")
        return n_src

    @property
    def src_off(self) -> Optional[int]:
        if self.src_region and self.src_region.is_contiguous():
            return self.src_region.to_segments()[0].offset
        return None

    @property
    def dst_off(self) -> Optional[int]:
        if self.dst_region and self.dst_region.is_contiguous():
            return self.dst_region.to_segments()[0].offset
        return None

    def split(self, num_splits: int) -> List["Transfer"]:
        if num_splits <= 1:
            return [self]
        if self.src_region is None or self.dst_region is None:
            raise ValueError("Cannot split a Transfer with dynamic regions.")
        src_parts = self.src_region.split(num_splits)
        dst_parts = self.dst_region.split(num_splits)
        if len(src_parts) != len(dst_parts):
            raise ValueError("Source and destination splits differ in count")
        self.period.split(num_splits)  # validates that the start time is still unknown
        pieces: List[Transfer] = []
        for i, (s, d) in enumerate(zip(src_parts, dst_parts)):
            assert len(self.dependency) == 0
            assert len(self.set_signals) == 0
            pieces.append(
                Transfer(
                    op=self.op,
                    src_buf=self.src_buf,
                    src_region=s,
                    dst_buf=self.dst_buf,
                    dst_region=d,
                    chunk_idx=self.chunk_idx * num_splits + i,
                    dependency=copy.deepcopy(self.dependency),
                    peer=self.peer,
                    set_signals=copy.deepcopy(self.set_signals),
                )
            )
        return pieces

    def to_memcpys(self) -> List[Tuple[int, int, int]]:
        """``(src_offset, dst_offset, nbytes)`` spans that move the source bytes, in order, into
        the destination bytes, in order; spans adjacent on both sides are joined."""
        if self.src_region is None or self.dst_region is None:
            raise ValueError("Cannot materialize memcpy plan for dynamic regions.")
        src = self.src_region.to_segments()
        dst = self.dst_region.to_segments()
        if not src or not dst:
            return []
        if len(src) == 1 and len(dst) == 1:
            if src[0].nbytes != dst[0].nbytes:
                raise ValueError("Source and destination byte counts differ.")
            return [(src[0].offset, dst[0].offset, src[0].nbytes)] if src[0].nbytes else []
        if sum(s.nbytes for s in src) != sum(s.nbytes for s in dst):
            raise ValueError("Source and destination regions disagree on total bytes.")
        if sum(s.nbytes for s in src) == 0:
            return []

        spans: List[Tuple[int, int, int]] = []
        si = di = 0
        s_pos, s_left = src[0].offset, src[0].nbytes
        d_pos, d_left = dst[0].offset, dst[0].nbytes
        while True:
            step = min(s_left, d_left)
            if step == 0:
                raise RuntimeError("Encountered zero-length segment while constructing memcpy plan.")
            if spans and spans[-1][0] + spans[-1][2] == s_pos and spans[-1][1] + spans[-1][2] == d_pos:
                spans[-1] = (spans[-1][0], spans[-1][1], spans[-1][2] + step)
            else:
                spans.append((s_pos, d_pos, step))
            s_pos += step
            d_pos += step
            s_left -= step
            d_left -= step
            if s_left == 0:
                si += 1
                if si == len(src):
                    if d_left != 0 or di != len(dst) - 1:
                        raise ValueError("Destination segments have remaining bytes after source exhausted.")
                    break
                s_pos, s_left = src[si].offset, src[si].nbytes
            if d_left == 0:
                di += 1
                if di == len(dst):
                    if s_left != 0 or si != len(src) - 1:
                        raise ValueError("Source segments have remaining bytes after destination exhausted.")
                    break
                d_pos, d_left = dst[di].offset, dst[di].nbytes
        return spans


@dataclass
class Collective:
    """A library collective (reduce-scatter / all-reduce / all-gather) over regions."""

    op: CollectiveOp
    src_buf: str
    src_region: Optional[BufferRegion]
    dst_buf: str
    dst_region: Optional[BufferRegion]
    dependency: List[Dependency] = field(default_factory=list)
    set_signals: List[Signal] = field(default_factory=list)
    period: Period = field(default_factory=Period)

    def split(self, num_splits: int) -> List["Collective"]:
        if num_splits <= 1:
            return [self]
        if self.src_region is None or self.dst_region is None:
            raise ValueError("Cannot split a Collective with dynamic regions.")
        src_parts = self.src_region.split(num_splits)
        dst_parts = self.dst_region.split(num_splits)
        if len(src_parts) != len(dst_parts):
            raise ValueError("Source and destination splits differ in count")
        shorter = self.period.split(num_splits)
        pieces: List[Collective] = []
        for s, d in zip(src_parts, dst_parts):
            assert len(self.dependency) == 0
            assert len(self.set_signals) == 0
            pieces.append(
                Collective(
                    op=self.op,
                    src_buf=self.src_buf,
                    src_region=s,
                    dst_buf=self.dst_buf,
                    dst_region=d,
                    dependency=copy.deepcopy(self.dependency),
                    set_signals=copy.deepcopy(self.set_signals),
                    period=shorter,
                )
            )
        return pieces


CommOp = Transfer | Collective


# --------------------------------------------------------------------------- DevicePlan
def _fmt_region(name: str, region: Optional[BufferRegion]) -> str:
    return f"{name}[?]" if region is None else f"{name}{region.describe()}"


def _fmt_signal(sig: Signal) -> str:
    return f"{sig.type.value}@{sig.dst_rank}[{sig.dst_offset}]"


def _fmt_op(op) -> str:
    if isinstance(op, Transfer):
        arrow = f"{_fmt_region(op.src_buf, op.src_region)} -> {_fmt_region(op.dst_buf, op.dst_region)}"
        if op.op == TransferOp.LOCAL_COPY:
            return "copy " + arrow
        peer = "?" if op.peer is None else op.peer
        return f"{op.op.value} peer={peer} {arrow}"
    if isinstance(op, Collective):
        return (
            f"collective {op.op.value} {_fmt_region(op.src_buf, op.src_region)} -> "
            f"{_fmt_region(op.dst_buf, op.dst_region)}"
        )
    return f"unknown op {op}"  # pragma: no cover


@dataclass
class DevicePlan:
    """Per-rank program: one op list per stream, plus what is resident before anything runs."""

    dev: int
    xfer: List[List[CommOp]] = field(default_factory=list)
    local_regions: Dict[str, List[BufferRegion]] = field(default_factory=dict)
    # (signal that arrives here, signal to forward): a push A->B that a third rank C waits on is
    # relayed by B, because only the destination of a push is guaranteed to see it complete.
    transit_signals: List[Tuple[Signal, Signal]] = field(default_factory=list)
    tensors_involved: Dict[str, Tuple[torch.Size, torch.dtype]] = field(default_factory=dict)

    def __post_init__(self) -> None:
        if not self.xfer:
            self.xfer.append([])

    def _ensure_stream(self, idx: int) -> List[CommOp]:
        if idx < 0:
            raise ValueError("stream index must be non-negative")
        while len(self.xfer) <= idx:
            self.xfer.append([])
        return self.xfer[idx]

    def add_op(self, op: CommOp, *, stream_idx: int = 0) -> None:
        self._ensure_stream(stream_idx).append(op)

    def add_stream(self) -> int:
        self.xfer.append([])
        return len(self.xfer) - 1

    def _transfers(self, kinds: Tuple[TransferOp, ...]) -> List[Transfer]:
        return [op for ops in self.xfer for op in ops if isinstance(op, Transfer) and op.op in kinds]

    @property
    def xfers(self) -> List[Transfer]:
        return self._transfers((TransferOp.PUSH, TransferOp.PULL))

    @property
    def local_copies(self) -> List[Transfer]:
        return self._transfers((TransferOp.LOCAL_COPY,))

    def pretty(self) -> str:
        out = [f"DevicePlan(dev={self.dev})"]
        for s, ops in enumerate(self.xfer):
            out.append(f"  Stream {s}:")
            if not ops:
                out.append("    (none)")
            for i, op in enumerate(ops):
                out.append(f"    [{i}] {_fmt_op(op)}")
        return "\n".join(out)

    def __str__(self) -> str:  # pragma: no cover
        return self.pretty()

    def split_xfers(self, num_splits: int) -> "DevicePlan":
        streams: List[List[CommOp]] = []
        for ops in self.xfer:
            expanded: List[CommOp] = []
            for op in ops:
                splittable = isinstance(op, Collective) or (
                    isinstance(op, Transfer) and op.op in (TransferOp.PUSH, TransferOp.PULL)
                )
                if splittable:
                    expanded.extend(op.split(num_splits))
                else:
                    expanded.append(copy.deepcopy(op))
            streams.append(expanded)
        return DevicePlan(
            dev=self.dev,
            xfer=streams,
            local_regions=copy.deepcopy(self.local_regions),
            transit_signals=copy.deepcopy(self.transit_signals),
            tensors_involved=copy.deepcopy(self.tensors_involved),
        )

    def check_no_dependency(self) -> bool:
        for ops in self.xfer:
            for op in ops:
                remote = isinstance(op, Transfer) and op.op in (TransferOp.PUSH, TransferOp.PULL)
                if (remote or isinstance(op, Collective)) and op.dependency is not None:
                    return False
        return True


# --------------------------------------------------------------------------- CommPlan
class _Counter:
    """Next free slot per device for one flag array."""

    def __init__(self, table: Dict[int, int]):
        self.table = table

    def take(self, dev: int) -> int:
        if dev not in self.table:
            raise ValueError(f"device {dev} not in signal counter")
        slot = self.table[dev]
        self.table[dev] = slot + 1
        return slot


@dataclass
class CommPlan:
    """All ranks' device plans plus signal planning and start-time estimation."""

    device_plans: dict[int, DevicePlan] = field(default_factory=dict)
    receive_signal_counters: dict[int, int] = field(default_factory=dict)
    transit_signal_counters: dict[int, int] = field(default_factory=dict)
    compute_signal_counters: dict[int, int] = field(default_factory=dict)

    def __init__(self, device_plans: Optional[dict[int, DevicePlan]] = None) -> None:
        self.device_plans = device_plans or {}
        self.receive_signal_counters = {d: 0 for d in self.device_plans}
        self.transit_signal_counters = {d: 0 for d in self.device_plans}
        self.compute_signal_counters = {d: 0 for d in self.device_plans}

    def add_device_plan(self, plan: DevicePlan) -> None:
        if plan.dev in self.device_plans:
            raise ValueError(f"device plan for dev {plan.dev} already exists")
        self.device_plans[plan.dev] = plan

    @property
    def xfers(self) -> List[Transfer]:
        return [t for plan in self.device_plans.values() for t in plan.xfers]

    def _walk(self):
        """(dev, plan, stream_idx, op_idx, op) in planning order."""
        for dev, plan in self.device_plans.items():
            for s, ops in enumerate(plan.xfer):
                for i, op in enumerate(ops):
                    yield dev, plan, s, i, op

    # ---- text
    def pretty(self, include_signals: bool = False) -> str:
        out = [f"CommPlan(devices={len(self.device_plans)})"]
        for dev in sorted(self.device_plans):
            plan = self.device_plans[dev]
            out.extend("  " + line for line in plan.pretty().splitlines())
            if include_signals:
                out.extend(self._format_signal_details(plan))
        return "\n".join(out)

    def visualize_signals(self) -> str:
        out = ["CommPlan Signals:"]
        for dev in sorted(self.device_plans):
            out.append(f"  Device {dev}:")
            out.extend(self._format_signal_details(self.device_plans[dev]) or ["    (no signal activity)"])
        return "\n".join(out)

    def _format_signal_details(self, dev_plan: DevicePlan) -> List[str]:
        out: List[str] = []
        for s, ops in enumerate(dev_plan.xfer):
            if not ops:
                out.append(f"    Stream {s}: (none)")
                continue
            out.append(f"    Stream {s}:")
            for i, op in enumerate(ops):
                raised = ", ".join(_fmt_signal(sig) for sig in op.set_signals) or "(none)"
                out.append(f"      op[{i}] {op.op.value} -> signals: {raised}")
                for k, dep in enumerate(op.dependency or []):
                    planned = _fmt_signal(dep.signal) if dep.signal is not None else "pending"
                    if isinstance(dep, XferDependency):
                        src = f"xfer({dep.depend_rank},{dep.depend_xfer_stream},{dep.depend_xfer_idx})"
                        out.append(f"        dep[{k}] <- {src} -> {planned}")
                    elif isinstance(dep, ComputeDependency):
                        out.append(f"        dep[{k}] <- compute({dep.compute_rank}) -> {planned}")
        if dev_plan.transit_signals:
            out.append("    Transit signals:")
            for arriving, forwarded in dev_plan.transit_signals:
                out.append(f"      {_fmt_signal(arriving)} -> {_fmt_signal(forwarded)}")
        return out

    # ---- signals
    def _check_compute_dependency_signals_set(self, plan_compute_signals: bool) -> bool:
        for _dev, _plan, _s, _i, op in self._walk():
            for dep in op.dependency:
                if isinstance(dep, ComputeDependency):
                    if plan_compute_signals and dep.signal is not None:
                        return False
                    if not plan_compute_signals and dep.signal is None:
                        return False
        return True

    def plan_signals(self, plan_compute_signals=True):
        """Assigns a flag slot to every completion and to every dependency.

        Pass 1: each op raises one RECEIVE_DATA flag — on the peer for a push, on the issuing rank
        otherwise — taking that rank's next receive slot.  Pass 2: each dependency is bound to a
        flag: the producer's own receive flag when the waiting rank can see it, otherwise a new
        transit flag (push to a third rank, relayed by the push target) or an extra
        REMOTE_DATA_READY flag (pull / local copy on another rank); compute dependencies get the
        waiting rank's next compute slot when ``plan_compute_signals`` is set.
        """
        plans = self.device_plans
        assert all(p.transit_signals == [] for p in plans.values()), (
            "transit_signals should be empty before planning signals"
        )
        assert all(op.set_signals == [] for *_x, op in self._walk()), (
            "set_signals should be empty before planning signals"
        )
        assert self._check_compute_dependency_signals_set(plan_compute_signals), (
            "if plan_compute_signals is True, compute dependency signals should be None before planning; "
            "if False, they should be already set"
        )
        recv = _Counter(self.receive_signal_counters)
        transit = _Counter(self.transit_signal_counters)
        compute = _Counter(self.compute_signal_counters)

        for dev, _plan, _s, _i, op in self._walk():
            owner = dev
            if isinstance(op, Transfer) and op.op == TransferOp.PUSH:
                assert op.peer is not None
                owner = op.peer
            slot = recv.take(owner)
            op.set_signals.append(Signal(dst_rank=owner, dst_offset=slot, type=SignalType.RECEIVE_DATA))

        for dev, _plan, _s, _i, op in self._walk():
            for dep in op.dependency:
                if isinstance(dep, XferDependency):
                    if isinstance(op, Collective):
                        raise ValueError("Collective operations cannot have XferDependency for now")
                    upstream_plan = plans.get(dep.depend_rank, None)
                    assert upstream_plan is not None, f"depend_rank {dep.depend_rank} not found in device_plans"
                    upstream = upstream_plan.xfer[dep.depend_xfer_stream][dep.depend_xfer_idx]
                    if not isinstance(upstream, Transfer):
                        raise ValueError("XferDependency can only depend on Collective operations for now")
                    if upstream.op == TransferOp.PUSH:
                        if dev == upstream.peer:
                            assert upstream.set_signals[0].type == SignalType.RECEIVE_DATA
                            dep.signal = upstream.set_signals[0]
                        else:
                            assert upstream.peer is not None
                            relay = Signal(
                                dst_rank=dev, dst_offset=transit.take(dev), type=SignalType.REMOTE_DATA_READY
                            )
                            plans[upstream.peer].transit_signals.append((upstream.set_signals[0], relay))
                            dep.signal = relay
                    elif dev == dep.depend_rank:
                        assert upstream.set_signals[0].type == SignalType.RECEIVE_DATA
                        dep.signal = upstream.set_signals[0]
                    else:
                        extra = Signal(dst_rank=dev, dst_offset=recv.take(dev), type=SignalType.REMOTE_DATA_READY)
                        upstream.set_signals.append(extra)
                        dep.signal = extra
                elif isinstance(dep, ComputeDependency):
                    if plan_compute_signals:
                        dep.signal = Signal(
                            dst_rank=dep.compute_rank, dst_offset=compute.take(dev), type=SignalType.COMPUTE_DONE
                        )
                else:
                    raise ValueError(f"unknown dependency type: {type(dep)}")

    # ---- timing
    def estimate_period(self):
        """Earliest start of every op: longest path over in-stream order and transfer
        dependencies (compute dependencies are ignored), each op lasting ``period.duration``."""
        index: Dict[Tuple[int, int, int], int] = {}
        nodes: List[CommOp] = []
        for dev, _plan, s, i, op in self._walk():
            index[(dev, s, i)] = len(nodes)
            nodes.append(op)
        if not nodes:
            return
        parents: List[set] = [set() for _ in nodes]
        children: List[List[int]] = [[] for _ in nodes]

        def link(parent: int, child: int) -> None:
            if parent not in parents[child]:
                parents[child].add(parent)
                children[parent].append(child)

        for (dev, s, i), node in index.items():
            if i > 0:
                link(index[(dev, s, i - 1)], node)
        for dev, _plan, s, i, op in self._walk():
            for dep in op.dependency:
                if not isinstance(dep, XferDependency):
                    continue
                key = (dep.depend_rank, dep.depend_xfer_stream, dep.depend_xfer_idx)
                if key not in index:
                    raise ValueError(f"dependency target {key} not found in communication plan")
                link(index[key], index[(dev, s, i)])

        waiting = [len(p) for p in parents]
        earliest = [0.0] * len(nodes)
        ready = deque(n for n, w in enumerate(waiting) if w == 0)
        done = 0
        while ready:
            n = ready.popleft()
            done += 1
            op = nodes[n]
            op.period.start = earliest[n]
            finish = earliest[n] + op.period.duration
            for sig in op.set_signals:
                sig.period.start = finish
            for c in children[n]:
                waiting[c] -= 1
                earliest[c] = max(earliest[c], finish)
                if waiting[c] == 0:
                    ready.append(c)
        if done != len(nodes):
            raise RuntimeError("cycle detected in transfer dependencies")


__all__ = [
    "CommPlan",
    "DevicePlan",
    "Transfer",
    "TransferOp",
    "Collective",
    "CollectiveOp",
    "CommOp",
    "Signal",
    "CommDescriptor",
    "DataPlacement",
    "XferDependency",
    "MemorySegment",
    "BufferRegion",
    "AxisSlice",
]
