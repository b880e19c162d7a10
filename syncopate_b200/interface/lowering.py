"""Lowering: a signal-planned communication plan -> per-rank, per-buffer wave schedules.

Restates ``lower_comm_plan_to_raw_schedules`` of syncopate/interface/lowering.py:91-331 (touch
rules :334-419, signal lookup :428-440, box -> tile :443-451) with its exact ordering rules, since
the resulting wave order is what the CUDA kernels execute:

1. ``estimate_period`` gives every op a start time; ops are visited by (start, rank, stream, index).
2. Every op *touches* buffers: on the issuing rank (source of a push, destination of a pull, both
   sides of a local copy or collective) and on the peer (destination of a push, source of a pull).
   A touch where communication READS the buffer is a consumer touch (compute is the producer of
   that block and raises the op's dependency flag); one where communication WRITES is a producer
   touch (compute consumes the block after the op's completion flag).
3. Consumer touches are de-duplicated per box, keeping the earliest; they are scheduled only when
   communication never writes that buffer on that rank.
4. Data resident before any transfer becomes wave 0 (unless the buffer is only read by
   communication); the remaining touches are sorted by (start, buffer, issue order, box) and
   grouped into waves of equal start time.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, NamedTuple, Optional, Tuple

from syncopate_b200.communication.descriptor import (
    BufferRegion,
    Collective,
    CommOp,
    CommPlan,
    ReduceOp,
    Signal,
    Transfer,
    TransferOp,
)

from .tile_schedule import RawSchedule, TileBlock, TileCoord


class _ScheduleError(ValueError):
    """Raised for plans that cannot be lowered (missing regions, inconsistent shapes)."""


def _same_time(a: float, b: float) -> bool:
    return math.isclose(a, b, rel_tol=1e-9, abs_tol=1e-9)


def _region_to_tiles(region: BufferRegion) -> List[TileCoord]:
    """One tile per non-empty box of the region."""
    tiles = []
    for box in region.regions:
        extent = tuple(ax.length() for ax in box)
        if extent and all(n > 0 for n in extent):
            tiles.append(TileCoord(offsets=tuple(ax.start for ax in box), shape=extent))
    return tiles


class _Touch(NamedTuple):
    device: int
    buffer: str
    region: BufferRegion
    comm_reads: bool                 # communication consumes the buffer here
    peer: Optional[int]              # the other rank of the exchange, if any
    peer_region: Optional[BufferRegion]
    remote: int                      # 0 = on the issuing rank, 1 = on the peer


def _need(name: str, region: Optional[BufferRegion]) -> BufferRegion:
    if region is None:
        raise _ScheduleError(f"transfer for buffer '{name}' lacks a concrete region")
    return region


def _touches(origin: int, op: CommOp) -> List[_Touch]:
    """Buffer touches of one op: issuing-rank touches first, then peer-side touches."""
    if isinstance(op, Collective):
        return [
            _Touch(origin, op.src_buf, _need(op.src_buf, op.src_region), True, None, None, 0),
            _Touch(origin, op.dst_buf, _need(op.dst_buf, op.dst_region), False, None, None, 0),
        ]
    if not isinstance(op, Transfer):
        raise _ScheduleError(f"unsupported op type: {type(op)}")
    src = _need(op.src_buf, op.src_region)
    dst = _need(op.dst_buf, op.dst_region)
    if op.op == TransferOp.PUSH:
        if op.peer is None:
            raise _ScheduleError("push transfer lacks peer device")
        return [
            _Touch(origin, op.src_buf, src, True, op.peer, dst, 0),
            _Touch(op.peer, op.dst_buf, dst, False, origin, src, 1),
        ]
    if op.op == TransferOp.PULL:
        if op.peer is None:
            raise _ScheduleError("pull transfer lacks peer device")
        return [
            _Touch(origin, op.dst_buf, dst, False, op.peer, src, 0),
            _Touch(op.peer, op.src_buf, src, True, origin, dst, 1),
        ]
    if op.op == TransferOp.LOCAL_COPY:
        # no peer rank, but the copy still has a "far side": recording it gives a fused producer
        # the destination offsets (e.g. row 0 of a reduce-scatter output) instead of its own
        out = [_Touch(origin, op.src_buf, src, True, None, dst, 0)]
        if op.dst_buf != op.src_buf or op.dst_region != op.src_region:
            out.append(_Touch(origin, op.dst_buf, dst, False, None, src, 0))
        return out
    raise _ScheduleError(f"unsupported transfer operation: {op.op}")


def _flag_for(op: CommOp, device: int, comm_reads: bool) -> Optional[Signal]:
    """Flag compute shares with this op on ``device``: the op's dependency flag when compute
    produces the data, the op's completion flag when compute consumes it."""
    if comm_reads:
        candidates = (getattr(dep, "signal", None) for dep in op.dependency)
    else:
        candidates = iter(op.set_signals)
    for sig in candidates:
        if sig is not None and sig.dst_rank == device:
            return sig
    return None


class _Event(NamedTuple):
    start: float
    buffer: str
    order: Tuple[int, ...]
    block: TileBlock

    def sort_key(self):
        return (self.start, self.buffer, self.order, self.block.tile.offsets, self.block.tile.shape)


@dataclass
class _BufferScheduleBuilder:
    """Collects the waves of one buffer on one rank."""

    expected_shape: Optional[Tuple[int, ...]] = None
    _waves: List[List[TileBlock]] = field(default_factory=list)

    def __post_init__(self) -> None:
        if self.expected_shape is not None and any(n <= 0 for n in self.expected_shape):
            raise _ScheduleError("expected_shape must contain positive dimensions")

    def append_wave(self, blocks: Iterable[TileBlock]) -> None:
        blocks = list(blocks)
        if blocks:
            self._waves.append(blocks)

    def has_waves(self) -> bool:
        return bool(self._waves)

    def build(self) -> RawSchedule:
        if not self._waves:
            raise _ScheduleError("cannot build schedule with no waves")
        reach: Optional[List[int]] = None
        for wave in self._waves:
            for block in wave:
                ends = [o + n for o, n in zip(block.tile.offsets, block.tile.shape)]
                if reach is None:
                    reach = ends
                elif len(reach) != len(ends):
                    raise _ScheduleError("inconsistent dimensionality encountered while lowering")
                else:
                    reach = [max(a, b) for a, b in zip(reach, ends)]
        if reach is None:
            raise _ScheduleError("buffer extent is unknown after lowering")
        shape = tuple(reach)
        if self.expected_shape is not None:
            if len(self.expected_shape) != len(reach):
                raise _ScheduleError("mismatched dimensionality between tiles and expected shape")
            for axis, (seen, allowed) in enumerate(zip(reach, self.expected_shape)):
                if seen > allowed:
                    raise _ScheduleError(
                        f"observed extent {seen} exceeds expected shape {allowed} on axis {axis}"
                    )
            shape = tuple(self.expected_shape)
        return RawSchedule(num_waves=len(self._waves), block_infos=[list(w) for w in self._waves], global_shape=shape)


def lower_comm_plan_to_raw_schedules(comm_plan: CommPlan) -> Dict[int, Dict[str, RawSchedule]]:
    """``{rank: {buffer: RawSchedule}}`` for every buffer that compute shares with communication."""
    comm_plan.estimate_period()
    plans = comm_plan.device_plans

    builders: Dict[int, Dict[str, _BufferScheduleBuilder]] = {}

    def builder_for(device: int, buffer: str) -> _BufferScheduleBuilder:
        per_dev = builders.setdefault(device, {})
        if buffer not in per_dev:
            hint = plans[device].tensors_involved.get(buffer) if device in plans else None
            per_dev[buffer] = _BufferScheduleBuilder(expected_shape=None if hint is None else tuple(hint[0]))
        return per_dev[buffer]

    # data resident before anything moves
    resident: Dict[Tuple[int, str], List[TileBlock]] = {}
    for dev, plan in plans.items():
        for buffer, regions in plan.local_regions.items():
            blocks = [TileBlock(tile=t) for region in regions for t in _region_to_tiles(region)]
            if blocks:
                resident.setdefault((dev, buffer), []).extend(blocks)

    # ops in time order
    timeline = []
    for dev, plan in plans.items():
        for s, ops in enumerate(plan.xfer):
            for i, op in enumerate(ops):
                if op.period.start is None:
                    raise _ScheduleError("transfer period start is unknown; run period estimation first")
                timeline.append((op.period.start, dev, s, i, op))
    timeline.sort(key=lambda item: item[:4])

    events: Dict[int, List[_Event]] = {}
    # (device, buffer) -> {box: earliest consumer touch}
    earliest_read: Dict[Tuple[int, str], Dict[Tuple[Tuple[int, ...], Tuple[int, ...]], _Event]] = {}
    comm_reads_buf: Dict[Tuple[int, str], bool] = {}
    comm_writes_buf: Dict[Tuple[int, str], bool] = {}

    for start, origin, s, i, op in timeline:
        reduce_op: Optional[ReduceOp] = op.reduce_op if isinstance(op, Transfer) else None
        for touch in _touches(origin, op):
            if touch.remote and touch.device not in plans:
                continue
            tiles = _region_to_tiles(touch.region)
            if not tiles:
                continue
            far_tiles = _region_to_tiles(touch.peer_region) if touch.peer_region is not None else []
            key = (touch.device, touch.buffer)
            comm_reads_buf.setdefault(key, False)
            comm_writes_buf.setdefault(key, False)
            if touch.comm_reads:
                comm_reads_buf[key] = True
            else:
                comm_writes_buf[key] = True
            flag = _flag_for(op, touch.device, touch.comm_reads)
            for t, tile in enumerate(tiles):
                block = TileBlock(
                    tile=tile,
                    signal=flag,
                    peer_rank=touch.peer,
                    reduce_op=reduce_op,
                    # the role recorded is compute's: the inverse of communication's
                    role="producer" if touch.comm_reads else "consumer",
                    dst_offsets=far_tiles[t].offsets if t < len(far_tiles) else None,
                )
                ev = _Event(start, touch.buffer, (origin, touch.remote, s, i, t), block)
                if not touch.comm_reads:
                    events.setdefault(touch.device, []).append(ev)
                    continue
                seen = earliest_read.setdefault(key, {})
                box = (tile.offsets, tile.shape)
                old = seen.get(box)
                if old is None or start < old.start - 1e-9 or (_same_time(start, old.start) and ev.order < old.order):
                    seen[box] = ev

    for key, per_box in earliest_read.items():
        if comm_writes_buf.get(key):
            continue  # a buffer communication also fills is scheduled from the fills only
        events.setdefault(key[0], []).extend(per_box.values())

    for (dev, buffer), blocks in resident.items():
        touched = (dev, buffer) in comm_reads_buf
        reads, writes = comm_reads_buf.get((dev, buffer), False), comm_writes_buf.get((dev, buffer), False)
        if touched and reads and not writes:
            continue
        role: Optional[str] = None
        if touched and writes and not reads:
            role = "consumer"
        elif touched and reads and not writes:
            role = "producer"
        builder_for(dev, buffer).append_wave(
            TileBlock(tile=b.tile, signal=b.signal, peer_rank=dev, reduce_op=b.reduce_op, role=role) for b in blocks
        )

    for dev, evs in events.items():
        if not evs:
            continue
        evs.sort(key=_Event.sort_key)
        group_start: Optional[float] = None
        group: Dict[str, List[TileBlock]] = {}
        for ev in evs + [None]:
            if ev is None or group_start is None or not _same_time(ev.start, group_start):
                for buffer, blocks in group.items():
                    builder_for(dev, buffer).append_wave(blocks)
                group = {}
                if ev is None:
                    break
                group_start = ev.start
            group.setdefault(ev.buffer, []).append(ev.block)

    lowered: Dict[int, Dict[str, RawSchedule]] = {}
    for dev, per_dev in builders.items():
        built = {name: b.build() for name, b in per_dev.items() if b.has_waves()}
        if built:
            lowered[dev] = built
    return lowered


__all__ = ["lower_comm_plan_to_raw_schedules"]
