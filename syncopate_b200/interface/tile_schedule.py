"""Tile schedules: what compute sees of a communication plan.

Communication tells compute *when* each block of a buffer becomes available (or must be produced),
as an ordered list of waves; compute never needs to know how the bytes travel.  Same classes as
syncopate/interface/tile_schedule.py (``TileCoord``/``TileBlock`` :14-61, ``RawSchedule`` and its
``gen_*`` flatteners :65-171, ``SimplifiedSchedule``/``Mod1DSchedule`` :177-272).  The ``gen_*``
lists are exactly what the CUDA kernels receive as schedule arrays.
"""
from __future__ import annotations

import abc
from dataclasses import dataclass
from typing import Iterator, List, Literal, Optional, Tuple

from syncopate_b200.communication.descriptor import ReduceOp, Signal

TileRole = Literal["producer", "consumer"]


@dataclass
class TileCoord:
    """Origin and extent of a box inside an N-D tensor."""

    offsets: Tuple[int, ...]
    shape: Tuple[int, ...]

    def __post_init__(self) -> None:
        if len(self.offsets) != len(self.shape):
            raise ValueError("offsets and shape must have identical length")
        if min(self.offsets, default=0) < 0:
            raise ValueError("offsets must be non-negative")
        if any(n <= 0 for n in self.shape):
            raise ValueError("shape must contain strictly positive sizes")

    @property
    def ndim(self) -> int:
        return len(self.offsets)

    def as_ranges(self) -> Tuple[Tuple[int, int], ...]:
        return tuple((o, o + n) for o, n in zip(self.offsets, self.shape))

    def __repr__(self) -> str:
        return f"TileCoord(offsets={self.offsets}, shape={self.shape})"


@dataclass
class TileBlock:
    """A box plus how it is synchronised and exchanged.

    ``signal``: flag that publishes the block (consumer: wait for it; producer: raise it).
    ``peer_rank``: rank the block is exchanged with when compute talks to the peer directly;
    ``None`` for purely local data.  ``reduce_op``: set when the transfer accumulates, so a fused
    producer must add instead of store.  ``role``: whether compute writes ("producer") or reads
    ("consumer") the block.  ``dst_offsets``: where the block sits inside the peer's allocation
    (destination box of a push, source box of a pull); ``None`` without a remote counterpart.
    """

    tile: TileCoord
    signal: Optional[Signal] = None
    peer_rank: Optional[int] = None
    reduce_op: Optional[ReduceOp] = None
    role: Optional[TileRole] = None
    dst_offsets: Optional[Tuple[int, ...]] = None


@dataclass
class RawSchedule:
    """Waves of blocks in the order communication makes them available."""

    num_waves: int
    block_infos: List[List[TileBlock]]
    global_shape: Tuple[int, ...]

    def __post_init__(self) -> None:
        if self.num_waves <= 0:
            raise ValueError("num_waves must be positive")
        if len(self.block_infos) != self.num_waves:
            raise ValueError("block_infos length must match num_waves")
        if any(len(wave) == 0 for wave in self.block_infos):
            raise ValueError("each wave must contain at least one block")
        rank = len(self.global_shape)
        if any(b.tile.ndim != rank for b in self._blocks()):
            raise ValueError("all blocks must have the same number of dimensions as global_shape")

    def _blocks(self) -> Iterator[TileBlock]:
        for wave in self.block_infos:
            yield from wave

    def __repr__(self) -> str:
        return (
            f"RawSchedule(num_waves={self.num_waves}, "
            f"global_shape={self.global_shape}, "
            f"block_infos=[{self.block_infos}])"
        )

    def gen_block_offset_lists(self) -> List[List[int]]:
        """Offsets of every block, wave-major."""
        return [list(b.tile.offsets) for b in self._blocks()]

    def gen_block_shape_lists(self) -> List[List[int]]:
        """Shapes of every block, wave-major."""
        return [list(b.tile.shape) for b in self._blocks()]

    def gen_signal_lists(self) -> List[int]:
        """Flag slot of every block, -1 when the block needs no flag."""
        return [-1 if b.signal is None else b.signal.dst_offset for b in self._blocks()]

    def gen_target_rank_list(self) -> List[int]:
        """Peer rank of every block for in-kernel direct reads/writes, -1 for local blocks."""
        return [-1 if b.peer_rank is None else b.peer_rank for b in self._blocks()]

    def gen_dst_offset_lists(self) -> List[List[int]]:
        """Peer-side offsets of every block; a block without a remote counterpart reports its own
        offsets, so that 'subtract own offset, add peer offset' leaves local accesses in place."""
        return [list(b.tile.offsets if b.dst_offsets is None else b.dst_offsets) for b in self._blocks()]

    def is_reduce(self) -> bool:
        """True when any block comes from an accumulating transfer."""
        return any(b.reduce_op is not None for b in self._blocks())

    def role(self) -> Optional[TileRole]:
        """The role shared by all blocks that carry one (``None`` if none does); blocks that
        disagree raise ``ValueError``."""
        seen: Optional[TileRole] = None
        for b in self._blocks():
            if b.role is None:
                continue
            if seen is None:
                seen = b.role
            elif seen != b.role:
                raise ValueError(f"schedule blocks disagree on role: {seen!r} vs {b.role!r}")
        return seen


@dataclass
class SimplifiedSchedule:
    """Tries to express a RawSchedule in closed form (so kernels need no schedule arrays)."""

    origin_schedule: RawSchedule
    simplified_schedule: "None | SimpleSchedule" = None

    def simplify(self) -> bool:
        for candidate in sorted(SimpleSchedule.__subclasses__(), key=lambda c: c.priority):
            try:
                self.simplified_schedule = candidate(self.origin_schedule)
            except Exception as exc:
                print(f"Failed to simplify schedule to {candidate.__name__}: {exc}")
                continue
            print(f"Simplified schedule to {candidate.__name__}")
            return True
        return False


class SimpleSchedule(abc.ABC):
    priority = 99

    @abc.abstractmethod
    def __init__(self, raw_schedule: RawSchedule):
        pass

    @abc.abstractmethod
    def __repr__(self) -> str:
        pass


class Mod1DSchedule(SimpleSchedule):
    """One equal-sized block per wave along a single axis, flags 0, 1, 2, ... from the second
    wave on: the pattern of ring and swizzled direct all-gathers."""

    priority = 1

    num_waves: int
    global_shape: Tuple[int, ...]
    stride: int
    starting_offset: int
    schedule_axis: int

    def __init__(self, raw_schedule: RawSchedule):
        self.num_waves = raw_schedule.num_waves
        self.global_shape = raw_schedule.global_shape
        waves = raw_schedule.block_infos
        if any(len(w) != 1 for w in waves):
            raise ValueError("all waves must contain exactly one block")
        blocks = [w[0] for w in waves]
        box = blocks[0].tile.shape
        if any(b.tile.shape != box for b in blocks):
            raise ValueError("all blocks must have the same shape")
        partial = [ax for ax, full in enumerate(self.global_shape) if box[ax] < full]
        if len(partial) != 1:
            raise ValueError("schedule must be defined along exactly one axis")
        self.schedule_axis = partial[0]
        self.stride = box[self.schedule_axis]
        self.starting_offset = blocks[0].tile.offsets[self.schedule_axis]
        if blocks[0].signal is not None:
            raise ValueError("first block (local) must not have any signals")
        for w, b in enumerate(blocks[1:], start=1):
            if b.signal is None or b.signal.dst_offset != w - 1:
                raise ValueError("signal offsets do not match expected pattern")

    def __post_init__(self) -> None:
        if self.schedule_axis < 0 or self.schedule_axis >= len(self.global_shape):
            raise ValueError("schedule_axis must be a valid axis index")
        if self.stride * self.num_waves != self.global_shape[self.schedule_axis]:
            raise ValueError("stride * num_waves must equal the size of the schedule_axis in global_shape")

    def __repr__(self) -> str:
        return (
            f"Mod1DSchedule(num_waves={self.num_waves}, "
            f"global_shape={self.global_shape}, "
            f"stride={self.stride}, "
            f"starting_offset={self.starting_offset}, "
            f"schedule_axis={self.schedule_axis})"
        )
