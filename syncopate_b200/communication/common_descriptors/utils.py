"""Helpers shared by the plan builders (cf. syncopate/communication/common_descriptors/utils.py)."""
from __future__ import annotations

from typing import Dict, List, Mapping, Sequence, Tuple

from ..descriptor import BufferRegion


def ensure_divisible(length: int, mesh_size: int, axis: str | int) -> None:
    if length % mesh_size:
        raise ValueError(f"axis '{axis}' length {length} must be divisible by mesh size {mesh_size}")


def lookup_mesh_size(mesh: Dict[str, int], mesh_axis: str) -> int:
    if mesh_axis not in mesh:
        raise ValueError(f"mesh axis '{mesh_axis}' not found in mesh")
    size = mesh[mesh_axis]
    if size <= 0:
        raise ValueError(f"mesh axis '{mesh_axis}' must be positive")
    return size


def row_major_strides(shape: Sequence[int]) -> Sequence[int]:
    strides: List[int] = []
    acc = 1
    for dim in reversed(shape):
        strides.append(acc)
        acc *= dim
    strides.reverse()
    return strides


def compute_offset(strides: Sequence[int], starts: Mapping[int, int]) -> int:
    return sum(starts.get(axis, 0) * stride for axis, stride in enumerate(strides))


def block_nbytes(shape: Sequence[int], elem_size: int, lengths: Mapping[int, int]) -> int:
    count = 1
    for axis, size in enumerate(shape):
        count *= lengths.get(axis, size)
    return count * elem_size


def normalize_axis(axis: int, ndim: int) -> int:
    """Python-style negative axis; IndexError text shared by every builder."""
    if axis < 0:
        axis += ndim
    if not 0 <= axis < ndim:
        raise IndexError(f"axis {axis} out of range for tensor with {ndim} dims")
    return axis


def box_region(
    shape: Sequence[int], elem_size: int, strides: Sequence[int], overrides: Mapping[int, Tuple[int, int]]
) -> BufferRegion:
    """Full extent on every axis except those given as ``axis -> (start, end)``."""
    slices = [overrides.get(d, (0, n)) for d, n in enumerate(shape)]
    return BufferRegion.from_slices(elem_size=elem_size, strides=strides, slices=slices)


__all__ = [
    "block_nbytes",
    "compute_offset",
    "ensure_divisible",
    "lookup_mesh_size",
    "row_major_strides",
]
