"""All-reduce plan builders: the reduction as one or several library collectives over slices of one
axis, optionally gated by the local producer (GEMM + all-reduce).

Same signatures and resulting plans as syncopate/communication/common_descriptors/all_reduce.py
(:13-113 in place, :116-214 separate source and destination buffers for the in-switch reduction).
``shape`` is the tensor every rank contributes; slice i of ``split_axis`` is reduced by collective i,
which (with ``compute_producer``) waits until the rank's producer has written that slice.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..descriptor import Collective, CollectiveOp, ComputeDependency, DevicePlan
from .utils import box_region, ensure_divisible, row_major_strides


def _slices_setup(shape: Sequence[int], dtype: torch.dtype, mesh_size: int, num_all_reduces: int,
                  split_axis: Optional[int]):
    """Argument checks shared by both builders; returns (shape, element size, strides, axis, chunk)."""
    es = dtype.itemsize
    if mesh_size <= 0:
        raise ValueError("mesh_size must be positive")
    if es <= 0:
        raise ValueError("elem_size must be positive")
    if num_all_reduces <= 0:
        raise ValueError("num_all_reduces must be positive")
    shape = tuple(shape)
    ndim = len(shape)
    if ndim == 0:
        raise ValueError("all_reduce expects at least one dimension")
    if split_axis is None:
        if num_all_reduces != 1:
            raise ValueError("split_axis is required when num_all_reduces > 1")
        split_axis = 0
    if split_axis < 0:
        split_axis += ndim
    if not 0 <= split_axis < ndim:
        raise IndexError(f"split_axis {split_axis} out of range for tensor with {ndim} dims")
    ensure_divisible(shape[split_axis], num_all_reduces, "num_all_reduces")
    chunk = shape[split_axis] // num_all_reduces
    if chunk == 0:
        raise ValueError("split produces empty chunks")
    return shape, es, row_major_strides(shape), split_axis, chunk


def _add_collectives(plan: DevicePlan, kind: CollectiveOp, src: str, dst: str, shape, es, strides, axis: int,
                     chunk: int, count: int, rank: int, compute_producer: bool) -> None:
    for i in range(count):
        region = box_region(shape, es, strides, {axis: (i * chunk, (i + 1) * chunk)})
        deps = [ComputeDependency(compute_rank=rank, src_region=region)] if compute_producer else []
        plan.add_op(Collective(op=kind, src_buf=src, src_region=region, dst_buf=dst, dst_region=region, dependency=deps))


def build_all_reduce_plan(
    shape: Sequence[int],
    *,
    dtype: torch.dtype,
    mesh_size: int,
    rank: int,
    buffer_name: str,
    num_all_reduces: int = 1,
    split_axis: int | None = None,
    compute_producer: bool = False,
) -> DevicePlan:
    """In-place all-reduce of ``buffer_name`` as ``num_all_reduces`` collectives along ``split_axis``."""
    shape, es, strides, axis, chunk = _slices_setup(shape, dtype, mesh_size, num_all_reduces, split_axis)
    plan = DevicePlan(dev=rank)
    plan.tensors_involved[buffer_name] = (torch.Size(shape), dtype)
    plan.local_regions.setdefault(buffer_name, []).append(box_region(shape, es, strides, {}))
    _add_collectives(plan, CollectiveOp.ALL_REDUCE, buffer_name, buffer_name, shape, es, strides, axis, chunk,
                     num_all_reduces, rank, compute_producer)
    return plan


def build_all_reduce_nvsharp_plan(
    shape: Sequence[int],
    *,
    dtype: torch.dtype,
    mesh_size: int,
    rank: int,
    src_name: str,
    dst_name: str,
    num_all_reduces: int = 1,
    split_axis: int | None = None,
    compute_producer: bool = False,
) -> DevicePlan:
    """All-reduce from ``src_name`` into ``dst_name`` (the form the in-switch reduction takes)."""
    shape, es, strides, axis, chunk = _slices_setup(shape, dtype, mesh_size, num_all_reduces, split_axis)
    plan = DevicePlan(dev=rank)
    plan.tensors_involved[src_name] = (torch.Size(shape), dtype)
    plan.tensors_involved[dst_name] = (torch.Size(shape), dtype)
    _add_collectives(plan, CollectiveOp.ALL_REDUCE_NVSHARP, src_name, dst_name, shape, es, strides, axis, chunk,
                     num_all_reduces, rank, compute_producer)
    return plan


__all__ = ["build_all_reduce_plan", "build_all_reduce_nvsharp_plan"]
