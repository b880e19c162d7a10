"""Reduce-scatter plan builders.

``build_reduce_scatter_collective_plan`` mirrors
syncopate/communication/common_descriptors/reduce_scatter.py:22-158 (library collectives, optionally
cut along a second axis); ``build_reduce_scatter_direct_reduce_plan`` mirrors :161-304 (every rank
pushes slab p of its partial result into rank p's output with ``reduce_op``; own slab last).
"""
from __future__ import annotations

from typing import Literal, Sequence

import torch

from ..descriptor import (
    BufferRegion,
    Collective,
    CollectiveOp,
    ComputeDependency,
    DevicePlan,
    ReduceOp,
    Transfer,
    TransferOp,
)
from .utils import box_region, ensure_divisible, row_major_strides


def _wrap_axis(axis: int, ndim: int, what: str = "axis") -> int:
    if axis < 0:
        axis += ndim
    if not 0 <= axis < ndim:
        raise IndexError(f"{what} {axis} out of range for tensor with {ndim} dims")
    return axis


def build_reduce_scatter_collective_plan(
    shape: Sequence[int],
    *,
    dtype: torch.dtype,
    axis: int,
    split_axis: int | None = None,
    mesh_size: int,
    rank: int,
    src_buffer: str,
    dst_buffer: str,
    num_reduce_scatters: int = 1,
    compute_producer: bool = False,
) -> DevicePlan:
    """Reduce-scatter along ``axis`` as ``num_reduce_scatters`` collectives over slices of
    ``split_axis``.  ``shape`` is the full pre-reduction tensor on every rank."""
    es = dtype.itemsize
    if mesh_size <= 0:
        raise ValueError("mesh_size must be positive")
    if es <= 0:
        raise ValueError("elem_size must be positive")
    if num_reduce_scatters <= 0:
        raise ValueError("num_reduce_scatters must be positive")
    shape = tuple(shape)
    ndim = len(shape)
    if ndim == 0:
        raise ValueError("reduce_scatter expects at least one dimension")
    axis = _wrap_axis(axis, ndim)
    ensure_divisible(shape[axis], mesh_size, axis)
    per_rank = shape[axis] // mesh_size

    if split_axis is None:
        if num_reduce_scatters != 1:
            raise ValueError("split_axis is required when num_reduce_scatters > 1")
        split_axis = axis + 1 if axis + 1 < ndim else 0
        if split_axis == axis:
            split_axis = (axis + 1) % ndim
    split_axis = _wrap_axis(split_axis, ndim, "split_axis")
    if split_axis == axis:
        raise ValueError("split_axis must differ from reduce axis")
    ensure_divisible(shape[split_axis], num_reduce_scatters, "num_reduce_scatters")
    piece = shape[split_axis] // num_reduce_scatters
    if piece == 0:
        raise ValueError("split produces empty chunks")

    dst_shape = tuple(per_rank if d == axis else n for d, n in enumerate(shape))
    s_str, d_str = row_major_strides(shape), row_major_strides(dst_shape)
    plan = DevicePlan(dev=rank)
    plan.tensors_involved[src_buffer] = (torch.Size(shape), dtype)
    plan.tensors_involved[dst_buffer] = (torch.Size(dst_shape), dtype)
    plan.local_regions.setdefault(src_buffer, []).append(
        box_region(shape, es, s_str, {split_axis: (0, shape[split_axis])})
    )
    for k in range(num_reduce_scatters):
        span = (k * piece, (k + 1) * piece)
        src = box_region(shape, es, s_str, {split_axis: span})
        dst = box_region(dst_shape, es, d_str, {split_axis: span})
        waits = [ComputeDependency(compute_rank=rank, src_region=src)] if compute_producer else []
        plan.add_op(
            Collective(op=CollectiveOp.REDUCE_SCATTER, src_buf=src_buffer, src_region=src, dst_buf=dst_buffer,
                       dst_region=dst, dependency=waits)
        )
    return plan


def build_reduce_scatter_direct_reduce_plan(
    shape: Sequence[int],
    *,
    dtype: torch.dtype,
    axis: int,
    mesh_size: int,
    rank: int,
    src_buffer: str,
    dst_buffer: str,
    reduce_op: ReduceOp = ReduceOp.SUM,
    transfer_kind: Literal["push", "pull"] = "push",
) -> DevicePlan:
    """Reduce-scatter by direct remote reduction: for i = 1..mesh-1 rank r sends slab (r+i) of its
    partial result into the whole output buffer of rank r+i (or pulls its own slab from r+i), each
    gated by the compute that produces the slab; the local slab is reduced in last."""
    es = dtype.itemsize
    if mesh_size <= 0:
        raise ValueError("mesh_size must be positive")
    if es <= 0:
        raise ValueError("elem_size must be positive")
    if rank < 0 or rank >= mesh_size:
        raise ValueError("rank must be in [0, mesh_size)")
    shape = tuple(shape)
    ndim = len(shape)
    if ndim == 0:
        raise ValueError("reduce_scatter expects at least one dimension")
    axis = _wrap_axis(axis, ndim)
    ensure_divisible(shape[axis], mesh_size, axis)
    per_rank = shape[axis] // mesh_size
    if per_rank == 0:
        raise ValueError("reduce_scatter requires non-empty slices along the reduce axis")
    if transfer_kind not in {"push", "pull"}:
        raise ValueError("transfer_kind must be 'push' or 'pull'")

    dst_shape = tuple(per_rank if d == axis else n for d, n in enumerate(shape))
    s_str, d_str = row_major_strides(shape), row_major_strides(dst_shape)
    plan = DevicePlan(dev=rank)
    plan.tensors_involved[src_buffer] = (torch.Size(shape), dtype)
    plan.tensors_involved[dst_buffer] = (torch.Size(dst_shape), dtype)
    plan.local_regions.setdefault(src_buffer, []).append(box_region(shape, es, s_str, {}))

    slab = lambda i: box_region(shape, es, s_str, {axis: (i * per_rank, (i + 1) * per_rank)})
    whole_dst = box_region(dst_shape, es, d_str, {})
    mine = slab(rank)
    for i in range(mesh_size - 1):
        peer = (rank + i + 1) % mesh_size
        if transfer_kind == "push":
            src = slab(peer)
            plan.add_op(
                Transfer(op=TransferOp.PUSH, src_buf=src_buffer, src_region=src, dst_buf=dst_buffer,
                         dst_region=whole_dst, chunk_idx=i, peer=peer,
                         dependency=[ComputeDependency(compute_rank=rank, src_region=src)], reduce_op=reduce_op)
            )
        else:
            plan.add_op(
                Transfer(op=TransferOp.PULL, src_buf=src_buffer, src_region=mine, dst_buf=dst_buffer,
                         dst_region=whole_dst, chunk_idx=i, peer=peer,
                         dependency=[ComputeDependency(compute_rank=peer, src_region=mine)], reduce_op=reduce_op)
            )
    plan.add_op(
        Transfer(op=TransferOp.LOCAL_COPY, src_buf=src_buffer, src_region=mine, dst_buf=dst_buffer,
                 dst_region=whole_dst, chunk_idx=mesh_size - 1,
                 dependency=[ComputeDependency(compute_rank=rank, src_region=mine)], reduce_op=reduce_op)
    )
    return plan


__all__ = ["build_reduce_scatter_collective_plan"]
