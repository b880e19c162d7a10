"""All-gather plan builders: swizzled direct pull/push, ring, hierarchical double ring.

Same signatures and resulting plans as syncopate/communication/common_descriptors/all_gather.py
(:14-115 swizzle, :129-218 ring, :221-372 double ring).  ``shape`` is the GLOBAL gathered shape;
every rank owns the ``rank``-th slab of ``shape[axis] // mesh_size`` along ``axis``.
"""
from __future__ import annotations

from typing import Callable, List, Literal, Sequence, Tuple

import torch

from ..descriptor import BufferRegion, DevicePlan, Transfer, TransferOp, XferDependency
from .utils import box_region, normalize_axis, row_major_strides


def _gather_setup(
    shape: Sequence[int], dtype: torch.dtype, axis: int, mesh_size: int, rank: int, buffer_name: str,
    require_nonempty: bool,
) -> Tuple[DevicePlan, Callable[[int], BufferRegion]]:
    """Validates the arguments, creates the plan with the local slab registered, and returns the
    slab-region factory."""
    elem_size = dtype.itemsize
    if mesh_size <= 0:
        raise ValueError("mesh_size must be positive")
    if elem_size <= 0:
        raise ValueError("elem_size must be positive")
    shape = tuple(shape)
    if len(shape) == 0:
        raise ValueError("all_gather expects at least one dimension")
    axis = normalize_axis(axis, len(shape))
    if shape[axis] % mesh_size:
        raise ValueError(
            f"axis length {shape[axis]} along dim {axis} must be divisible by mesh_size {mesh_size}"
        )
    slab = shape[axis] // mesh_size
    if require_nonempty and slab == 0:
        raise ValueError("all-gather requires non-empty slices along the gather axis")
    strides = row_major_strides(shape)

    def slab_region(owner: int) -> BufferRegion:
        return box_region(shape, elem_size, strides, {axis: (owner * slab, owner * slab + slab)})

    plan = DevicePlan(dev=rank)
    plan.tensors_involved[buffer_name] = (torch.Size(shape), dtype)
    return plan, slab_region


def build_all_gather_plan_1d_swizzle(
    shape: Sequence[int],
    dtype: torch.dtype,
    axis: int,
    mesh_size: int,
    rank: int,
    buffer_name: str = "buffer",
    transfer_kind: Literal["push", "pull"] = "pull",
) -> DevicePlan:
    """Direct all-gather: rank r exchanges with peers r+1, r+2, ... (mod mesh) in that order, so
    that at every step each rank talks to a different peer."""
    plan, slab_region = _gather_setup(shape, dtype, axis, mesh_size, rank, buffer_name, False)
    if transfer_kind not in {"push", "pull"}:
        raise ValueError("transfer_kind must be 'push' or 'pull'")
    mine = slab_region(rank)
    plan.local_regions.setdefault(buffer_name, []).append(mine)
    for step in range(mesh_size):
        peer = (rank + step) % mesh_size
        if peer == rank:
            continue
        if transfer_kind == "pull":
            theirs = slab_region(peer)
            op = Transfer(op=TransferOp.PULL, src_buf=buffer_name, src_region=theirs, dst_buf=buffer_name,
                          dst_region=theirs, chunk_idx=peer, peer=peer)
        else:
            op = Transfer(op=TransferOp.PUSH, src_buf=buffer_name, src_region=mine, dst_buf=buffer_name,
                          dst_region=mine, chunk_idx=rank, peer=peer)
        plan.add_op(op)
    return plan


def _normalize_dim(axis: int, ndim: int) -> int:
    return normalize_axis(axis, ndim)


def build_ring_all_gather_plan(
    shape: Sequence[int],
    dtype: torch.dtype,
    axis: int,
    mesh_size: int,
    rank: int,
    buffer_name: str = "buffer",
) -> DevicePlan:
    """Ring all-gather with pushes: at step s rank r forwards the slab of rank r-s to rank r+1,
    after its upstream neighbour's step s-1 push has delivered that slab."""
    plan, slab_region = _gather_setup(shape, dtype, axis, mesh_size, rank, buffer_name, True)
    plan.local_regions.setdefault(buffer_name, []).append(slab_region(rank))
    if mesh_size == 1:
        return plan
    downstream = (rank + 1) % mesh_size
    upstream = (rank - 1) % mesh_size
    for step in range(mesh_size - 1):
        owner = (rank - step) % mesh_size
        waits: List[XferDependency] = []
        if step > 0:
            waits.append(XferDependency(depend_rank=upstream, depend_xfer_stream=0, depend_xfer_idx=step - 1))
        region = slab_region(owner)
        plan.add_op(
            Transfer(op=TransferOp.PUSH, src_buf=buffer_name, src_region=region, dst_buf=buffer_name,
                     dst_region=region, chunk_idx=owner, peer=downstream, dependency=waits)
        )
    return plan


def build_double_ring_all_gather_plan(
    shape: Sequence[int],
    dtype: torch.dtype,
    axis: int,
    mesh_size: int,
    inner_mesh_size: int,
    rank: int,
    buffer_name: str = "buffer",
) -> DevicePlan:
    """Two-level ring: ranks form contiguous groups of ``inner_mesh_size``.  For each outer step
    the group's current set of slabs circulates once around the inner ring and is then handed to
    the same inner position of the next group."""
    if mesh_size <= 0:
        raise ValueError("mesh_size must be positive")
    if inner_mesh_size <= 0:
        raise ValueError("inner_mesh_size must be positive")
    if mesh_size % inner_mesh_size:
        raise ValueError("mesh_size must be divisible by inner_mesh_size")
    plan, slab_region = _gather_setup(shape, dtype, axis, mesh_size, rank, buffer_name, True)
    plan.local_regions.setdefault(buffer_name, []).append(slab_region(rank))
    if mesh_size == 1:
        return plan

    g = inner_mesh_size
    groups = mesh_size // g
    gid, pos = divmod(rank, g)
    inner_next = gid * g + (pos + 1) % g
    inner_prev = gid * g + (pos - 1) % g
    outer_next = ((gid + 1) % groups) * g + pos
    outer_prev = ((gid - 1) % groups) * g + pos
    per_step = g  # g-1 inner pushes followed by one outer push

    def after(peer: int, op_idx: int) -> List[XferDependency]:
        return [XferDependency(depend_rank=peer, depend_xfer_stream=0, depend_xfer_idx=op_idx)]

    for outer in range(groups):
        src_group = (gid - outer) % groups
        arrived = after(outer_prev, outer * per_step - 1) if outer > 0 else []
        for inner in range(g - 1):
            owner = src_group * g + (pos + outer - inner) % g
            region = slab_region(owner)
            waits = arrived if inner == 0 else after(inner_prev, outer * per_step + inner - 1)
            plan.add_op(
                Transfer(op=TransferOp.PUSH, src_buf=buffer_name, src_region=region, dst_buf=buffer_name,
                         dst_region=region, chunk_idx=src_group * g + pos, peer=inner_next, dependency=waits)
            )
        if outer < groups - 1:
            owner = src_group * g + (pos + outer + 1) % g
            region = slab_region(owner)
            waits = arrived if g == 1 else after(inner_prev, outer * per_step + (g - 2))
            plan.add_op(
                Transfer(op=TransferOp.PUSH, src_buf=buffer_name, src_region=region, dst_buf=buffer_name,
                         dst_region=region, chunk_idx=src_group * g + pos, peer=outer_next, dependency=waits)
            )
    return plan


__all__ = [
    "build_all_gather_plan_1d_swizzle",
    "build_ring_all_gather_plan",
    "build_double_ring_all_gather_plan",
]
