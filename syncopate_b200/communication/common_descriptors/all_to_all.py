"""All-to-all plan builders.

Same signatures and resulting plans as syncopate/communication/common_descriptors/all_to_all.py:
``build_all_to_all_plan`` (:11-169, dim-0 exchange into a ``(mesh, chunk, ...)`` buffer),
``build_all_to_all_plan_dim`` (:179-370, moves the sharding from one axis to another — the Ulysses
reshard), ``build_all_to_all_plan_dim_waves`` (:373-572) and ``build_all_to_all_plan_axis`` (:575-735).

All four share one skeleton: a source-slab factory (what this rank holds for peer p), a
destination-slab factory (where data from rank s lands), a peer order, and the rule that the local
copy goes first when communication produces the buffer and last when compute produces it.
"""
from __future__ import annotations

from typing import Callable, List, Literal, Optional, Sequence

import torch

from ..descriptor import BufferRegion, ComputeDependency, DevicePlan, Transfer, TransferOp
from .utils import block_nbytes, box_region, ensure_divisible, normalize_axis, row_major_strides

RegionOf = Callable[[int], BufferRegion]


def _check_common(shape: Sequence[int], dtype: torch.dtype, mesh_size: int) -> tuple:
    if mesh_size <= 0:
        raise ValueError("mesh_size must be positive")
    if dtype.itemsize <= 0:
        raise ValueError("elem_size must be positive")
    shape = tuple(shape)
    if not shape:
        raise ValueError("all_to_all expects at least one dimension in the source shape")
    return shape


def _new_plan(rank: int, src_buffer: str, dst_buffer: str, shape, dst_shape, dtype) -> DevicePlan:
    plan = DevicePlan(dev=rank)
    plan.src_shape = shape  # type: ignore[attr-defined]
    plan.dst_shape = dst_shape  # type: ignore[attr-defined]
    plan.tensors_involved[src_buffer] = (torch.Size(shape), dtype)
    plan.tensors_involved[dst_buffer] = (torch.Size(dst_shape), dtype)
    return plan


def _after_compute(rank: int, region: BufferRegion, explicit_none: bool = True) -> List[ComputeDependency]:
    if explicit_none:
        return [ComputeDependency(compute_rank=rank, src_region=region, signal=None)]
    return [ComputeDependency(compute_rank=rank, src_region=region)]


def _exchange(
    plan: DevicePlan,
    *,
    rank: int,
    peers: Sequence[int],
    mesh_size: int,
    src_buffer: str,
    dst_buffer: str,
    src_for: RegionOf,
    dst_for: RegionOf,
    transfer_kind: str,
    compute_producer: bool,
) -> DevicePlan:
    """Local copy + one transfer per peer (the skeleton of the three single-wave builders)."""
    mine_src, mine_dst = src_for(rank), dst_for(rank)
    plan.local_regions.setdefault(src_buffer, []).append(mine_src)
    local_copy = Transfer(
        op=TransferOp.LOCAL_COPY,
        src_buf=src_buffer,
        dst_buf=dst_buffer,
        src_region=mine_src,
        dst_region=mine_dst,
        chunk_idx=-1,
        dependency=_after_compute(rank, mine_src) if compute_producer else [],
    )
    if not compute_producer:
        plan.add_op(local_copy, stream_idx=0)
    for peer in peers:
        if transfer_kind == "push":
            outgoing = src_for(peer)
            plan.add_op(
                Transfer(
                    op=TransferOp.PUSH,
                    src_buf=src_buffer,
                    src_region=outgoing,
                    peer=peer,
                    chunk_idx=rank * mesh_size + peer,
                    dst_buf=dst_buffer,
                    dst_region=mine_dst,
                    dependency=_after_compute(rank, src_for(peer)) if compute_producer else [],
                )
            )
        else:
            plan.add_op(
                Transfer(
                    op=TransferOp.PULL,
                    dst_buf=dst_buffer,
                    dst_region=dst_for(peer),
                    peer=peer,
                    chunk_idx=peer * mesh_size + rank,
                    src_buf=src_buffer,
                    src_region=mine_src,
                    dependency=_after_compute(peer, mine_src, explicit_none=False) if compute_producer else [],
                )
            )
    if compute_producer:
        plan.add_op(local_copy)
    return plan


def build_all_to_all_plan(
    shape: Sequence[int],
    *,
    dtype: torch.dtype,
    mesh_size: int,
    rank: int,
    src_buffer: str,
    dst_buffer: str,
    transfer_kind: Literal["push", "pull"] = "push",
    compute_producer: bool = False,
) -> DevicePlan:
    """Dim-0 all-to-all: slab p of the local ``shape`` goes to rank p, which stores the slab coming
    from rank s at ``dst[s]`` of a ``(mesh_size, shape[0] // mesh_size, *shape[1:])`` buffer."""
    shape = _check_common(shape, dtype, mesh_size)
    es = dtype.itemsize
    ensure_divisible(shape[0], mesh_size, axis=0)
    chunk = shape[0] // mesh_size
    if chunk == 0:
        raise ValueError("all-to-all requires non-empty slices along dim0")
    if block_nbytes(shape, es, {0: chunk}) == 0:
        raise ValueError("all-to-all transfer would be empty")
    dst_shape = (mesh_size, chunk, *shape[1:])
    s_str, d_str = row_major_strides(shape), row_major_strides(dst_shape)
    plan = _new_plan(rank, src_buffer, dst_buffer, shape, dst_shape, dtype)
    src_for = lambda p: box_region(shape, es, s_str, {0: (p * chunk, (p + 1) * chunk)})
    dst_for = lambda s: box_region(dst_shape, es, d_str, {0: (s, s + 1)})
    mine_src, mine_dst = src_for(rank), dst_for(rank)  # built before validation, as the reference does
    del mine_src, mine_dst
    if transfer_kind not in {"push", "pull"}:
        raise ValueError("transfer_kind must be 'push' or 'pull'")
    peers = [(rank + i) % mesh_size for i in range(1, mesh_size)]
    return _exchange(plan, rank=rank, peers=peers, mesh_size=mesh_size, src_buffer=src_buffer,
                     dst_buffer=dst_buffer, src_for=src_for, dst_for=dst_for, transfer_kind=transfer_kind,
                     compute_producer=compute_producer)


def _normalize_dim(axis: int, ndim: int) -> int:
    return normalize_axis(axis, ndim)


def _reshard_geometry(shape, dtype, mesh_size, src_split_axis, dst_split_axis, wave_div: Optional[int]):
    """Shapes and region factories of a reshard from ``src_split_axis`` to ``dst_split_axis``."""
    es = dtype.itemsize
    ndim = len(shape)
    sa = normalize_axis(src_split_axis, ndim)
    da = normalize_axis(dst_split_axis, ndim)
    if sa == da:
        raise ValueError("src_split_axis and dst_split_axis must differ")
    src_chunk = shape[sa]
    if src_chunk <= 0:
        raise ValueError("all-to-all requires non-empty slices along the split axis")
    ensure_divisible(shape[da], mesh_size, axis=da)
    dst_chunk = shape[da] // mesh_size
    if dst_chunk == 0:
        raise ValueError("all-to-all requires non-empty slices along the destination axis")
    piece = dst_chunk
    if wave_div is not None:
        ensure_divisible(dst_chunk, wave_div, "num_waves")
        piece = dst_chunk // wave_div
        if piece == 0:
            raise ValueError("wave splitting produced an empty chunk along dst_split_axis")
    if block_nbytes(shape, es, {sa: src_chunk, da: piece}) == 0:
        raise ValueError("all-to-all transfer would be empty")
    dst_shape = list(shape)
    dst_shape[sa] = src_chunk * mesh_size
    dst_shape[da] = dst_chunk
    s_str, d_str = row_major_strides(shape), row_major_strides(dst_shape)

    def src_for(peer: int, wave: Optional[int] = None) -> BufferRegion:
        lo = peer * dst_chunk
        if wave is None:
            return box_region(shape, es, s_str, {sa: (0, src_chunk), da: (lo, lo + dst_chunk)})
        lo += wave * piece
        return box_region(shape, es, s_str, {sa: (0, src_chunk), da: (lo, lo + piece)})

    def dst_for(source: int, wave: Optional[int] = None) -> BufferRegion:
        rows = (source * src_chunk, (source + 1) * src_chunk)
        if wave is None:
            return box_region(dst_shape, es, d_str, {sa: rows, da: (0, dst_chunk)})
        return box_region(dst_shape, es, d_str, {sa: rows, da: (wave * piece, (wave + 1) * piece)})

    return dst_shape, src_for, dst_for


def _ordered_peers(rank: int, mesh_size: int, peer_order: str, include_self: bool) -> List[int]:
    sign = 1 if peer_order == "clockwise" else -1
    first = 0 if include_self else 1
    return [(rank + sign * i) % mesh_size for i in range(first, mesh_size)]


def build_all_to_all_plan_dim(
    shape: Sequence[int],
    *,
    dtype: torch.dtype,
    mesh_size: int,
    rank: int,
    src_buffer: str,
    dst_buffer: str,
    src_split_axis: int,
    dst_split_axis: int,
    transfer_kind: Literal["push", "pull"] = "push",
    compute_producer: bool = False,
    peer_order: Literal["clockwise", "counter-clockwise"] = "clockwise",
) -> DevicePlan:
    """Reshard ``[.., S/w, .., H, ..] -> [.., S, .., H/w, ..]``: ``shape`` is the local source shape
    (sharded along ``src_split_axis``); the destination is sharded along ``dst_split_axis``."""
    shape = _check_common(shape, dtype, mesh_size)
    dst_shape, src_for, dst_for = _reshard_geometry(shape, dtype, mesh_size, src_split_axis, dst_split_axis, None)
    plan = _new_plan(rank, src_buffer, dst_buffer, shape, tuple(dst_shape), dtype)
    plan.tensors_involved[dst_buffer] = (torch.Size(dst_shape), dtype)
    if transfer_kind not in {"push", "pull"}:
        raise ValueError("transfer_kind must be 'push' or 'pull'")
    if peer_order not in {"clockwise", "counter-clockwise"}:
        raise ValueError("peer_order must be 'clockwise' or 'counter-clockwise'")
    peers = _ordered_peers(rank, mesh_size, peer_order, include_self=False)
    return _exchange(plan, rank=rank, peers=peers, mesh_size=mesh_size, src_buffer=src_buffer,
                     dst_buffer=dst_buffer, src_for=src_for, dst_for=dst_for, transfer_kind=transfer_kind,
                     compute_producer=compute_producer)


def build_all_to_all_plan_dim_waves(
    shape: Sequence[int],
    *,
    dtype: torch.dtype,
    mesh_size: int,
    rank: int,
    src_buffer: str,
    dst_buffer: str,
    src_split_axis: int,
    dst_split_axis: int,
    num_waves: int,
    transfer_kind: Literal["push", "pull"] = "push",
    compute_producer: bool = False,
    peer_order: Literal["clockwise", "counter-clockwise"] = "clockwise",
) -> DevicePlan:
    """Reshard as above, cut into ``num_waves`` slices along ``dst_split_axis`` so that receivers
    can start on early slices; the local slab is treated like any peer (a LOCAL_COPY per wave)."""
    if mesh_size <= 0:
        raise ValueError("mesh_size must be positive")
    if dtype.itemsize <= 0:
        raise ValueError("elem_size must be positive")
    if num_waves <= 0:
        raise ValueError("num_waves must be positive")
    shape = _check_common(shape, dtype, mesh_size)
    dst_shape, src_for, dst_for = _reshard_geometry(
        shape, dtype, mesh_size, src_split_axis, dst_split_axis, num_waves
    )
    plan = _new_plan(rank, src_buffer, dst_buffer, shape, tuple(dst_shape), dtype)
    plan.tensors_involved[dst_buffer] = (torch.Size(dst_shape), dtype)
    plan.local_regions.setdefault(src_buffer, []).append(src_for(rank))
    if transfer_kind not in {"push", "pull"}:
        raise ValueError("transfer_kind must be 'push' or 'pull'")
    if peer_order not in {"clockwise", "counter-clockwise"}:
        raise ValueError("peer_order must be 'clockwise' or 'counter-clockwise'")
    peers = _ordered_peers(rank, mesh_size, peer_order, include_self=True)
    for wave in range(num_waves):
        for peer in peers:
            if peer == rank:
                waits = _after_compute(rank, src_for(rank, wave)) if compute_producer else []
                plan.add_op(
                    Transfer(
                        op=TransferOp.LOCAL_COPY,
                        src_buf=src_buffer,
                        dst_buf=dst_buffer,
                        src_region=src_for(rank, wave),
                        dst_region=dst_for(rank, wave),
                        chunk_idx=(rank * mesh_size + rank) * num_waves + wave,
                        dependency=waits,
                    )
                )
            elif transfer_kind == "push":
                waits = _after_compute(rank, src_for(peer, wave)) if compute_producer else []
                plan.add_op(
                    Transfer(
                        op=TransferOp.PUSH,
                        src_buf=src_buffer,
                        src_region=src_for(peer, wave),
                        peer=peer,
                        chunk_idx=(rank * mesh_size + peer) * num_waves + wave,
                        dst_buf=dst_buffer,
                        dst_region=dst_for(rank, wave),
                        dependency=waits,
                    )
                )
            else:
                waits = _after_compute(peer, src_for(rank, wave), explicit_none=False) if compute_producer else []
                plan.add_op(
                    Transfer(
                        op=TransferOp.PULL,
                        dst_buf=dst_buffer,
                        dst_region=dst_for(peer, wave),
                        peer=peer,
                        chunk_idx=(peer * mesh_size + rank) * num_waves + wave,
                        src_buf=src_buffer,
                        src_region=src_for(rank, wave),
                        dependency=waits,
                    )
                )
    return plan


def build_all_to_all_plan_axis(
    shape: Sequence[int],
    *,
    dtype: torch.dtype,
    mesh_size: int,
    rank: int,
    src_buffer: str,
    dst_buffer: str,
    split_axis: int,
    transfer_kind: Literal["push", "pull"] = "push",
    compute_producer: bool = False,
) -> DevicePlan:
    """All-to-all along one axis with identical source and destination shapes: slab p of
    ``split_axis`` goes to rank p and lands in slab ``source_rank`` there."""
    shape = _check_common(shape, dtype, mesh_size)
    es = dtype.itemsize
    ax = normalize_axis(split_axis, len(shape))
    ensure_divisible(shape[ax], mesh_size, axis=ax)
    chunk = shape[ax] // mesh_size
    if chunk == 0:
        raise ValueError("all-to-all requires non-empty slices along the split axis")
    if block_nbytes(shape, es, {ax: chunk}) == 0:
        raise ValueError("all-to-all transfer would be empty")
    strides = row_major_strides(shape)
    slab = lambda i: box_region(shape, es, strides, {ax: (i * chunk, (i + 1) * chunk)})
    plan = _new_plan(rank, src_buffer, dst_buffer, shape, shape, dtype)
    if transfer_kind not in {"push", "pull"}:
        raise ValueError("transfer_kind must be 'push' or 'pull'")
    peers = [(rank + i) % mesh_size for i in range(1, mesh_size)]
    return _exchange(plan, rank=rank, peers=peers, mesh_size=mesh_size, src_buffer=src_buffer,
                     dst_buffer=dst_buffer, src_for=slab, dst_for=slab, transfer_kind=transfer_kind,
                     compute_producer=compute_producer)


__all__ = [
    "build_all_to_all_plan",
    "build_all_to_all_plan_dim",
    "build_all_to_all_plan_dim_waves",
    "build_all_to_all_plan_axis",
]
