"""Host logic that joins the front end's outputs (CommInfo op program + lowered RawSchedules) into
the per-wave arguments of the fused GEMM kernels."""
from __future__ import annotations

from typing import Dict, List, Sequence


def push_completion_signals(comm_info, rank: int) -> Dict[int, List[int]]:
    """For the op program of ``rank``: first-axis start of every pushed / copied source box ->
    ``[dst_rank, flag index raised on dst_rank]``, read off the copy op and the signal ops that
    follow it (the order ``generate_code_for_plan`` emits: waits, body, signals)."""
    out: Dict[int, List[int]] = {}
    for stream in comm_info.operations[rank]:
        pending = None
        for op in stream:
            kind = type(op).__name__
            if kind == "SMCopyOp":
                pending = (op.src_slice[0].start, op.dst_rank)
            elif kind == "CopyEngineOp":
                if pending is None or pending[1] != op.dst_rank or pending[2:] != ("ce",):
                    pending = (op.src_offset, op.dst_rank, "ce")
            elif kind == "IntraNodeSignal" and pending is not None:
                if op.rank == pending[1] and pending[0] not in out:
                    out[pending[0]] = [op.rank, op.offset]
                pending = None
            elif kind == "WaitIntraNodeSignal":
                pending = None
    return out


def rs_remote_signals(comm_info, rank: int, src_schedule) -> List[int]:
    """Per wave of the partial-C schedule: the flag index to raise on the wave's target rank
    (-1 for the wave kept locally)."""
    table = push_completion_signals(comm_info, rank)
    offsets = src_schedule.gen_block_offset_lists()
    targets = src_schedule.gen_target_rank_list()
    out = []
    for off, tgt in zip(offsets, targets):
        hit = table.get(off[0])
        if tgt < 0 or tgt == rank or hit is None or hit[0] != tgt:
            out.append(-1)
        else:
            out.append(hit[1])
    return out


def rs_transport_program(rank: int, world: int, slab_rows: int, row_bytes: int, epoch: int, src_schedule,
                         remote_signals, send_ptr: int, send_flags_ptr: int, stage_ptrs, flag_ptrs):
    """What moves the slabs of a GEMM + reduce-scatter call when the kernel stores them locally
    (``syn_gemm_rs_args.send_buf``): one entry per wave of the partial-C schedule whose target is
    another rank, in wave order,

        ``(local flag address, source address, destination address, bytes, remote flag address)``

    A wave is a run of rows of its target's slab (the whole slab, or one piece of it when the plan
    was cut into smaller chunks).  The source is those rows of slab ``target`` of the local send
    buffer and the local flag word is the wave's own (index = wave index); the destination is the
    same rows of slot ``(epoch & 1) * world + rank`` of the target's staging buffer (the half
    alternates with the epoch so that a rank one call ahead does not overwrite what a slower rank
    still reads) and the remote flag the one the target's reduce wave for these rows waits for."""
    half = (epoch & 1) * world
    slab_bytes = slab_rows * row_bytes
    prog = []
    offsets, shapes = src_schedule.gen_block_offset_lists(), src_schedule.gen_block_shape_lists()
    for w, tgt in enumerate(src_schedule.gen_target_rank_list()):
        tgt = rank if tgt is None or tgt < 0 else int(tgt)
        if tgt == rank or remote_signals[w] < 0:
            continue
        row_in_slab = offsets[w][0] - tgt * slab_rows
        inner = row_in_slab * row_bytes
        prog.append((send_flags_ptr + 8 * w,
                     send_ptr + tgt * slab_bytes + inner,
                     stage_ptrs[tgt] + (half + rank) * slab_bytes + inner,
                     shapes[w][0] * row_bytes,
                     flag_ptrs[tgt] + 8 * int(remote_signals[w])))
    return prog


__all__ = ["push_completion_signals", "rs_remote_signals", "rs_transport_program"]


def tile_order(wave_offsets, wave_sizes, block_m: int = 128, block_n: int = 256, group_size_m: int = 8):
    """Host model of the kernel's tile scheduler: the ``(pid_m, pid_n)`` sequence for global tile
    ids 0, 1, 2, ...  Waves are walked in array order; inside a wave the grouped raster of
    syncopate/computation/gemm/template.py:10-18 applies to the wave's own tile grid, then the
    wave's offset is added (:130-136).  Offsets and sizes are in elements."""
    order = []
    for (off_m, off_n), (size_m, size_n) in zip(wave_offsets, wave_sizes):
        tm, tn = -(-size_m // block_m), -(-size_n // block_n)
        for local in range(tm * tn):
            in_group = group_size_m * tn
            group_id, r = divmod(local, in_group)
            first_m = group_id * group_size_m
            gsz = min(tm - first_m, group_size_m)
            order.append((first_m + r % gsz + off_m // block_m, r // gsz + off_n // block_n))
    return order


__all__ += ["tile_order"]
