"""Host logic that turns the front end's outputs into the arguments of the attention kernel:

* wave metadata over (Z, H, Q, KV) derived from a lowered RawSchedule, restating the two
  derivations the reference's drivers use (all-to-all: tests/test_all2all_attn_transform.py:58-117;
  KV all-gather: tests/test_double_ring_ag_attn.py:60-81),
* the comm warps' 2-D copy list derived from the same schedule (N-D boxes cut into runs that are
  contiguous on both sides, then grouped into rows with constant pitches),
* position tables for zigzag context parallelism.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

from syncopate_b200 import _lib as L


# --------------------------------------------------------------------------- wave metadata
def _runs_of(slabs):
    """``[(offset, length)]`` sorted by offset -> the maximal contiguous runs ``[(offset, length)]``."""
    out = []
    for off, n in sorted(slabs):
        if out and out[-1][0] + out[-1][1] == off:
            out[-1] = (out[-1][0], out[-1][1] + n)
        else:
            out.append((off, n))
    return out


def all_to_all_wave_metadata(schedule, axes: Dict[str, int], causal: bool = False, join: bool = False):
    """Waves for attention fed by a sequence all-to-all.  Slab n (Q, K and V rows of one source rank)
    arrives with flag n; once it is there the kernel can run (Q_n, KV_n) and, for every earlier slab
    j, (Q_j, KV_n) and (Q_n, KV_j).  Returns ``(offsets, shapes, signals, cum_rows)`` with 4-entry
    rows (z, h, q, kv) in tokens; ``cum_rows`` counts Z * H * Q rows as the reference does.

    ``causal`` (positions = sequence offsets): a pair whose keys all lie behind its queries does no
    work, so slab n only brings (Q_n, KV of every arrived slab at or below n) - one wave per
    contiguous key range - and (Q of the arrived slabs above n, KV_n) - one wave per contiguous
    query range.  All of them are gated by flag n, which implies the flags of the slabs that arrived
    before (the comm warps walk the op list in order).  A query tile is then visited once per slab
    that arrives after its own instead of once per slab.  ``join`` without ``causal``: the same
    joining with every arrived slab on both sides (slab n's queries against all arrived keys, the
    earlier slabs' queries against its keys)."""
    offs_src = schedule.gen_block_offset_lists()
    shp_src = schedule.gen_block_shape_lists()
    sig_src = schedule.gen_signal_lists()
    b, h, s = axes["batch"], axes["head"], axes["seq"]
    offsets, shapes, signals, cum = [], [], [], []
    total = 0
    if causal or join:
        for n in range(len(shp_src)):
            on, sn = offs_src[n], shp_src[n]
            # slabs whose keys slab n's queries see / whose queries see slab n's keys
            below = [(offs_src[j][s], shp_src[j][s]) for j in range(n) if not causal or offs_src[j][s] < on[s]]
            above = [(offs_src[j][s], shp_src[j][s]) for j in range(n) if not causal or offs_src[j][s] > on[s]]
            for k_off, k_len in _runs_of(below + [(on[s], sn[s])]):
                offsets.append([on[b], on[h], on[s], k_off])
                shapes.append([sn[b], sn[h], sn[s], k_len])
                signals.append(sig_src[n])
                total += sn[b] * sn[h] * sn[s]
                cum.append(total)
            for q_off, q_len in _runs_of(above):
                offsets.append([on[b], on[h], q_off, on[s]])
                shapes.append([sn[b], sn[h], q_len, sn[s]])
                signals.append(sig_src[n])
                total += sn[b] * sn[h] * q_len
                cum.append(total)
        return offsets, shapes, signals, cum

    def emit(q_wave, kv_wave, sig):
        nonlocal total
        oq, sq = offs_src[q_wave], shp_src[q_wave]
        ok, sk = offs_src[kv_wave], shp_src[kv_wave]
        offsets.append([oq[b], oq[h], oq[s], ok[s]])
        shapes.append([sq[b], sq[h], sq[s], sk[s]])
        signals.append(sig)
        total += sq[b] * sq[h] * sq[s]
        cum.append(total)

    for n in range(len(shp_src)):
        emit(n, n, sig_src[n])
        for j in range(n):
            emit(j, n, sig_src[n])
            emit(n, j, sig_src[n])
    return offsets, shapes, signals, cum


def all_gather_wave_metadata(schedule, q_rows: int, axes: Dict[str, int], q_heads: Optional[int] = None):
    """Waves for attention over an all-gathered KV buffer: one wave per KV chunk, every local query
    row attends to the chunk once its flag is up.  ``q_heads`` overrides the head extent for
    grouped-query attention (the KV buffer has fewer heads than Q)."""
    b, h, s = axes["batch"], axes["head"], axes["seq"]
    offsets, shapes, cum = [], [], []
    total = 0
    for off, shp in zip(schedule.gen_block_offset_lists(), schedule.gen_block_shape_lists()):
        heads = q_heads if q_heads is not None else shp[h]
        head0 = 0 if q_heads is not None else off[h]
        offsets.append([off[b], head0, 0, off[s]])
        shapes.append([shp[b], heads, q_rows, shp[s]])
        total += shp[b] * heads * q_rows
        cum.append(total)
    return offsets, shapes, schedule.gen_signal_lists(), cum


def merge_wave_tail(waves, keep: int):
    """Joins the waves behind the first ``keep`` into as few waves as their key ranges allow: waves
    that follow each other, cover the same (batch, head, query) box and whose key ranges are
    adjacent in the buffer become one wave over the joined range, gated by the flag of the LAST of
    them.  That flag implies the earlier ones when the chunks arrive in wave order (the comm warps
    walk the rank's op list in order, and a chunk's flag rises only after every CTA has finished
    its pieces of it).  Fewer waves = fewer visits of every query tile (one Q load, one merge through
    the stored O per visit); the price is that the joined wave starts after its last chunk, which
    is free once the transfers run ahead of the attention, i.e. for all but the first few waves.
    ``waves`` = ``(offsets, shapes, signals, cum)`` as built by ``all_gather_wave_metadata``."""
    offsets, shapes, signals, cum = waves
    n = len(offsets)
    if keep < 0 or keep >= n - 1:
        return waves
    out_o, out_s, out_g, out_c = [list(o) for o in offsets[:keep]], [list(x) for x in shapes[:keep]], list(signals[:keep]), list(cum[:keep])
    i = keep
    while i < n:
        o, sh, g = list(offsets[i]), list(shapes[i]), signals[i]
        j = i + 1
        while j < n and offsets[j][:3] == o[:3] and shapes[j][:3] == sh[:3] and signals[j] >= 0:
            if offsets[j][3] == o[3] + sh[3]:          # next chunk continues this range upwards
                sh[3] += shapes[j][3]
            elif offsets[j][3] + shapes[j][3] == o[3]:  # or downwards
                o[3] = offsets[j][3]
                sh[3] += shapes[j][3]
            else:
                break
            g = signals[j]
            j += 1
        out_o.append(o)
        out_s.append(sh)
        out_g.append(g)
        out_c.append(cum[j - 1])
        i = j
    return out_o, out_s, out_g, out_c


# --------------------------------------------------------------------------- box copies
def _strides(shape: Sequence[int]) -> List[int]:
    out, acc = [], 1
    for n in reversed(shape):
        out.append(acc)
        acc *= n
    return out[::-1]


def _runs(shape: Sequence[int], offsets: Sequence[int], extent: Sequence[int], elem: int) -> Tuple[List[int], int]:
    """Byte offsets of the contiguous runs of a box inside a row-major tensor, and the run length."""
    strides = _strides(shape)
    nd = len(shape)
    run = elem
    k = nd
    while k > 0 and strides[k - 1] * elem == run:
        run *= extent[k - 1]
        k -= 1
    base = sum(o * st for o, st in zip(offsets[k:], strides[k:])) * elem
    starts = [base]
    for ax in range(k):
        step = strides[ax] * elem
        starts = [b0 + (offsets[ax] + i) * step for b0 in starts for i in range(extent[ax])]
    return starts, run


def box_copy_ops(src_shape, src_off, dst_shape, dst_off, extent, elem: int) -> List[Tuple[int, int, int, int, int, int]]:
    """Cuts the copy of one N-D box (same ``extent`` on both sides) into 2-D strided copies
    ``(src_offset, dst_offset, rows, row_bytes, src_pitch, dst_pitch)``, all in bytes."""
    s_starts, s_run = _runs(src_shape, src_off, extent, elem)
    d_starts, d_run = _runs(dst_shape, dst_off, extent, elem)
    piece = min(s_run, d_run)
    if s_run % piece or d_run % piece:
        raise ValueError("source and destination runs of the box do not nest")
    src = [b0 + i * piece for b0 in s_starts for i in range(s_run // piece)]
    dst = [b0 + i * piece for b0 in d_starts for i in range(d_run // piece)]
    if len(src) != len(dst):
        raise ValueError("source and destination boxes differ in size")
    ops = []
    i, n = 0, len(src)
    while i < n:
        rows = 1
        if i + 1 < n:
            ds, dd = src[i + 1] - src[i], dst[i + 1] - dst[i]
            while i + rows < n and src[i + rows] - src[i + rows - 1] == ds and dst[i + rows] - dst[i + rows - 1] == dd:
                rows += 1
        else:
            ds = dd = 0
        if rows == 1:
            ds = dd = 0
        # a run of rows that is contiguous on both sides is one long row
        if rows > 1 and ds == piece and dd == piece:
            ops.append((src[i], dst[i], 1, piece * rows, 0, 0))
        else:
            ops.append((src[i], dst[i], rows, piece, ds, dd))
        i += rows
    return ops


def pull_ops_from_schedule(schedule, rank: int, world: int, src_shape, dst_shape, elem: int,
                           src_buf: int, dst_buf: int, gather_axis: Optional[int] = None) -> List[L.CopyOp]:
    """Copy list that fills this rank's destination buffer in the order of its lowered schedule.

    Each scheduled block is fetched from the rank that holds it - the block's peer, reading at the
    block's peer-side offsets; or, when ``gather_axis`` is given (all-gather of one buffer, ring and
    double-ring plans included), the owner of that slab of the gathered axis at the same offsets -
    and raises the block's flag on this rank when it has landed.  Blocks without a flag that are
    already resident are skipped."""
    ops: List[L.CopyOp] = []
    offs = schedule.gen_block_offset_lists()
    shps = schedule.gen_block_shape_lists()
    sigs = schedule.gen_signal_lists()
    tgts = schedule.gen_target_rank_list()
    peer_offs = schedule.gen_dst_offset_lists()
    for off, shp, sig, tgt, poff in zip(offs, shps, sigs, tgts, peer_offs):
        if gather_axis is not None:
            slab = dst_shape[gather_axis] // world
            owner = off[gather_axis] // slab
            if owner == rank:
                continue  # resident
            src_rank, src_off = owner, off
        else:
            src_rank = rank if tgt < 0 else tgt
            src_off = poff
        pieces = box_copy_ops(src_shape, src_off, dst_shape, off, shp, elem)
        for i, (so, do, rows, row_bytes, sp, dp) in enumerate(pieces):
            op = L.CopyOp()
            op.src_rank, op.dst_rank = src_rank, rank
            op.src_buf, op.dst_buf = src_buf, dst_buf
            op.src_offset, op.dst_offset = so, do
            op.src_pitch, op.dst_pitch = sp, dp
            op.rows, op.row_bytes = rows, row_bytes
            last = i == len(pieces) - 1
            op.flag_rank = rank
            op.flag = sig if (last and sig >= 0) else -1  # ops run in order: the last piece publishes the block
            ops.append(op)
    return ops


def push_ops_from_schedule(schedule, rank: int, src_shape, dst_shape, elem: int, src_buf: int, dst_buf: int,
                           remote_signals: Sequence[int]) -> List[L.CopyOp]:
    """Copy list that sends this rank's blocks of a compute-produced buffer to their targets in the
    order of the lowered schedule (target = receiving rank, peer-side offsets = where the block
    lands there); a block without a target is copied to this rank's own destination buffer.  The
    last piece of each block raises ``remote_signals[i]`` on the receiving rank."""
    ops: List[L.CopyOp] = []
    rows = zip(schedule.gen_block_offset_lists(), schedule.gen_block_shape_lists(), schedule.gen_target_rank_list(),
               schedule.gen_dst_offset_lists(), remote_signals)
    for off, shp, tgt, poff, rsig in rows:
        dst_rank = rank if tgt < 0 else tgt
        pieces = box_copy_ops(src_shape, off, dst_shape, poff, shp, elem)
        for i, (so, do, nrows, row_bytes, sp, dp) in enumerate(pieces):
            op = L.CopyOp()
            op.src_rank, op.dst_rank = rank, dst_rank
            op.src_buf, op.dst_buf = src_buf, dst_buf
            op.src_offset, op.dst_offset = so, do
            op.src_pitch, op.dst_pitch = sp, dp
            op.rows, op.row_bytes = nrows, row_bytes
            op.flag_rank = dst_rank
            op.flag = rsig if (i == len(pieces) - 1 and rsig >= 0) else -1
            ops.append(op)
    return ops


def completion_signals(comm_info, rank: int, schedule) -> List[int]:
    """Per block of ``schedule`` (a compute-produced buffer of ``rank``): the flag index that the
    op program raises on the receiving rank once the block's copy is done (local copies included),
    read off ``comm_info.operations[rank]``: copy op(s) followed by their signal op(s)."""
    table = {}
    for stream in comm_info.operations[rank]:
        pending = None
        for op in stream:
            kind = type(op).__name__
            if kind == "SMCopyOp":
                pending = (tuple(a.start for a in op.src_slice), op.dst_rank)
            elif kind == "IntraNodeSignal" and pending is not None:
                if op.rank == pending[1]:
                    table.setdefault(pending, op.offset)
                pending = None
            elif kind == "WaitIntraNodeSignal":
                pending = None
    out = []
    for off, tgt in zip(schedule.gen_block_offset_lists(), schedule.gen_target_rank_list()):
        out.append(table.get((tuple(off), rank if tgt < 0 else tgt), -1))
    return out


def zigzag_tables(world: int, rank: int, seq_total: int, block: int = 128):
    """Position tables for zigzag context parallelism with ``2 * world`` chunks: rank r holds chunks
    r and 2 * world - 1 - r (queries: local rows in that order; keys: the gathered buffer is laid
    out rank after rank).  Returns ``(q_pos, kv_pos)`` lists with one entry per ``block`` rows."""
    chunk = seq_total // (2 * world)

    def rank_positions(r):
        return [r * chunk + i for i in range(0, chunk, block)] + [
            (2 * world - 1 - r) * chunk + i for i in range(0, chunk, block)
        ]

    q_pos = rank_positions(rank)
    kv_pos = [p for r in range(world) for p in rank_positions(r)]
    return q_pos, kv_pos


__all__ = [
    "all_to_all_wave_metadata",
    "all_gather_wave_metadata",
    "merge_wave_tail",
    "box_copy_ops",
    "pull_ops_from_schedule",
    "push_ops_from_schedule",
    "completion_signals",
    "zigzag_tables",
]
