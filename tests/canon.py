"""Canonical (JSON-able) form of front-end objects, shared by the golden-vector generator and the
parity tests.  Works on objects of either implementation (this package or the reference), since it
only reads public attributes."""
from __future__ import annotations

import hashlib
import json
from typing import Any, Dict, List

MAX_INLINE_SEGMENTS = 16


def region(r) -> Any:
    if r is None:
        return None
    segs = [[s.offset, s.nbytes] for s in r.to_segments()]
    out = {
        "boxes": [[[a.start, a.end] for a in box] for box in r.regions],
        "elem_size": r.elem_size,
        "strides": list(r.strides),
        "base_offset": r.base_offset,
        "num_segments": len(segs),
        "total_nbytes": r.total_nbytes(),
    }
    if len(segs) <= MAX_INLINE_SEGMENTS:
        out["segments"] = segs
    else:
        out["segments_sha"] = hashlib.sha256(json.dumps(segs).encode()).hexdigest()[:16]
    return out


def signal(s) -> Any:
    if s is None:
        return None
    return [s.dst_rank, s.dst_offset, s.type.value, s.period.start]


def dependency(d) -> Any:
    name = type(d).__name__
    if name == "XferDependency":
        return ["xfer", d.depend_rank, d.depend_xfer_stream, d.depend_xfer_idx, signal(d.signal)]
    return ["compute", d.compute_rank, region(d.src_region), signal(d.signal)]


def comm_op(op) -> Any:
    base = {
        "kind": type(op).__name__,
        "op": op.op.value,
        "src_buf": op.src_buf,
        "dst_buf": op.dst_buf,
        "src_region": region(op.src_region),
        "dst_region": region(op.dst_region),
        "deps": [dependency(d) for d in op.dependency],
        "set_signals": [signal(s) for s in op.set_signals],
        "period": [op.period.start, op.period.duration],
    }
    if type(op).__name__ == "Transfer":
        base["chunk_idx"] = op.chunk_idx
        base["peer"] = op.peer
        base["reduce_op"] = None if op.reduce_op is None else op.reduce_op.name
    return base


def device_plan(p) -> Any:
    return {
        "dev": p.dev,
        "streams": [[comm_op(op) for op in ops] for ops in p.xfer],
        "local_regions": {k: [region(r) for r in v] for k, v in p.local_regions.items()},
        "tensors": {k: [list(s), str(d)] for k, (s, d) in p.tensors_involved.items()},
        "transit": [[signal(a), signal(b)] for a, b in p.transit_signals],
        "pretty": p.pretty(),
    }


def info_op(op) -> Any:
    name = type(op).__name__
    if name == "CopyEngineOp":
        return [name, op.src, op.dst, op.src_rank, op.dst_rank, op.src_offset, op.dst_offset, op.size]
    if name == "SMCopyOp":
        return [
            name, op.src, op.dst, op.src_rank, op.dst_rank,
            [[a.start, a.end] for a in op.src_slice], [[a.start, a.end] for a in op.dst_slice],
            None if op.reduce_op is None else op.reduce_op.name, op.use_tma,
        ]
    if name == "CollectiveComm":
        return [
            name, op.op.value, op.src, op.dst,
            [[a.start, a.end] for a in op.src_slice], [[a.start, a.end] for a in op.dst_slice],
        ]
    return [name, op.signal_type.value, op.offset, op.rank]


def comm_info(info, max_ops_inline: int = 64) -> Any:
    ops = [[[info_op(op) for op in stream] for stream in rank] for rank in info.operations]
    out = {
        "world_size": info.world_size,
        "recv": info.recv_signal_num,
        "transit": info.transit_signal_num,
        "compute": info.compute_signal_num,
        "buffers": {k: [list(s), str(d)] for k, (s, d) in info.comm_buffer_sizes.items()},
        "ops_per_rank": [sum(len(s) for s in rank) for rank in ops],
    }
    if max(out["ops_per_rank"], default=0) <= max_ops_inline:
        out["operations"] = ops
    else:
        out["operations_sha"] = hashlib.sha256(json.dumps(ops).encode()).hexdigest()[:16]
    return out


def raw_schedule(s) -> Any:
    blocks = [b for wave in s.block_infos for b in wave]
    return {
        "num_waves": s.num_waves,
        "wave_lens": [len(w) for w in s.block_infos],
        "global_shape": list(s.global_shape),
        "offsets": s.gen_block_offset_lists(),
        "shapes": s.gen_block_shape_lists(),
        "signals": s.gen_signal_lists(),
        "targets": s.gen_target_rank_list(),
        "dst_offsets": s.gen_dst_offset_lists(),
        "signal_types": [None if b.signal is None else b.signal.type.value for b in blocks],
        "signal_ranks": [None if b.signal is None else b.signal.dst_rank for b in blocks],
        "roles": [b.role for b in blocks],
        "reduce": [None if b.reduce_op is None else b.reduce_op.name for b in blocks],
        "is_reduce": s.is_reduce(),
    }


def lowered(low) -> Any:
    return {str(dev): {buf: raw_schedule(s) for buf, s in sorted(per.items())} for dev, per in sorted(low.items())}
