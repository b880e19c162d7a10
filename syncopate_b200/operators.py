"""The fused operators as objects: plan once (front end), allocate symmetric state once, call many
times.  Each object does, for one rank, what the reference's test drivers do by hand
(tests/test_ag_gemm_gen.py:120-176, tests/test_gemm_rs_direct_reduce.py:120-189): build every
rank's plan, plan signals, generate the op program, lower to schedules, allocate the symmetric
buffers and flags, then launch the fused kernel with this rank's schedule.

Flags carry an epoch that grows by one per call, so nothing is reset between calls; the one
synchronisation per call is the device-side barrier described in the operators' docstrings.
"""
from __future__ import annotations

from typing import Optional

import torch

from .communication.code_gen import CodeGenOptions, CommGenerator
from . import _lib as _L
from .communication.common_descriptors import (
    build_all_gather_plan_1d_swizzle,
    build_all_to_all_plan,
    build_reduce_scatter_direct_reduce_plan,
    build_ring_all_gather_plan,
    split_transfers_along_axis,
)
from .computation.gemm import ag_gemm, gemm, gemm_rs
from .computation.gemm.plan import rs_remote_signals, rs_transport_program
from .interface import lower_comm_plan_to_raw_schedules
from .runtime import SymmetricContext

def _raw_lib():
    from . import _lib

    return _lib.lib()


NUM_COUNTERS = 130  # SYN_NUM_COUNTERS: wave counters, copy counters, tile scheduler


def plan_all_gather(world: int, rows_per_rank: int, K: int, dtype: torch.dtype, kind: str = "swizzle",
                    copy_engine: bool = False, chunk_split: int = 1, transfer: str = "pull"):
    """(generator, comm_info, lowered) for gathering ``[rows_per_rank, K]`` shards along dim 0.
    ``chunk_split`` > 1 cuts every remote slab into that many row pieces, each with a flag and a
    wave of its own (``split_transfers_along_axis``)."""
    shape = (rows_per_rank * world, K)
    if kind == "swizzle":
        plans = {r: build_all_gather_plan_1d_swizzle(shape, dtype, 0, world, r, "a", transfer) for r in range(world)}
    elif kind == "ring":
        plans = {r: build_ring_all_gather_plan(shape, dtype, 0, world, r, "a") for r in range(world)}
    else:
        raise ValueError("kind must be 'swizzle' or 'ring'")
    if chunk_split > 1:
        plans = {r: split_transfers_along_axis(pl, chunk_split, 0) for r, pl in plans.items()}
    gen = CommGenerator(plans)
    gen.plan_signals(plan_compute_signals=True)
    info = gen.generate_code_for_plan(CodeGenOptions(copy_engine=copy_engine))
    return gen, info, lower_comm_plan_to_raw_schedules(gen)


def plan_reduce_scatter(world: int, M: int, N: int, dtype: torch.dtype, kind: str = "direct", chunk_split: int = 1):
    """(generator, comm_info, lowered) for reduce-scattering a partial ``[M, N]`` along dim 0.
    ``chunk_split`` > 1 sends every slab as that many row pieces."""
    if kind == "direct":
        plans = {
            r: build_reduce_scatter_direct_reduce_plan(
                (M, N), dtype=dtype, axis=0, mesh_size=world, rank=r, src_buffer="src", dst_buffer="dst"
            )
            for r in range(world)
        }
    elif kind == "a2a":
        plans = {
            r: build_all_to_all_plan(
                (M, N), dtype=dtype, mesh_size=world, rank=r, src_buffer="src", dst_buffer="dst",
                transfer_kind="push", compute_producer=True,
            )
            for r in range(world)
        }
    else:
        raise ValueError("kind must be 'direct' or 'a2a'")
    if chunk_split > 1:
        if kind != "direct":
            raise ValueError("chunk_split needs the direct plan (its source and destination rows share one axis)")
        plans = {r: split_transfers_along_axis(pl, chunk_split, 0) for r, pl in plans.items()}
    gen = CommGenerator(plans)
    gen.plan_signals(plan_compute_signals=True)
    info = gen.generate_code_for_plan(CodeGenOptions(copy_engine=False))
    return gen, info, lower_comm_plan_to_raw_schedules(gen)


_HAZARD_NOTE = """

    **Who may write what, and when.**  Peers read this rank's symmetric input (and write its
    symmetric output) directly.  With ``lockstep=True`` (default) every call starts with a
    device-side barrier over all ranks, placed so that no transfer of the call starts before every
    rank has entered it: whatever a rank wrote into its symmetric input *before* the call, in stream
    order, is what the peers see.  Nothing in a call tells a rank when the peers are done with that
    input: rewrite it only after a barrier that follows the call (``ctx.barrier()`` on the same
    stream), or construct the operator with ``sync_after=True``, which ends every call with a
    second barrier so that inputs may be rewritten and outputs read as soon as the call has
    returned in stream order.  With ``lockstep=False`` the caller provides both guarantees."""


class AllGatherGemm:
    """``C[rows * world, N] = all_gather(A_shard)[rows * world, K] @ B[N, K]^T`` per rank.

    ``comm="sm"``: the kernel's comm warps pull the chunks (``CodeGenOptions(copy_engine=False)``
    program); ``comm="ce"``: the rank's copy-engine program (``copy_engine=True``) runs on side
    streams while the flag-gated GEMM runs on the caller's stream, as in the reference's
    tests/test_ag_gemm_gen.py:44-77.  ``chunk_split`` cuts every remote slab into row pieces with
    flags of their own: the first tiles of a slab start after a piece has arrived instead of the
    whole slab, and the step ends one piece's GEMM after the last arrival."""

    __doc__ += _HAZARD_NOTE

    def __init__(self, ctx: SymmetricContext, rows_per_rank: int, K: int, N: int, dtype=torch.bfloat16,
                 plan: str = "swizzle", num_sms: int = 0, block_n: int = 0, timeout_ns: int = 0, comm: str = "sm",
                 copy_streams: int = 1, lockstep=True, chunk_split: int = 1, sync_after: bool = False,
                 transfer: str = "pull", flag_stream: bool = True):
        """``transfer`` (copy-engine mode): ``"pull"`` - every rank's copy engines fetch the peers' slabs;
        ``"push"`` - every rank's copy engines write its slab into the peers' buffers and raise the
        peers' flags (the swizzled plan in its push form)."""
        if comm not in ("sm", "ce"):
            raise ValueError("comm must be 'sm' or 'ce'")
        if transfer not in ("pull", "push") or (transfer == "push" and (comm != "ce" or plan != "swizzle")):
            raise ValueError("transfer='push' needs the swizzled plan moved by copy engines")
        self.ctx = ctx
        self.world, self.rank = ctx.world, ctx.rank
        self.rows, self.K, self.N, self.dtype = rows_per_rank, K, N, dtype
        self.M = rows_per_rank * self.world
        self.num_sms, self.block_n, self.timeout_ns = num_sms, block_n, timeout_ns
        self.comm = comm
        # The swizzled order gives every rank a different peer at every step only while the ranks
        # move in step; free-running ranks drift, two of them then load the same peer's link and
        # the transfers slow down.  A device-side barrier at the start of each call keeps them
        # aligned (and orders the peers' shard writes before the pulls).
        # lockstep="pairwise" (copy-engine pulls only): no barrier; every rank tells every peer that it
        # has entered the call (a flag write per peer) and a pull from peer p waits for p's word only,
        # so that a pull from a rank that is already there does not wait for the slowest rank.
        if lockstep == "pairwise" and (comm != "ce" or transfer != "pull"):
            raise ValueError("lockstep='pairwise' needs copy-engine pulls")
        self.lockstep = lockstep
        self.sync_after = sync_after
        self.chunk_split = chunk_split
        self.generator, self.info, lowered = plan_all_gather(self.world, rows_per_rank, K, dtype, plan,
                                                             copy_engine=(comm == "ce"), chunk_split=chunk_split,
                                                             transfer=transfer)
        self.schedule = lowered[self.rank]["a"]
        self.epoch = 0
        self.trace = None  # optional uint64 stamp buffer handed to the kernel (see syn_gemm_args.trace)
        self.a = ctx.alloc((self.M, K), dtype)
        self.flags = ctx.alloc((max(self.info.recv_signal_num, 1),), torch.int64)
        self.counters = torch.zeros(NUM_COUNTERS, dtype=torch.int32, device=ctx.device)
        if comm == "ce":
            self._wave_offsets = [[o[0], 0] for o in self.schedule.gen_block_offset_lists()]
            self._wave_sizes = [[s[0], N] for s in self.schedule.gen_block_shape_lists()]
            self._signals = self.schedule.gen_signal_lists()
            # Consecutive chunks go round-robin over the copy streams.  Measured on eight GPUs under
            # the running GEMM: ONE stream whose copies run back to back (flags on the flag stream)
            # moves the most bytes per second; copies in flight on several streams slow each other
            # down and delay the first chunk, the one the GEMM waits for.
            self._copy_streams = [torch.cuda.Stream(device=ctx.device) for _ in range(max(1, copy_streams))]
            # flag writes go to a stream of their own (behind an event per copy): a copy stream then
            # runs its copies back to back instead of stopping for a stream memory operation after each
            self._flag_stream = torch.cuda.Stream(device=ctx.device) if flag_stream else None
            self._ev_start = torch.cuda.Event()
            self._ev_go = torch.cuda.Event()
            self._ready = None
            if lockstep == "pairwise" and self.world > 1:
                self._ready = ctx.alloc((self.world,), torch.int64)   # [peer]: the peer's last entered call
                self._announce_stream = torch.cuda.Stream(device=ctx.device)
                hello = [(0, 0, 0, 0, self._ready.symm.ptrs[(self.rank + i) % self.world] + 8 * self.rank, 0)
                         for i in range(1, self.world)]
                self._hello, self._hello_len = _L.make_ce_program(hello), len(hello)
            steps = self.copy_program()
            self._program, self._program_len = _L.make_ce_program(steps), len(steps)

    def copy_program(self):
        """``[(0, dst, src, nbytes, flag or 0, stream index)]``: the rank's copy-engine program (its
        CopyEngineOp records, each group followed by the IntraNodeSignal that publishes it) with all
        addresses resolved; groups go round-robin over the copy streams."""
        steps, pending, group = [], [], 0
        es = self.dtype.itemsize
        assert es == self.a.local.element_size()
        for op in self.info.operations[self.rank][0]:
            kind = type(op).__name__
            if kind == "CopyEngineOp":
                if op.src_rank == op.dst_rank:
                    continue
                pending.append((self.a.symm.ptrs[op.dst_rank] + op.dst_offset, self.a.symm.ptrs[op.src_rank] + op.src_offset,
                                op.size, op.src_rank))
            elif kind == "IntraNodeSignal" and pending:
                flag = self.flags.symm.ptrs[op.rank] + 8 * op.offset
                for i, (dst, src, nbytes, src_rank) in enumerate(pending):
                    wait = self._ready.local.data_ptr() + 8 * src_rank if self._ready is not None else 0
                    steps.append((wait, dst, src, nbytes, flag if i == len(pending) - 1 else 0, group))
                pending = []
                group += 1
        return steps

    @property
    def shard(self) -> torch.Tensor:
        """This rank's slab of the gathered buffer (write the local activations here)."""
        return self.a.local[self.rank * self.rows : (self.rank + 1) * self.rows]

    def __call__(self, b: torch.Tensor, c: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        if c is None:
            c = torch.empty(self.M, self.N, dtype=self.dtype, device=self.ctx.device)
        self.epoch += 1
        if self.world == 1:
            return gemm(self.a.local, b, c, 1, self.num_sms, BLOCK_SIZE_N=self.block_n, status=self.ctx.status,
                        timeout_ns=self.timeout_ns, stream=stream)
        cur = stream or torch.cuda.current_stream()
        if self.comm == "ce":
            # The GEMM starts at once on the caller's stream (its first wave is the resident slab);
            # the barrier sits on the copy streams, in front of the transfers it is there for.
            side = self._copy_streams
            self._ev_start.record(cur)
            side[0].wait_event(self._ev_start)
            if self._ready is not None:
                self._announce_stream.wait_event(self._ev_start)
                _L.ce_run(self._hello, self._hello_len, [self._announce_stream], self.epoch, None)
            elif self.lockstep:
                self.ctx.barrier(side[0])
            self._ev_go.record(side[0])
            for s in side[1:]:
                s.wait_event(self._ev_go)
            _L.ce_run(self._program, self._program_len, side, self.epoch, self._flag_stream)
            gemm(self.a.local, b, c, self.world, self.num_sms, BLOCK_SIZE_N=self.block_n,
                 cur_wave_sizes=self._wave_sizes, wave_offsets=self._wave_offsets, signal_ptr=self.flags.local,
                 signal_offsets=self._signals, signal_value=self.epoch, status=self.ctx.status,
                 timeout_ns=self.timeout_ns, trace=self.trace, stream=cur)
            for s in side:
                cur.wait_stream(s)
            if self._flag_stream is not None:
                cur.wait_stream(self._flag_stream)
            if self._ready is not None:
                cur.wait_stream(self._announce_stream)
        else:
            if self.lockstep:
                self.ctx.barrier(cur)
            ag_gemm(self.a.symm, self.a.local, b, c, self.schedule, self.flags.local, self.counters,
                    epoch=self.epoch, num_sms=self.num_sms, block_n=self.block_n, timeout_ns=self.timeout_ns,
                    status=self.ctx.status, trace=self.trace, stream=cur)
        if self.sync_after:
            self.ctx.barrier(cur)
        return c


class GemmReduceScatter:
    """``out[M / world, N] = sum over ranks of (A_r[M, K_r] @ B_r[N, K_r]^T)[own rows]``.

    Inputs are private to the rank; the symmetric state (staging slabs, flags) is the operator's
    own and alternates with the call's parity, so back-to-back calls need no barrier for
    correctness (a rank can only be two calls ahead of a peer after that peer has read the half it
    overwrites).  ``lockstep`` keeps the ranks' transfers aligned in time (see AllGatherGemm)."""

    def __init__(self, ctx: SymmetricContext, M: int, N: int, dtype=torch.bfloat16, plan: str = "direct",
                 num_sms: int = 0, block_n: int = 0, timeout_ns: int = 0, lockstep: bool = True, comm: str = "sm",
                 copy_streams: int = 2, chunk_split: int = 1, publish_pieces: bool = False, flag_stream: bool = True,
                 reduce: str = "auto"):
        """``comm="sm"``: the GEMM's epilogue stores each tile straight into the target rank's staging
        slab (TMA stores to peer memory).  ``comm="ce"``: the epilogue stores locally and raises a
        local flag per wave; side streams wait for the flag (a stream memory operation), move the
        rows with a copy engine and raise the target's flag.  ``chunk_split`` sends every slab as
        that many row pieces; the rows kept here are then reduced piece by piece as the matching
        pieces arrive.  ``publish_pieces``: the kernel also raises the local flag ``out_flags[g]`` when
        row piece g of the result is complete (for whoever passes the reduced rows on).
        ``reduce="epilogue"``: the tiles of the rows kept here wait for the staged partial sums and
        add them in their epilogue (one kernel).  ``reduce="pass"``: the kernel stores the own partial
        sum and a pass launched behind it adds the staged slabs with coalesced loads (and raises
        ``out_flags``); the own partial sum is then rounded to 16 bits before the sum.  Measured on
        eight GPUs at M = N = 8192, K = 3584 per rank: sm + pass 0.417 ms, ce + pass 0.44-0.46,
        sm + epilogue 0.47, ce + epilogue 0.55 (the reduce waves sit at the end of the kernel, behind
        the last arrival, where nothing overlaps their latency-bound reads)."""
        if comm not in ("sm", "ce"):
            raise ValueError("comm must be 'sm' or 'ce'")
        if reduce not in ("auto", "epilogue", "pass"):
            raise ValueError("reduce must be 'auto', 'epilogue' or 'pass'")
        # "auto": the pass pays once seven slabs are staged (eight ranks: 0.40 ms against 0.47); with one
        # or three staged slabs and waves that are long against a transfer the epilogue form is level
        # or ahead (two ranks 1.49 against 1.62 ms, four ranks 0.71 against 0.71-0.79)
        if reduce == "auto":
            reduce = "pass" if ctx.world >= 6 else "epilogue"
        self.reduce = reduce
        self.reduce_pass = reduce == "pass"
        self.ctx = ctx
        self.comm = comm
        self.lockstep = lockstep
        self.world, self.rank = ctx.world, ctx.rank
        self.M, self.N, self.dtype = M, N, dtype
        self.pieces = max(int(chunk_split), 1)   # row pieces of the slab kept here
        self.out_flags = None
        self.slab = M // self.world
        self.num_sms, self.block_n, self.timeout_ns = num_sms, block_n, timeout_ns
        self.epoch = 0
        self.trace = None  # optional uint64 stamp buffer (see syn_gemm_args.trace): waits of the reduce waves
        if self.world == 1:
            return
        self.generator, self.info, lowered = plan_reduce_scatter(self.world, M, N, dtype, plan, chunk_split)
        self.src_schedule = lowered[self.rank]["src"]
        self.dst_schedule = lowered[self.rank]["dst"]
        self.remote_signals = rs_remote_signals(self.info, self.rank, self.src_schedule)
        self.stage = ctx.alloc((2, self.world, self.slab, N), dtype)
        self.flags = ctx.alloc((max(self.info.recv_signal_num, 1),), torch.int64)
        self.counters = torch.zeros(NUM_COUNTERS, dtype=torch.int32, device=ctx.device)
        if publish_pieces:
            self.out_flags = torch.zeros(self.pieces, dtype=torch.int64, device=ctx.device)
        self.send = self.send_flags = None
        if comm == "ce":
            self.send = torch.empty(self.world, self.slab, N, dtype=dtype, device=ctx.device)
            self.send_flags = torch.zeros(len(self.remote_signals), dtype=torch.int64, device=ctx.device)
            self._copy_streams = [torch.cuda.Stream(device=ctx.device) for _ in range(max(1, copy_streams))]
            self._flag_stream = torch.cuda.Stream(device=ctx.device) if flag_stream else None
            self._ev_start = torch.cuda.Event()
            self._ev_go = torch.cuda.Event()
            self._programs = []
            for parity in (0, 1):
                steps = [(lflag, dst, src, nbytes, rflag, i)
                         for i, (lflag, src, dst, nbytes, rflag) in enumerate(self.transport_program(parity))]
                self._programs.append((_L.make_ce_program(steps), len(steps)))

    def transport_program(self, epoch: int):
        """The side streams' work for the call with this epoch (see ``rs_transport_program``)."""
        return rs_transport_program(self.rank, self.world, self.slab, self.N * self.dtype.itemsize, epoch,
                                    self.src_schedule, self.remote_signals, self.send.data_ptr(),
                                    self.send_flags.data_ptr(), self.stage.symm.ptrs, self.flags.symm.ptrs)

    def __call__(self, a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, stream=None):
        if out is None:
            out = torch.empty(self.slab, self.N, dtype=self.dtype, device=self.ctx.device)
        self.epoch += 1
        if self.world == 1:
            return gemm(a, b, out, 1, self.num_sms, BLOCK_SIZE_N=self.block_n, status=self.ctx.status,
                        timeout_ns=self.timeout_ns, stream=stream)
        cur = stream or torch.cuda.current_stream()
        if self.comm == "ce":
            # Order of issue: the barrier kernel (side stream) BEFORE the kernels - it must be on the
            # GPU before a kernel that waits for the peers' partial sums, never launched past one - and
            # the flag-gated copies AFTER the kernel that raises their flags: a stream wait issued
            # ahead of its producer can block the producer where the two streams share a hardware
            # queue.  Per wave the transport is "wait for the wave's local flag, copy its rows, raise
            # the target's flag".
            side = self._copy_streams
            self._ev_start.record(cur)
            side[0].wait_event(self._ev_start)
            if self.lockstep:
                self.ctx.barrier(side[0])
            self._ev_go.record(side[0])
            gemm_rs(a, b, out, self.src_schedule, self.dst_schedule, self.remote_signals, self.stage.symm,
                    self.flags.symm, self.counters, epoch=self.epoch, num_sms=self.num_sms, block_n=self.block_n,
                    timeout_ns=self.timeout_ns, status=self.ctx.status, stream=cur, send_buf=self.send,
                    send_flags=self.send_flags, trace=self.trace, out_flags=self.out_flags,
                    reduce_pass=self.reduce_pass)
            for s in side[1:]:
                s.wait_event(self._ev_go)
            program, n = self._programs[self.epoch & 1]
            _L.ce_run(program, n, side, self.epoch, self._flag_stream)
            for s in side:
                cur.wait_stream(s)  # the next call's kernel may overwrite the send slabs
            if self._flag_stream is not None:
                cur.wait_stream(self._flag_stream)
            return out
        if self.lockstep:
            self.ctx.barrier(cur)
        return gemm_rs(a, b, out, self.src_schedule, self.dst_schedule, self.remote_signals, self.stage.symm,
                       self.flags.symm, self.counters, epoch=self.epoch, num_sms=self.num_sms,
                       block_n=self.block_n, timeout_ns=self.timeout_ns, status=self.ctx.status, stream=cur,
                       trace=self.trace, out_flags=self.out_flags, reduce_pass=self.reduce_pass)


class GemmAllReduce:
    """``out[M, N]`` (the same on every rank) ``= sum over ranks of A_r[M, K_r] @ B_r[N, K_r]^T``.

    The reference overlaps a library all-reduce per row slice with the producer GEMM
    (``build_all_reduce_plan(num_all_reduces=..., split_axis=0, compute_producer=True)``,
    tests/test_gemm_ar_collective.py:97-160).  Here every slice is a GEMM + reduce-scatter (partial
    sums pushed to the slab's owner, fp32 reduction by the owner: in the reduce pass behind the kernel,
    or in the own tiles' epilogue with ``reduce="epilogue"``) whose reduced rows are
    then all-gathered by copy engines: a local flag is raised per finished row piece, side
    streams wait for it and push the rows to every peer's copy of ``out``.  With ``num_splits`` > 1
    the slices are separate launches, and the all-gather of one slice runs under the GEMM of the
    next.  ``out`` is a symmetric buffer that the peers write: read it after the call has returned
    in stream order (the call ends with a wait for every peer's rows) and before the next call
    starts on any rank (``sync_after=True`` adds the barrier that guarantees the latter)."""

    def __init__(self, ctx: SymmetricContext, M: int, N: int, dtype=torch.bfloat16, num_splits: int = 1,
                 chunk_split: int = 1, comm: str = "sm", copy_streams: int = 2, timeout_ns: int = 0,
                 lockstep: bool = True, sync_after: bool = False, reduce: str = "auto"):
        if M % (num_splits * ctx.world):
            raise ValueError("M must be divisible by num_splits * world")
        self.ctx, self.world, self.rank = ctx, ctx.world, ctx.rank
        self.M, self.N, self.dtype = M, N, dtype
        self.num_splits, self.sync_after = num_splits, sync_after
        self.part_rows = M // num_splits
        self.out = ctx.alloc((M, N), dtype)
        self.rs = GemmReduceScatter(ctx, self.part_rows, N, dtype, plan="direct", timeout_ns=timeout_ns,
                                    lockstep=lockstep, comm=comm, copy_streams=copy_streams, chunk_split=chunk_split,
                                    publish_pieces=True, reduce=reduce)
        self.slab = self.part_rows // self.world
        if self.world == 1:
            return
        pieces = self.rs.pieces
        self.gather_flags = ctx.alloc((self.world * pieces,), torch.int64)  # [sender][piece], raised by the sender
        self._gather_streams = [torch.cuda.Stream(device=ctx.device) for _ in range(max(1, copy_streams))]
        self._gather_flag_stream = torch.cuda.Stream(device=ctx.device)
        self._ev = torch.cuda.Event()
        self._programs = []
        for part in range(num_splits):
            steps = self.gather_program(part)
            self._programs.append((_L.make_ce_program(steps), len(steps)))

    def piece_rows(self):
        """``[(first row inside the slab, rows)]`` of the row pieces the slab is reduced (and published) in."""
        rows = -(-self.slab // self.rs.pieces)
        return [(lo, min(rows, self.slab - lo)) for lo in range(0, self.slab, rows)]

    def gather_program(self, part: int):
        """Copy-engine steps that pass this rank's reduced rows of slice ``part`` on: per row piece,
        wait for the kernel's local flag, copy the rows into every peer's ``out`` (peers in swizzled
        order), raise ``gather_flags[rank][piece]`` there.  A piece always uses the same stream, so
        its flag on a peer never runs ahead of the rows of an earlier slice."""
        row_bytes = self.N * self.dtype.itemsize
        steps = []
        for g, (lo, rows) in enumerate(self.piece_rows()):
            first = part * self.part_rows + self.rank * self.slab + lo
            wait = self.rs.out_flags.data_ptr() + 8 * g
            for i in range(1, self.world):
                peer = (self.rank + i) % self.world
                steps.append((wait, self.out.symm.ptrs[peer] + first * row_bytes,
                              self.out.symm.ptrs[self.rank] + first * row_bytes, rows * row_bytes,
                              self.gather_flags.symm.ptrs[peer] + 8 * (self.rank * self.rs.pieces + g), g))
        return steps

    def __call__(self, a: torch.Tensor, b: torch.Tensor, stream=None) -> torch.Tensor:
        cur = stream or torch.cuda.current_stream()
        if self.world == 1:
            return self.rs(a, b, self.out.local, stream=cur)
        lib = _raw_lib()
        for part in range(self.num_splits):
            r0 = part * self.part_rows
            own = self.out.local[r0 + self.rank * self.slab : r0 + (self.rank + 1) * self.slab]
            self._ev.record(cur)
            for s in self._gather_streams:
                s.wait_event(self._ev)   # the previous call's readers of `out` are behind this point
            self.rs(a[r0 : r0 + self.part_rows], b, own, stream=cur)
            program, n = self._programs[part]
            _L.ce_run(program, n, self._gather_streams, self.rs.epoch, self._gather_flag_stream)
        # every peer's rows of the last slice (and, flag by flag in order, of the earlier ones)
        for src in range(self.world):
            if src == self.rank:
                continue
            for g in range(self.rs.pieces):
                _L.check(lib.syn_flag_wait_stream(self.gather_flags.local.data_ptr() + 8 * (src * self.rs.pieces + g),
                                                  self.rs.epoch, cur.cuda_stream or None), "syn_flag_wait_stream")
        for s in self._gather_streams + [self._gather_flag_stream]:
            cur.wait_stream(s)
        if self.sync_after:
            self.ctx.barrier(cur)
        return self.out.local


class AllToAllGemm:
    """``out[B * S / world, N] = all_to_all(x)[B, S / world, H, D].reshape(B * S / world, H * D) @ W[N, H * D]^T``:
    the head-sharded attention output ``x`` ``[B, S, H / world, D]`` of every rank is re-sharded along
    the sequence while the output projection already runs (the reference's
    tests/test_all2all_gemm.py:112-160).  The all-to-all is the rank's SM-copy program on a side
    stream (``CommContext.execute`` on ``num_copy_sms`` SMs: pushes, each followed by the receiver's
    flag); the GEMM runs on the other SMs, and every tile walks the K ranges (one per sending rank)
    in arrival order, waiting for a range's flag before its first load from it."""

    __doc__ += _HAZARD_NOTE + """
    The symmetric input is ``src``."""

    def __init__(self, ctx, B: int, S: int, H: int, D: int, N: int, dtype=torch.bfloat16, num_copy_sms: int = 16,
                 timeout_ns: int = 0, lockstep: bool = True, sync_after: bool = False):
        from .communication.comm_runtime.communication_context import CommContext

        self.ctx, self.world, self.rank = ctx, ctx.world, ctx.rank
        W = self.world
        self.B, self.S, self.H, self.D, self.N, self.dtype = B, S, H, D, N, dtype
        self.Hl, self.S_local = H // W, S // W
        self.lockstep, self.sync_after, self.timeout_ns = lockstep, sync_after, timeout_ns
        plans = {r: build_all_to_all_plan_dim((B, S, self.Hl, D), dtype=dtype, mesh_size=W, rank=r, src_buffer="src",
                                              dst_buffer="dst", src_split_axis=2, dst_split_axis=1, transfer_kind="push")
                 for r in range(W)}
        gen = CommGenerator(plans)
        gen.plan_signals()
        self.info = gen.generate_code_for_plan(CodeGenOptions(copy_engine=False))
        self.info.local_world_size = W
        self.info.num_copy_sms = num_copy_sms if W > 1 else 0
        self.comm = CommContext(self.rank, self.info, symmetric=ctx, timeout_ns=timeout_ns)
        dst = lower_comm_plan_to_raw_schedules(gen)[self.rank]["dst"]
        rows = B * self.S_local
        # one wave per arriving slab: all rows, all N, the K range of the sender's heads
        self.wave_offsets = [[0, 0, o[2] * D + o[3]] for o in dst.gen_block_offset_lists()]
        self.wave_sizes = [[s_[0] * s_[1], N, s_[2] * s_[3]] for s_ in dst.gen_block_shape_lists()]
        self.signals = dst.gen_signal_lists()
        assert all(sz[0] == rows for sz in self.wave_sizes)
        self.src = self.comm.comm_buffers["src"][self.rank]
        self.a = self.comm.comm_buffers["dst"][self.rank].view(rows, H * D)
        self.num_gemm_sms = 0
        if W > 1 and num_copy_sms > 0:
            sms = torch.cuda.get_device_properties(ctx.device).multi_processor_count
            self.num_gemm_sms = max(sms - num_copy_sms, 2) & ~1

    def send(self, stream=None):
        """The all-to-all: this rank's slabs to their ranks (side streams), each followed by its flag."""
        cur = stream or torch.cuda.current_stream()
        self.comm.next_epoch()
        if self.lockstep and self.world > 1:
            self.ctx.barrier(cur)
        self.comm.start_after(cur)
        self.comm.execute()

    def consume(self, w: torch.Tensor, out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        """The projection over the K ranges as they arrive."""
        cur = stream or torch.cuda.current_stream()
        if out is None:
            out = torch.empty(self.a.shape[0], self.N, dtype=self.dtype, device=self.ctx.device)
        gemm(self.a, w, out, self.world, self.num_gemm_sms, cur_wave_sizes=self.wave_sizes, wave_offsets=self.wave_offsets,
             signal_ptr=self.comm.recv_signal_bufs[self.rank], signal_offsets=self.signals,
             signal_value=self.comm.signal_value, timeout_ns=self.timeout_ns, status=self.ctx.status, stream=cur)
        self.comm.end_before(cur)
        if self.sync_after and self.world > 1:
            self.ctx.barrier(cur)
        return out

    def __call__(self, w: torch.Tensor, out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        self.send(stream)
        return self.consume(w, out, stream)


class GemmAllToAllGemm:
    """Tensor-parallel MLP without a reduction: ``out[M / world, hidden] = all_to_all(x @ W1_r^T) @ W2^T``
    (the reference's tests/test_gemm_all2all_gemm.py:126-207).  ``x`` ``[M, hidden]`` is replicated,
    ``W1_r`` ``[ffn / world, hidden]`` is this rank's shard, ``W2`` ``[hidden, ffn]`` is whole.  The
    first GEMM is a producer (one wave of rows per destination rank, raising a COMPUTE_DONE flag),
    the rank's SM-copy program pushes each finished row block to its rank and raises the receiver's
    flag, and the second GEMM consumes the arriving K ranges (one per sending rank)."""

    def __init__(self, ctx, M: int, hidden: int, ffn: int, dtype=torch.bfloat16, num_copy_sms: int = 16,
                 timeout_ns: int = 0, lockstep: bool = True):
        from .communication.comm_runtime.communication_context import CommContext

        self.ctx, self.world, self.rank = ctx, ctx.world, ctx.rank
        W = self.world
        self.M, self.hidden, self.ffn, self.dtype = M, hidden, ffn, dtype
        self.rows, self.ffn_local = M // W, ffn // W
        self.lockstep, self.timeout_ns = lockstep, timeout_ns
        plans = {r: build_all_to_all_plan_dim((M, self.ffn_local), dtype=dtype, mesh_size=W, rank=r, src_buffer="src",
                                              dst_buffer="dst", src_split_axis=1, dst_split_axis=0, transfer_kind="push",
                                              compute_producer=True)
                 for r in range(W)}
        gen = CommGenerator(plans)
        gen.plan_signals()
        self.info = gen.generate_code_for_plan(CodeGenOptions(copy_engine=False))
        self.info.local_world_size = W
        self.info.num_copy_sms = num_copy_sms if W > 1 else 0
        self.comm = CommContext(self.rank, self.info, symmetric=ctx, timeout_ns=timeout_ns)
        low = lower_comm_plan_to_raw_schedules(gen)[self.rank]
        src, dst = low["src"], low["dst"]
        self.prod_offsets, self.prod_sizes = src.gen_block_offset_lists(), src.gen_block_shape_lists()
        self.prod_signals = src.gen_signal_lists()
        self.wave_offsets = [[o[0], 0, o[1]] for o in dst.gen_block_offset_lists()]
        self.wave_sizes = [[s_[0], hidden, s_[1]] for s_ in dst.gen_block_shape_lists()]
        self.signals = dst.gen_signal_lists()
        self.counters = torch.zeros(NUM_COUNTERS, dtype=torch.int32, device=ctx.device)
        self.mid = self.comm.comm_buffers["src"][self.rank]   # [M, ffn / world]: the first GEMM's output
        self.a2 = self.comm.comm_buffers["dst"][self.rank]    # [M / world, ffn]: the second GEMM's input
        self.num_gemm_sms = 0
        if W > 1 and num_copy_sms > 0:
            sms = torch.cuda.get_device_properties(ctx.device).multi_processor_count
            self.num_gemm_sms = max(sms - num_copy_sms, 2) & ~1

    def produce_and_send(self, x: torch.Tensor, w1: torch.Tensor, stream=None):
        cur = stream or torch.cuda.current_stream()
        self.comm.next_epoch()
        if self.lockstep and self.world > 1:
            self.ctx.barrier(cur)
        self.comm.start_after(cur)
        gemm(x, w1, self.mid, self.world, self.num_gemm_sms, cur_wave_sizes=self.prod_sizes, wave_offsets=self.prod_offsets,
             signal_offsets=[-1] * len(self.prod_signals), producer_signal_ptr=self.comm.compute_signal_bufs[self.rank],
             producer_signal_offsets=self.prod_signals, counter_ptr=self.counters, signal_value=self.comm.signal_value,
             timeout_ns=self.timeout_ns, status=self.ctx.status, stream=cur)
        self.comm.execute()

    def consume(self, w2: torch.Tensor, out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        cur = stream or torch.cuda.current_stream()
        if out is None:
            out = torch.empty(self.rows, self.hidden, dtype=self.dtype, device=self.ctx.device)
        gemm(self.a2, w2, out, self.world, self.num_gemm_sms, cur_wave_sizes=self.wave_sizes, wave_offsets=self.wave_offsets,
             signal_ptr=self.comm.recv_signal_bufs[self.rank], signal_offsets=self.signals,
             signal_value=self.comm.signal_value, timeout_ns=self.timeout_ns, status=self.ctx.status, stream=cur)
        self.comm.end_before(cur)
        return out

    def __call__(self, x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, out: Optional[torch.Tensor] = None, stream=None):
        self.produce_and_send(x, w1, stream)
        return self.consume(w2, out, stream)


# ----------------------------------------------------------------------------------------------
# attention operators
# ----------------------------------------------------------------------------------------------
import ctypes as _C

from .communication.common_descriptors import (
    build_all_to_all_plan_dim,
    build_double_ring_all_gather_plan,
)
from .computation.attn import AttentionState, attention_forward
from .computation.attn.plan import (
    all_gather_wave_metadata,
    all_to_all_wave_metadata,
    completion_signals,
    merge_wave_tail,
    pull_ops_from_schedule,
    push_ops_from_schedule,
    zigzag_tables,
)


def _plan(plans):
    gen = CommGenerator(plans)
    gen.plan_signals(plan_compute_signals=True)
    info = gen.generate_code_for_plan(CodeGenOptions(copy_engine=False))
    return gen, info, lower_comm_plan_to_raw_schedules(gen)


def _local_table(ctx, t: torch.Tensor) -> "_L.Symm":
    """Buffer table for a buffer only this rank touches (every slot holds the local address)."""
    return _L.Symm.of(ctx.rank, [t.data_ptr()] * ctx.world)


class UlyssesAttention:
    """Sequence-parallel attention, Ulysses style: all-to-all (sequence-sharded -> head-sharded),
    causal flash attention over the full sequence for this rank's heads, all-to-all back.

    Per rank: ``qkv`` ``[3, B, H, S / world, D]`` in, ``[B, S / world, H, D]`` out.  The inbound
    all-to-all runs inside the attention kernel (comm warps pull the slabs in the plan's order, the
    tiles follow the triangular (Q slab, KV slab) order of the reference driver,
    tests/test_all2all_attn_transform.py:58-117, with the pairs a causal mask leaves joined into
    contiguous ranges); the outbound one is an SM copy kernel launched
    behind it (tests/test_attn_all2all_transform.py is the reference's overlapped form)."""

    __doc__ += _HAZARD_NOTE + """
    The symmetric input is ``qkv_src``; the symmetric output ``out`` is written by the peers: read it
    after ``wait_output`` and before the next call starts."""

    def __init__(self, ctx, B: int, H: int, S_local: int, D: int = 128, dtype=torch.bfloat16, causal: bool = True,
                 sm_scale: Optional[float] = None, timeout_ns: int = 0, lockstep: bool = True, sync_after: bool = False,
                 overlap_out: bool = True, join_waves: bool = True):
        """``join_waves``: a slab's arrival opens one wave per contiguous range of keys (its queries
        against every arrived slab - with a causal mask: at or below it) and of queries (the arrived
        slabs - causal: above it - against its keys) instead of one wave per pair of slabs, so that a query tile is
        visited a few times instead of once per slab (``all_to_all_wave_metadata(causal=True)``).
        ``overlap_out``: the attention kernel sends every query tile's final rows to their rank
        itself, at the tile's last visit, while the other tiles are still being computed (the
        reference's overlapped form, tests/test_attn_all2all_transform.py:182-215); otherwise, or
        when the problem has more tile pairs than an ownership plan holds, the outbound all-to-all
        is an SM copy kernel behind the attention kernel."""
        self.ctx, self.world, self.rank = ctx, ctx.world, ctx.rank
        self.lockstep, self.sync_after = lockstep, sync_after
        W = self.world
        self.B, self.H, self.S_local, self.D, self.dtype, self.causal = B, H, S_local, D, dtype, causal
        self.sm_scale = sm_scale if sm_scale is not None else D ** -0.5
        self.timeout_ns = timeout_ns
        self.S, self.Hl = S_local * W, H // W
        es = dtype.itemsize
        # ---- inbound plan: [3, B, H, S/W, D] -> [3, B, H/W, S, D]
        self.in_src_shape = (3, B, H, S_local, D)
        self.in_dst_shape = (3, B, self.Hl, self.S, D)
        _g, self.in_info, low = _plan({
            r: build_all_to_all_plan_dim(self.in_src_shape, dtype=dtype, mesh_size=W, rank=r, src_buffer="src",
                                         dst_buffer="dst", src_split_axis=3, dst_split_axis=2, transfer_kind="pull")
            for r in range(W)})
        self.in_schedule = low[self.rank]["dst"]
        self.qkv_src = ctx.alloc(self.in_src_shape, dtype)       # peers read it
        self.in_flags = ctx.alloc((max(self.in_info.recv_signal_num, 1),), torch.int64)
        self.qkv_dst = torch.zeros(self.in_dst_shape, dtype=dtype, device=ctx.device)
        self.waves = all_to_all_wave_metadata(self.in_schedule, {"batch": 1, "head": 2, "seq": 3},
                                              causal=causal and join_waves, join=join_waves)
        self.in_ops = pull_ops_from_schedule(self.in_schedule, self.rank, W, self.in_src_shape, self.in_dst_shape, es,
                                             src_buf=0, dst_buf=1)
        self.counters = torch.zeros(NUM_COUNTERS, dtype=torch.int32, device=ctx.device)
        self.in_comm, self._keep_in = _L.make_attn_comm(
            self.in_ops, [self.qkv_src.symm, _local_table(ctx, self.qkv_dst)], self.in_flags.symm,
            self.counters.data_ptr())
        # ---- attention output in [B, S, H/W, D], read by the kernel as [B, H/W, S, D]
        self.attn_out = torch.zeros(B, self.S, self.Hl, D, dtype=dtype, device=ctx.device)
        self.state = AttentionState(B, self.Hl, self.S, ctx.device)
        # ---- outbound plan: [B, S, H/W, D] -> [B, S/W, H, D]
        self.out_src_shape = (B, self.S, self.Hl, D)
        self.out_dst_shape = (B, S_local, H, D)
        _g2, self.out_info, low2 = _plan({
            r: build_all_to_all_plan_dim(self.out_src_shape, dtype=dtype, mesh_size=W, rank=r, src_buffer="src",
                                         dst_buffer="dst", src_split_axis=2, dst_split_axis=1, transfer_kind="push",
                                         compute_producer=True)
            for r in range(W)})
        self.out_schedule = low2[self.rank]["src"]
        self.out = ctx.alloc(self.out_dst_shape, dtype)           # peers write it
        self.out_flags = ctx.alloc((max(self.out_info.recv_signal_num, 1),), torch.int64)
        self.out_counters = torch.zeros(NUM_COUNTERS, dtype=torch.int32, device=ctx.device)
        sig = completion_signals(self.out_info, self.rank, self.out_schedule)
        self.out_ops = push_ops_from_schedule(self.out_schedule, self.rank, self.out_src_shape, self.out_dst_shape, es,
                                              src_buf=0, dst_buf=1, remote_signals=sig)
        self.out_comm, self._keep_out = _L.make_attn_comm(
            self.out_ops, [_local_table(ctx, self.attn_out), self.out.symm], self.out_flags.symm,
            self.out_counters.data_ptr())
        # ---- the same outbound plan as the kernel's producer role: one slab of query rows per target
        units = B * self.Hl * ((self.S + 255) // 256)
        self.push = None
        if overlap_out and W > 1 and units <= _L.ATTN_PLAN_MAX_UNITS and S_local % 128 == 0 and D == 128:
            slabs = []
            rows = zip(self.out_schedule.gen_block_offset_lists(), self.out_schedule.gen_block_shape_lists(),
                       self.out_schedule.gen_target_rank_list(), self.out_schedule.gen_dst_offset_lists(), sig)
            head_offset = None
            for off, shp, tgt, poff, rsig in rows:
                head_offset = poff[2] if head_offset is None else head_offset
                if (off[0], off[2], off[3]) != (0, 0, 0) or (shp[0], shp[2], shp[3]) != (B, self.Hl, D) or poff[2] != head_offset:
                    slabs = None
                    break
                slabs.append((off[1], shp[1], self.rank if tgt < 0 else tgt, poff[1], rsig))
            if slabs:
                slabs.sort()
                arr = (_L.AttnPushSlab * len(slabs))()
                for i, (q0, qn, dst, row0, flag) in enumerate(slabs):
                    arr[i].q_begin, arr[i].q_rows, arr[i].dst_rank, arr[i].dst_row0, arr[i].flag = q0, qn, dst, row0, flag
                self.push_counters = torch.zeros(8, dtype=torch.int32, device=ctx.device)
                push = _L.AttnPush()
                push.num_slabs = len(slabs)
                push.slabs = _C.cast(arr, _C.POINTER(_L.AttnPushSlab))
                push.dst = self.out.symm
                push.dst_strides = (_C.c_int64 * 3)(S_local * H * D, H * D, D)
                push.dst_rows, push.dst_heads, push.head_offset = S_local, H, head_offset
                push.flags = self.out_flags.symm
                push.counters = self.push_counters.data_ptr()
                self.push, self._keep_push = push, arr
        self.epoch = 0

    def launch_attention(self, stream=None, push: bool = False):
        """Inbound all-to-all fused with attention; fills ``attn_out`` - or, with ``push``, sends every
        tile's final rows to ``out`` on their rank and raises the slabs' flags there."""
        self.epoch += 1
        if self.lockstep and self.world > 1:
            self.ctx.barrier(stream)  # every peer's qkv_src is written before anybody pulls from it
        offs, sizes, sigs, _cum = self.waves
        q, k, v = self.qkv_dst[0], self.qkv_dst[1], self.qkv_dst[2]
        attention_forward(q, k, v, self.sm_scale, self.attn_out.permute(0, 2, 1, 3), wave_offsets=offs,
                          wave_sizes=sizes, signal_ptr=self.in_flags.local, signal_offsets=sigs, causal=self.causal,
                          state=self.state, signal_value=self.epoch, comm=self.in_comm, timeout_ns=self.timeout_ns,
                          status=self.ctx.status, stream=stream, push=self.push if push else None)

    def launch_scatter(self, stream=None):
        """Outbound all-to-all: pushes ``attn_out`` slabs to their ranks and raises their flags."""
        s = (stream or torch.cuda.current_stream()).cuda_stream or None
        _L.check(_L.lib().syn_copy(_C.byref(self.out_comm), 0, self.epoch, self.timeout_ns,
                                   self.ctx.status.data_ptr(), s), "syn_copy")

    def wait_output(self, stream=None):
        """Stream-ordered wait until every rank's slab has landed in ``out``."""
        s = (stream or torch.cuda.current_stream()).cuda_stream or None
        for i in range(self.out_info.recv_signal_num):
            _L.check(_L.lib().syn_flag_wait(self.out_flags.local.data_ptr() + 8 * i, self.epoch, self.timeout_ns,
                                            self.ctx.status.data_ptr(), i, s), "syn_flag_wait")

    def __call__(self, stream=None) -> torch.Tensor:
        if self.push is not None:
            self.launch_attention(stream, push=True)
        else:
            self.launch_attention(stream)
            self.launch_scatter(stream)
        self.wait_output(stream)
        if self.sync_after and self.world > 1:
            self.ctx.barrier(stream)
        return self.out.local


class ContextParallelAttention:
    """Context-parallel attention: queries stay local, K/V chunks are all-gathered by the kernel's
    comm warps in the order of the plan (swizzled direct, ring or double ring; on an all-to-all
    fabric every chunk is fetched from its owner), and the flash-attention tiles consume chunk
    after chunk (tests/test_allgather_attn_transform.py, test_ring_allgather_attn_transform.py,
    test_double_ring_ag_attn.py in the reference).  Causal masking uses true token positions, so the
    zigzag placement (rank r holds chunks r and 2 * world - 1 - r) balances the work."""

    __doc__ += _HAZARD_NOTE + """
    The symmetric input is ``kv_shard``."""

    def __init__(self, ctx, B: int, Hq: int, Hkv: int, S_local: int, D: int = 128, dtype=torch.bfloat16,
                 causal: bool = True, zigzag: bool = True, plan: str = "swizzle", inner_mesh_size: int = 2,
                 sm_scale: Optional[float] = None, timeout_ns: int = 0, lockstep: bool = True, sync_after: bool = False,
                 merge_waves_after: int = -1):
        """``merge_waves_after`` = k >= 1: the waves behind the first k are joined where their key ranges
        are adjacent in the gathered buffer (``merge_wave_tail``): fewer visits per query tile once the
        transfers run ahead of the attention.  -1 = one wave per chunk."""
        self.ctx, self.world, self.rank = ctx, ctx.world, ctx.rank
        self.lockstep, self.sync_after = lockstep, sync_after
        W = self.world
        self.B, self.Hq, self.Hkv, self.S_local, self.D = B, Hq, Hkv, S_local, D
        self.dtype, self.causal, self.timeout_ns = dtype, causal, timeout_ns
        self.sm_scale = sm_scale if sm_scale is not None else D ** -0.5
        self.S = S_local * W
        self.kv_shape = (2, B, Hkv, self.S, D)
        if plan == "swizzle":
            plans = {r: build_all_gather_plan_1d_swizzle(self.kv_shape, dtype, 3, W, r, "kv", "pull") for r in range(W)}
        elif plan == "ring":
            plans = {r: build_ring_all_gather_plan(self.kv_shape, dtype, 3, W, r, "kv") for r in range(W)}
        elif plan == "double_ring":
            plans = {r: build_double_ring_all_gather_plan(self.kv_shape, dtype, 3, W, inner_mesh_size, r, "kv")
                     for r in range(W)}
        else:
            raise ValueError("plan must be 'swizzle', 'ring' or 'double_ring'")
        _g, self.info, low = _plan(plans)
        self.schedule = low[self.rank]["kv"]
        self.kv = ctx.alloc(self.kv_shape, dtype)
        self.flags = ctx.alloc((max(self.info.recv_signal_num, 1),), torch.int64)
        self.counters = torch.zeros(NUM_COUNTERS, dtype=torch.int32, device=ctx.device)
        self.waves = all_gather_wave_metadata(self.schedule, S_local, {"batch": 1, "head": 2, "seq": 3}, q_heads=Hq)
        if merge_waves_after >= 1:
            self.waves = merge_wave_tail(self.waves, merge_waves_after)
        self.ops = pull_ops_from_schedule(self.schedule, self.rank, W, self.kv_shape, self.kv_shape, dtype.itemsize,
                                          src_buf=0, dst_buf=0, gather_axis=3)
        self.comm, self._keep = _L.make_attn_comm(self.ops, [self.kv.symm], self.flags.symm, self.counters.data_ptr())
        self.q_pos = self.kv_pos = None
        if causal and zigzag:
            qp, kp = zigzag_tables(W, self.rank, self.S)
            self.q_pos = torch.tensor(qp, dtype=torch.int32, device=ctx.device)
            self.kv_pos = torch.tensor(kp, dtype=torch.int32, device=ctx.device)
        elif causal:
            self.q_pos = torch.arange(self.rank * S_local, (self.rank + 1) * S_local, 128, dtype=torch.int32,
                                      device=ctx.device)
        self.state = AttentionState(B, Hq, S_local, ctx.device)
        self.epoch = 0

    @property
    def kv_shard(self) -> torch.Tensor:
        """This rank's slab ``[2, B, Hkv, S / world, D]`` of the gathered K/V buffer."""
        return self.kv.local[:, :, :, self.rank * self.S_local : (self.rank + 1) * self.S_local]

    def __call__(self, q: torch.Tensor, out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        if out is None:
            out = torch.empty_like(q)
        self.epoch += 1
        offs, sizes, sigs, _cum = self.waves
        comm = self.comm if self.ops else None
        if self.lockstep and self.world > 1 and comm is not None:
            self.ctx.barrier(stream)  # every peer's K/V shard is written before anybody pulls from it
        attention_forward(q, self.kv.local[0], self.kv.local[1], self.sm_scale, out, wave_offsets=offs,
                          wave_sizes=sizes, signal_ptr=self.flags.local, signal_offsets=sigs, causal=self.causal,
                          q_pos=self.q_pos, kv_pos=self.kv_pos, state=self.state, signal_value=self.epoch,
                          comm=comm, timeout_ns=self.timeout_ns, status=self.ctx.status, stream=stream)
        if self.sync_after and self.world > 1 and comm is not None:
            self.ctx.barrier(stream)
        return out
