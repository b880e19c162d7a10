"""The fused operators as objects: plan once (front end), allocate symmetric state once, call many
times.  Each object does, for one rank, what the reference's test drivers do by hand
(tests/test_ag_gemm_gen.py:120-176, tests/test_gemm_rs_direct_reduce.py:120-189): build every
rank's plan, plan signals, generate the op program, lower to schedules, allocate the symmetric
buffers and flags, then launch the fused kernel with this rank's schedule.

Flags carry an epoch that grows by one per call, so nothing is reset between calls and no barrier
is needed inside the timed path.
"""
from __future__ import annotations

from typing import Optional

import torch

from .communication.code_gen import CodeGenOptions, CommGenerator
from .communication.common_descriptors import (
    build_all_gather_plan_1d_swizzle,
    build_all_to_all_plan,
    build_reduce_scatter_direct_reduce_plan,
    build_ring_all_gather_plan,
)
from .computation.gemm import ag_gemm, gemm, gemm_rs
from .computation.gemm.plan import rs_remote_signals
from .interface import lower_comm_plan_to_raw_schedules
from .runtime import SymmetricContext

NUM_COUNTERS = 128  # SYN_MAX_WAVES + SYN_MAX_COMM_OPS


def plan_all_gather(world: int, rows_per_rank: int, K: int, dtype: torch.dtype, kind: str = "swizzle",
                    copy_engine: bool = False):
    """(generator, comm_info, lowered) for gathering ``[rows_per_rank, K]`` shards along dim 0."""
    shape = (rows_per_rank * world, K)
    if kind == "swizzle":
        plans = {r: build_all_gather_plan_1d_swizzle(shape, dtype, 0, world, r, "a", "pull") for r in range(world)}
    elif kind == "ring":
        plans = {r: build_ring_all_gather_plan(shape, dtype, 0, world, r, "a") for r in range(world)}
    else:
        raise ValueError("kind must be 'swizzle' or 'ring'")
    gen = CommGenerator(plans)
    gen.plan_signals(plan_compute_signals=True)
    info = gen.generate_code_for_plan(CodeGenOptions(copy_engine=copy_engine))
    return gen, info, lower_comm_plan_to_raw_schedules(gen)


def plan_reduce_scatter(world: int, M: int, N: int, dtype: torch.dtype, kind: str = "direct"):
    """(generator, comm_info, lowered) for reduce-scattering a partial ``[M, N]`` along dim 0."""
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
    gen = CommGenerator(plans)
    gen.plan_signals(plan_compute_signals=True)
    info = gen.generate_code_for_plan(CodeGenOptions(copy_engine=False))
    return gen, info, lower_comm_plan_to_raw_schedules(gen)


class AllGatherGemm:
    """``C[rows * world, N] = all_gather(A_shard)[rows * world, K] @ B[N, K]^T`` per rank.

    ``comm="sm"``: the kernel's comm warps pull the chunks (``CodeGenOptions(copy_engine=False)``
    program); ``comm="ce"``: the rank's copy-engine program (``copy_engine=True``) runs on a side
    stream through ``CommContext.execute`` while the flag-gated GEMM runs on the caller's stream,
    as in the reference's tests/test_ag_gemm_gen.py:44-77."""

    def __init__(self, ctx: SymmetricContext, rows_per_rank: int, K: int, N: int, dtype=torch.bfloat16,
                 plan: str = "swizzle", num_sms: int = 0, block_n: int = 0, timeout_ns: int = 0, comm: str = "sm"):
        self.ctx = ctx
        self.world, self.rank = ctx.world, ctx.rank
        self.rows, self.K, self.N, self.dtype = rows_per_rank, K, N, dtype
        self.M = rows_per_rank * self.world
        self.num_sms, self.block_n, self.timeout_ns = num_sms, block_n, timeout_ns
        self.comm = comm
        self.generator, self.info, lowered = plan_all_gather(self.world, rows_per_rank, K, dtype, plan,
                                                             copy_engine=(comm == "ce"))
        self.schedule = lowered[self.rank]["a"]
        self.epoch = 0
        if comm == "ce":
            from .communication.comm_runtime.communication_context import CommContext

            self.info.local_world_size = self.world
            self.comm_ctx = CommContext(self.rank, self.info, symmetric=ctx, timeout_ns=timeout_ns)
            self.a = self.comm_ctx._buffers["a"]
            self.flags = self.comm_ctx._recv
            self._wave_offsets = [[o[0], 0] for o in self.schedule.gen_block_offset_lists()]
            self._wave_sizes = [[s[0], N] for s in self.schedule.gen_block_shape_lists()]
            self._signals = self.schedule.gen_signal_lists()
            return
        self.a = ctx.alloc((self.M, K), dtype)
        self.flags = ctx.alloc((max(self.info.recv_signal_num, 1),), torch.int64)
        self.counters = torch.zeros(NUM_COUNTERS, dtype=torch.int32, device=ctx.device)

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
        if self.comm == "ce":
            cur = stream or torch.cuda.current_stream()
            self.comm_ctx.signal_value = self.epoch
            self.comm_ctx.start_after(cur)
            self.comm_ctx.execute(neglect_local=True)
            gemm(self.a.local, b, c, self.world, self.num_sms, BLOCK_SIZE_N=self.block_n,
                 cur_wave_sizes=self._wave_sizes, wave_offsets=self._wave_offsets, signal_ptr=self.flags.local,
                 signal_offsets=self._signals, signal_value=self.epoch, status=self.ctx.status,
                 timeout_ns=self.timeout_ns, stream=cur)
            self.comm_ctx.end_before(cur)
            return c
        return ag_gemm(self.a.symm, self.a.local, b, c, self.schedule, self.flags.local, self.counters,
                       epoch=self.epoch, num_sms=self.num_sms, block_n=self.block_n, timeout_ns=self.timeout_ns,
                       status=self.ctx.status, stream=stream)


class GemmReduceScatter:
    """``out[M / world, N] = sum over ranks of (A_r[M, K_r] @ B_r[N, K_r]^T)[own rows]``."""

    def __init__(self, ctx: SymmetricContext, M: int, N: int, dtype=torch.bfloat16, plan: str = "direct",
                 num_sms: int = 0, block_n: int = 0, timeout_ns: int = 0):
        self.ctx = ctx
        self.world, self.rank = ctx.world, ctx.rank
        self.M, self.N, self.dtype = M, N, dtype
        self.slab = M // self.world
        self.num_sms, self.block_n, self.timeout_ns = num_sms, block_n, timeout_ns
        self.epoch = 0
        if self.world == 1:
            return
        self.generator, self.info, lowered = plan_reduce_scatter(self.world, M, N, dtype, plan)
        self.src_schedule = lowered[self.rank]["src"]
        self.dst_schedule = lowered[self.rank]["dst"]
        self.remote_signals = rs_remote_signals(self.info, self.rank, self.src_schedule)
        self.stage = ctx.alloc((2, self.world, self.slab, N), dtype)
        self.flags = ctx.alloc((max(self.info.recv_signal_num, 1),), torch.int64)
        self.counters = torch.zeros(NUM_COUNTERS, dtype=torch.int32, device=ctx.device)

    def __call__(self, a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, stream=None):
        if out is None:
            out = torch.empty(self.slab, self.N, dtype=self.dtype, device=self.ctx.device)
        self.epoch += 1
        if self.world == 1:
            return gemm(a, b, out, 1, self.num_sms, BLOCK_SIZE_N=self.block_n, status=self.ctx.status,
                        timeout_ns=self.timeout_ns, stream=stream)
        return gemm_rs(a, b, out, self.src_schedule, self.dst_schedule, self.remote_signals, self.stage.symm,
                       self.flags.symm, self.counters, epoch=self.epoch, num_sms=self.num_sms,
                       block_n=self.block_n, timeout_ns=self.timeout_ns, status=self.ctx.status, stream=stream)
