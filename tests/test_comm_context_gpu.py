"""``CommContext`` on a GPU: the op-program interpreter (copy-engine copies, SM box copies incl. the
reducing form, flag sets and waits), the sequence the reference's drivers run around a flag-gated
GEMM (tests/test_ag_gemm_gen.py:44-77 in the reference: reset_signals -> barrier -> start_after ->
execute -> gemm(signal_ptr=...) -> end_before) and one graph replay of it.  All ranks of the plan
live on one GPU (``EmulatedWorld``) and run one after the other."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from parity import assert_gemm_close  # noqa: E402

pytestmark = pytest.mark.gpu
DT = torch.bfloat16


def _seeded(seed, shape, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g, dtype=torch.float32) * scale).to(DT)


def test_copy_engine_program_feeds_a_flag_gated_gemm_and_replays_as_a_graph():
    from syncopate_b200.communication.comm_runtime.communication_context import CommContext
    from syncopate_b200.computation.gemm import gemm
    from syncopate_b200.operators import plan_all_gather
    from syncopate_b200.runtime import EmulatedWorld

    W, rows, K, N = 4, 256, 512, 512
    _gen, info, low = plan_all_gather(W, rows, K, DT, "swizzle", copy_engine=True)
    ew = EmulatedWorld(W)
    ctxs = [CommContext(r, info, symmetric=ew.contexts[r], timeout_ns=500_000_000) for r in range(W)]
    shards = [_seeded(100 + r, (rows, K)).cuda() for r in range(W)]
    full = torch.cat(shards, 0)
    b = _seeded(7, (N, K), 0.02).cuda()
    ref = full.float() @ b.float().t()

    def reset(r):
        buf = ctxs[r].comm_buffers["a"][r]
        buf.fill_(float("nan"))
        buf[r * rows:(r + 1) * rows] = shards[r]

    for r in range(W):
        reset(r)
    cur = torch.cuda.current_stream()
    for r, ctx in enumerate(ctxs):
        sched = low[r]["a"]
        offs = [[o[0], 0] for o in sched.gen_block_offset_lists()]
        sizes = [[s[0], N] for s in sched.gen_block_shape_lists()]
        a_local = ctx.comm_buffers["a"][r]
        c = torch.zeros(W * rows, N, dtype=DT, device="cuda")
        assert len(ctx.streams) == len(info.operations[r]) and ctx.get_comm_sms() == info.num_copy_sms

        def run_gemm():
            gemm(a_local, b, c, W, cur_wave_sizes=sizes, wave_offsets=offs, signal_ptr=ctx.recv_signal_bufs[r],
                 signal_offsets=sched.gen_signal_lists(), signal_value=ctx.signal_value, timeout_ns=500_000_000,
                 status=ew.contexts[r].status)

        # the reference driver's sequence
        ctx.reset_signals()
        ew.contexts[r].barrier()
        ctx.start_after(cur)
        ctx.execute()
        run_gemm()
        ctx.end_before(cur)
        ew.contexts[r].check()
        assert torch.equal(a_local, full)
        assert ctx.recv_signal_bufs[r][:info.recv_signal_num].tolist() == [1] * info.recv_signal_num
        assert_gemm_close(c, ref, f"rank {r}")

        # the same program captured once and replayed
        graph = ctx.get_graph()
        torch.cuda.synchronize()
        reset(r)
        c.zero_()
        ctx.reset_signals()
        ew.contexts[r].barrier()
        graph.replay()
        run_gemm()
        ew.contexts[r].check()
        assert torch.equal(a_local, full)
        assert_gemm_close(c, ref, f"rank {r} (graph replay)")

        # a later epoch needs neither a reset nor a barrier
        reset(r)
        ctx.next_epoch()
        ctx.update_comm_info(info)   # same program again: streams are rebuilt
        ctx.start_after(cur)
        ctx.execute(neglect_local=True)
        run_gemm()
        ctx.end_before(cur)
        ew.contexts[r].check()
        assert torch.equal(a_local, full)
        assert ctx.recv_signal_bufs[r][:info.recv_signal_num].tolist() == [2] * info.recv_signal_num
        reset(r)


@pytest.mark.parametrize("stream_waits", [False, True])
def test_sm_copy_program_with_reducing_copies(stream_waits):
    """The reduce-scatter program of the direct-reduce plan: wait for the producer's flag, add the
    slab into the owner's buffer (a reducing SM copy, local or to a peer), raise the owner's flag."""
    from syncopate_b200.communication.comm_runtime.communication_context import CommContext
    from syncopate_b200.operators import plan_reduce_scatter
    from syncopate_b200.runtime import EmulatedWorld

    W, M, N = 4, 512, 384
    slab = M // W
    _gen, info, _low = plan_reduce_scatter(W, M, N, DT, "direct")
    kinds = {type(op).__name__ for ops in info.operations[0] for op in ops}
    assert {"WaitIntraNodeSignal", "SMCopyOp", "IntraNodeSignal"} <= kinds
    ew = EmulatedWorld(W)
    ctxs = [CommContext(r, info, symmetric=ew.contexts[r], timeout_ns=500_000_000, stream_waits=stream_waits)
            for r in range(W)]
    parts = [_seeded(300 + r, (M, N)).cuda() for r in range(W)]
    for r, ctx in enumerate(ctxs):
        ctx.comm_buffers["src"][r].copy_(parts[r])
        ctx.comm_buffers["dst"][r].zero_()
        ctx.compute_signal_bufs[r].fill_(1)   # the producer GEMM of this test has already finished
    cur = torch.cuda.current_stream()
    for r, ctx in enumerate(ctxs):
        ctx.start_after(cur)
        ctx.execute()
        ctx.end_before(cur)
        ew.contexts[r].check()
    for r, ctx in enumerate(ctxs):
        want = sum(p[r * slab:(r + 1) * slab].float() for p in parts)
        got = ctx.comm_buffers["dst"][r].float()
        # W additions, each rounded to bf16: a few output rounding steps
        assert (got - want).abs().max().item() <= 4 * 2.0 ** -8 * want.abs().max().item()
        assert ((got - want).norm() / want.norm()).item() < 1e-2
        assert ctx.recv_signal_bufs[r][:info.recv_signal_num].tolist() == [1] * info.recv_signal_num


def test_comm_context_takes_the_process_context_by_default():
    from syncopate_b200.communication.comm_runtime.communication_context import CommContext
    from syncopate_b200.operators import plan_all_gather
    from syncopate_b200.runtime import SymmetricContext

    _gen, info, _low = plan_all_gather(1, 128, 64, DT, "swizzle", copy_engine=True)
    sym = SymmetricContext(0, 1)
    try:
        ctx = CommContext(0, info)          # the reference's signature: nothing but rank and info
        assert ctx.symmetric is sym and ctx.comm_buffers["a"][0].shape == (128, 64)
    finally:
        sym.close()
