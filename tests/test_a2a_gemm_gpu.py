"""All-to-all + GEMM and GEMM + all-to-all + GEMM on a GPU: the K-gated consumer GEMM (waves over
(M, N, K)), the closed-form (Mod1D) schedule entry point, and the two operators on emulated ranks
(all ranks of the plan on one GPU: first every rank sends, then every rank consumes), against
torch on the gathered inputs - the reference's own checks (tests/test_all2all_gemm.py:273-286,
tests/test_gemm_all2all_gemm.py:311-327)."""
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


@pytest.mark.parametrize("M,N,K,ranges", [(512, 512, 1024, [(512, 256), (0, 512), (768, 256)]),
                                          (256, 384, 320, [(128, 192), (0, 128)]),
                                          (384, 256, 512, [(0, 512)])])
def test_k_gated_consumer_gemm(M, N, K, ranges):
    """Waves over (M, N, K) in a scrambled arrival order, all flags already up: every tile walks the K
    ranges in wave order and the result is the whole product."""
    from syncopate_b200.computation.gemm import gemm

    a, b = _seeded(1, (M, K)).cuda(), _seeded(2, (N, K), 0.02).cuda()
    c = torch.zeros(M, N, dtype=DT, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    flags = torch.full((len(ranges),), 3, dtype=torch.int64, device="cuda")
    gemm(a, b, c, cur_wave_sizes=[[M, N, n] for _o, n in ranges], wave_offsets=[[0, 0, o] for o, _n in ranges],
         signal_ptr=flags, signal_offsets=list(range(len(ranges))), signal_value=3, status=status, timeout_ns=300_000_000)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    assert_gemm_close(c, a.float() @ b.float().t())


def test_k_gate_whose_flag_never_comes_times_out_cleanly():
    from syncopate_b200.computation.gemm import gemm

    M, N, K = 256, 256, 256
    a, b = _seeded(1, (M, K)).cuda(), _seeded(2, (N, K), 0.02).cuda()
    c = torch.zeros(M, N, dtype=DT, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    flags = torch.tensor([1, 0], dtype=torch.int64, device="cuda")
    gemm(a, b, c, cur_wave_sizes=[[M, N, 128], [M, N, 128]], wave_offsets=[[0, 0, 0], [0, 0, 128]], signal_ptr=flags,
         signal_offsets=[0, 1], status=status, timeout_ns=1_000_000)
    torch.cuda.synchronize()
    assert status.tolist()[:3] == [1, 1, 1]   # flag timeout on K range 1 / flag 1


def test_k_gated_schedule_errors():
    from syncopate_b200 import _lib as L
    from syncopate_b200.computation.gemm import gemm

    a = torch.zeros(256, 256, dtype=DT, device="cuda")
    c = torch.zeros(256, 256, dtype=DT, device="cuda")
    with pytest.raises(L.SynError, match="SYN_ERR_SHAPE"):      # the ranges leave a hole
        gemm(a, a, c, cur_wave_sizes=[[256, 256, 64]], wave_offsets=[[0, 0, 0]], signal_offsets=[-1])
    with pytest.raises(L.SynError, match="SYN_ERR_SHAPE"):      # overlapping ranges
        gemm(a, a, c, cur_wave_sizes=[[256, 256, 192], [256, 256, 128]], wave_offsets=[[0, 0, 0], [0, 0, 128]],
             signal_offsets=[-1, -1])
    with pytest.raises(L.SynError, match="SYN_ERR_UNSUPPORTED"):  # a K range must span all of C
        gemm(a, a, c, cur_wave_sizes=[[128, 256, 256]], wave_offsets=[[0, 0, 0]], signal_offsets=[-1])


@pytest.mark.parametrize("world,rank", [(4, 1), (2, 0)])
def test_closed_form_schedule_matches_the_explicit_one(world, rank):
    """The swizzled all-gather's lowered schedule simplifies to a Mod1DSchedule; the GEMM driven by
    the closed form equals the GEMM driven by the schedule arrays, bit for bit."""
    from syncopate_b200.computation.gemm import gemm, gemm_mod1d
    from syncopate_b200.interface.tile_schedule import Mod1DSchedule, SimplifiedSchedule
    from syncopate_b200.operators import plan_all_gather

    rows, K, N = 256, 256, 384
    _gen, info, low = plan_all_gather(world, rows, K, DT, "swizzle")
    raw = low[rank]["a"]
    simple = SimplifiedSchedule(raw)
    assert simple.simplify() and isinstance(simple.simplified_schedule, Mod1DSchedule)
    form = simple.simplified_schedule
    assert (form.num_waves, form.stride, form.starting_offset, form.schedule_axis) == (world, rows, rank * rows, 0)
    a, b = _seeded(5, (world * rows, K)).cuda(), _seeded(6, (N, K), 0.02).cuda()
    flags = torch.ones(max(info.recv_signal_num, 1), dtype=torch.int64, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    c1 = torch.zeros(world * rows, N, dtype=DT, device="cuda")
    c2 = torch.zeros_like(c1)
    gemm_mod1d(a, b, c1, form, flags, status=status)
    gemm(a, b, c2, cur_wave_sizes=[[s[0], N] for s in raw.gen_block_shape_lists()],
         wave_offsets=[[o[0], 0] for o in raw.gen_block_offset_lists()], signal_ptr=flags,
         signal_offsets=raw.gen_signal_lists(), status=status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    assert torch.equal(c1, c2)
    assert_gemm_close(c1, a.float() @ b.float().t())


@pytest.mark.parametrize("world,B,S,H,D,N", [(2, 1, 512, 4, 128, 512), (4, 2, 512, 8, 64, 256)])
def test_all_to_all_gemm_emulated_ranks(world, B, S, H, D, N):
    from syncopate_b200.operators import AllToAllGemm
    from syncopate_b200.runtime import EmulatedWorld

    ew = EmulatedWorld(world)
    ops = [AllToAllGemm(c, B, S, H, D, N, DT, num_copy_sms=8, timeout_ns=500_000_000) for c in ew.contexts]
    Hl, Sl = H // world, S // world
    xs = [_seeded(10 + r, (B, S, Hl, D)) for r in range(world)]
    w = _seeded(3, (N, H * D), 0.02).cuda()
    full = torch.cat(xs, dim=2)  # [B, S, H, D]: rank r holds heads [r * Hl, (r + 1) * Hl)
    for it in range(2):
        for r, op in enumerate(ops):
            op.src.copy_(xs[r].cuda())
            op.comm.comm_buffers["dst"][r].fill_(float("nan"))
        for op in ops:
            op.send()
        torch.cuda.synchronize()
        for r, op in enumerate(ops):
            out = op.consume(w)
            torch.cuda.synchronize()
            op.ctx.check()
            a_ref = full[:, r * Sl:(r + 1) * Sl].reshape(B * Sl, H * D)
            assert torch.equal(op.a.cpu(), a_ref)                      # the re-sharded input: bit-exact
            assert_gemm_close(out, a_ref.float() @ w.float().cpu().t(), f"rank {r}")


@pytest.mark.parametrize("world,M,hidden,ffn", [(2, 512, 256, 1024), (4, 1024, 512, 1024)])
def test_gemm_all_to_all_gemm_emulated_ranks(world, M, hidden, ffn):
    from syncopate_b200.operators import GemmAllToAllGemm
    from syncopate_b200.runtime import EmulatedWorld

    ew = EmulatedWorld(world)
    ops = [GemmAllToAllGemm(c, M, hidden, ffn, DT, num_copy_sms=8, timeout_ns=500_000_000) for c in ew.contexts]
    x = _seeded(1, (M, hidden), 0.1)
    w1 = [_seeded(20 + r, (ffn // world, hidden), 0.1) for r in range(world)]
    w2 = _seeded(2, (hidden, ffn), 0.1)
    mid = x.float() @ torch.cat(w1, 0).float().t()                      # [M, ffn]
    want = mid.to(DT).float() @ w2.float().t()                          # the middle activations are 16 bit
    for it in range(2):
        for op in ops:
            op.a2.fill_(float("nan"))
        for r, op in enumerate(ops):
            op.produce_and_send(x.cuda(), w1[r].cuda())
        torch.cuda.synchronize()
        for r, op in enumerate(ops):
            out = op.consume(w2.cuda())
            torch.cuda.synchronize()
            op.ctx.check()
            rows = slice(r * (M // world), (r + 1) * (M // world))
            assert_gemm_close(op.a2, mid[rows], f"rank {r} middle")
            assert_gemm_close(out, want[rows], f"rank {r}")
