"""GPU parity of the tcgen05 GEMM and of the fused operators, through the C ABI, against the CPU
oracle (same seeded inputs).  Tolerance: relative Frobenius error <= 1e-2 for 16-bit outputs of an
fp32-accumulated product (the bound the operators are specified to), applied to the whole output
AND to every 128 x 256 tile of it, plus an element-wise bound of a few output rounding steps
(tests/parity.py); the values seen are ~2e-3, i.e. output rounding."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle import emulate as E  # noqa: E402
from parity import assert_gemm_close, gemm_errors  # noqa: E402

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _rel(x, ref):
    return ((x.float().cpu() - ref.float()).norm() / ref.float().norm()).item()


def _seeded(seed, shape, scale, dtype):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g, dtype=torch.float32) * scale).to(dtype)


@pytest.fixture(scope="module")
def status():
    return torch.zeros(4, dtype=torch.int32, device="cuda")


@pytest.mark.parametrize(
    "M,N,K,bn,dtype",
    [
        (128, 256, 64, 256, torch.bfloat16),
        (256, 512, 512, 256, torch.bfloat16),
        (384, 448, 192, 224, torch.bfloat16),
        (128, 128, 128, 128, torch.float16),
        (200, 264, 136, 64, torch.bfloat16),      # ragged M, N and K edges
        (1024, 1024, 1024, 0, torch.float16),
        (8, 8, 8, 0, torch.bfloat16),             # smaller than one tile
    ],
)
def test_local_gemm_matches_oracle(M, N, K, bn, dtype, status):
    from syncopate_b200.computation.gemm import gemm

    a, b = _seeded(1, (M, K), 1.0, dtype), _seeded(2, (N, K), 0.02, dtype)
    c = torch.zeros(M, N, dtype=dtype, device="cuda")
    gemm(a.cuda(), b.cuda(), c, BLOCK_SIZE_N=bn, status=status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    ref = a.float() @ b.float().t()
    assert_gemm_close(c, ref)


def test_pair_kernel_with_split_tail(status):
    """76 tiles of 256 x 256 on 74 CTA pairs: one full round, the two left-over tiles are cut along K
    over all pairs and reduced through the fp32 workspace; twice, to see the workspace counters rewind."""
    from syncopate_b200.computation.gemm import gemm

    M, N, K = 4864, 1024, 2048
    a, b = _seeded(7, (M, K), 1.0, torch.bfloat16), _seeded(8, (N, K), 0.02, torch.bfloat16)
    ref = a.float() @ b.float().t()
    ad, bd = a.cuda(), b.cuda()
    for _ in range(2):
        c = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
        gemm(ad, bd, c, BLOCK_SIZE_N=256, status=status)
        torch.cuda.synchronize()
        assert status.tolist() == [0, 0, 0, 0]
        assert_gemm_close(c, ref)


def test_gemm_rejects_bad_arguments(status):
    from syncopate_b200 import _lib as L
    from syncopate_b200.computation.gemm import gemm

    a = torch.zeros(128, 60, dtype=torch.bfloat16, device="cuda")  # K pitch not a multiple of 16 bytes
    b = torch.zeros(128, 60, dtype=torch.bfloat16, device="cuda")
    c = torch.zeros(128, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(L.SynError, match="SYN_ERR_INVALID"):
        gemm(a, b, c)
    a = torch.zeros(256, 64, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros(256, 64, dtype=torch.bfloat16, device="cuda")
    c = torch.zeros(256, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(L.SynError, match="SYN_ERR_SHAPE"):  # wave reaches past M
        gemm(a, b, c, cur_wave_sizes=[[256, 256]], wave_offsets=[[128, 0]], signal_offsets=[-1])
    with pytest.raises(L.SynError, match="SYN_ERR_SHAPE"):  # wave offset not on a tile boundary
        gemm(a, b, c, cur_wave_sizes=[[128, 256]], wave_offsets=[[64, 0]], signal_offsets=[-1])


def test_wave_schedule_with_consumer_flags(status):
    from syncopate_b200.computation.gemm import gemm

    M, N, K = 1024, 512, 512
    a, b = _seeded(3, (M, K), 1.0, torch.bfloat16), _seeded(4, (N, K), 0.02, torch.bfloat16)
    sched = E.swizzle_pull_schedule(4, 2, 256, N)
    flags = torch.ones(3, dtype=torch.int64, device="cuda")  # all chunks already "arrived"
    c = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    gemm(a.cuda(), b.cuda(), c, cur_wave_sizes=sched["shapes"], wave_offsets=sched["offsets"], signal_ptr=flags,
         signal_offsets=sched["signals"], status=status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    assert_gemm_close(c, a.float() @ b.float().t())


def test_flag_that_is_never_set_times_out_cleanly():
    """A wave whose flag nobody raises must end the kernel with a status code after the bounded
    wait (1 ms here), leaving the context usable."""
    from syncopate_b200.computation.gemm import gemm

    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    a = torch.zeros(256, 64, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros(256, 64, dtype=torch.bfloat16, device="cuda")
    c = torch.zeros(256, 256, dtype=torch.bfloat16, device="cuda")
    flags = torch.zeros(2, dtype=torch.int64, device="cuda")
    gemm(a, b, c, cur_wave_sizes=[[128, 256], [128, 256]], wave_offsets=[[0, 0], [128, 0]], signal_ptr=flags,
         signal_offsets=[-1, 1], timeout_ns=1_000_000, status=status)
    torch.cuda.synchronize()
    code, wave, flag, _block = status.tolist()
    assert code == 1 and wave == 1 and flag == 1   # SYN_DEV_TIMEOUT_FLAG on wave 1 / flag 1
    status.zero_()
    gemm(a, b, c, status=status)                   # the context still works
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]


def test_producer_flags_are_raised_after_each_wave(status):
    from syncopate_b200.computation.gemm import gemm

    M, N, K = 512, 512, 256
    a, b = _seeded(5, (M, K), 1.0, torch.bfloat16), _seeded(6, (N, K), 0.02, torch.bfloat16)
    c = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    flags = torch.zeros(4, dtype=torch.int64, device="cuda")
    counters = torch.zeros(130, dtype=torch.int32, device="cuda")
    offs = [[128, 0], [256, 0], [384, 0], [0, 0]]
    for epoch in (1, 2):
        gemm(a.cuda(), b.cuda(), c, cur_wave_sizes=[[128, N]] * 4, wave_offsets=offs, signal_offsets=[-1] * 4,
             producer_signal_ptr=flags, producer_signal_offsets=[3, 2, -1, 0], counter_ptr=counters,
             signal_value=epoch, status=status)
        torch.cuda.synchronize()
        assert flags.tolist() == [epoch, 0, epoch, epoch]
        assert int(counters.abs().sum()) == 0
    assert_gemm_close(c, a.float() @ b.float().t())


def _front_end(builder_kwargs, builder):
    from syncopate_b200.communication import common_descriptors as cd
    from syncopate_b200.communication.code_gen import CodeGenOptions, CommGenerator
    from syncopate_b200.interface import lower_comm_plan_to_raw_schedules

    world = builder_kwargs["mesh_size"]
    plans = {r: getattr(cd, builder)(rank=r, **builder_kwargs) for r in range(world)}
    gen = CommGenerator(plans)
    gen.plan_signals()
    info = gen.generate_code_for_plan(CodeGenOptions(copy_engine=False))
    return info, lower_comm_plan_to_raw_schedules(gen)


@pytest.mark.parametrize("world,rows,K,N,kind", [(4, 256, 512, 512, "swizzle"), (2, 1024, 1024, 1792, "swizzle"),
                                                 (4, 128, 256, 256, "ring")])
def test_fused_ag_gemm_emulated_ranks(world, rows, K, N, kind, status):
    """All ranks of the plan on one GPU, one after the other, with local pointer tables: the comm
    warps pull every remote chunk, raise the flags, and the tiles consume them."""
    from syncopate_b200 import _lib as L
    from syncopate_b200.computation.gemm import ag_gemm
    from syncopate_b200.operators import plan_all_gather

    dt = torch.bfloat16
    _gen, info, low = plan_all_gather(world, rows, K, dt, kind)
    shards = [_seeded(10 + r, (rows, K), 1.0, dt) for r in range(world)]
    bufs = []
    for r in range(world):
        buf = torch.full((world * rows, K), float("nan"), dtype=dt, device="cuda")
        buf[r * rows : (r + 1) * rows] = shards[r].cuda()
        bufs.append(buf)
    full = torch.cat(shards, 0)
    for r in range(world):
        b = _seeded(20 + r, (N, K), 0.02, dt)
        sched = low[r]["a"]
        o_gather, o_c = E.ag_gemm({"offsets": sched.gen_block_offset_lists(), "shapes": sched.gen_block_shape_lists()},
                                  shards, b)
        c = torch.zeros(world * rows, N, dtype=dt, device="cuda")
        flags = torch.zeros(max(info.recv_signal_num, 1), dtype=torch.int64, device="cuda")
        counters = torch.zeros(130, dtype=torch.int32, device="cuda")
        symm = L.Symm.of(r, [x.data_ptr() for x in bufs])
        for epoch in (1, 2):
            if epoch == 2:  # forget the gathered chunks: the second call must fetch them again
                bufs[r][:] = float("nan")
                bufs[r][r * rows : (r + 1) * rows] = shards[r].cuda()
            ag_gemm(symm, bufs[r], b.cuda(), c, sched, flags, counters, epoch=epoch, timeout_ns=500_000_000,
                    status=status)
            torch.cuda.synchronize()
            assert status.tolist() == [0, 0, 0, 0]
            assert torch.equal(bufs[r].cpu(), o_gather)          # bytes moved: bit-exact
            assert torch.equal(bufs[r].cpu(), full)
            assert_gemm_close(c, o_c)
            assert flags.tolist() == [epoch] * info.recv_signal_num
            assert int(counters.abs().sum()) == 0


@pytest.mark.parametrize("world,M,N,Kl,kind", [(4, 1024, 512, 256, "direct"), (4, 1024, 512, 256, "a2a"),
                                                (2, 512, 1024, 512, "direct")])
def test_fused_gemm_rs_emulated_ranks(world, M, N, Kl, kind, status):
    """All ranks on one GPU: first every rank's pushing waves, then every rank's owner wave (which
    adds the staged partial sums), twice to exercise the epoch-parity staging halves."""
    from syncopate_b200 import _lib as L
    from syncopate_b200.computation.gemm import gemm_rs
    from syncopate_b200.computation.gemm.plan import rs_remote_signals
    from syncopate_b200.operators import plan_reduce_scatter

    dt = torch.bfloat16
    slab = M // world
    _gen, info, low = plan_reduce_scatter(world, M, N, dt, kind)
    A = [_seeded(30 + r, (M, Kl), 1.0, dt) for r in range(world)]
    B = [_seeded(40 + r, (N, Kl), 0.02, dt) for r in range(world)]
    scheds = [{"offsets": low[r]["src"].gen_block_offset_lists(), "shapes": low[r]["src"].gen_block_shape_lists()}
              for r in range(world)]
    want = E.gemm_rs(scheds, A, B, out_dtype=torch.float32)
    Ad, Bd = [x.cuda() for x in A], [x.cuda() for x in B]
    stages = [torch.full((2, world, slab, N), float("nan"), dtype=dt, device="cuda") for _ in range(world)]
    flags = [torch.zeros(max(info.recv_signal_num, 1), dtype=torch.int64, device="cuda") for _ in range(world)]
    outs = [torch.zeros(slab, N, dtype=dt, device="cuda") for _ in range(world)]
    counters = torch.zeros(130, dtype=torch.int32, device="cuda")
    for epoch in (1, 2):
        for phase in (0, 1):
            for r in range(world):
                src, dst = low[r]["src"], low[r]["dst"]
                rsig = rs_remote_signals(info, r, src)
                cols = (src.gen_block_offset_lists(), src.gen_block_shape_lists(), src.gen_signal_lists(),
                        src.gen_target_rank_list(), src.gen_dst_offset_lists())
                tgt = cols[3]
                own = [i for i in range(len(tgt)) if tgt[i] < 0 or tgt[i] == r]
                sel = own if phase == 1 else [i for i in range(len(tgt)) if i not in own]
                sched = tuple([col[i] for i in sel] for col in cols)
                gemm_rs(Ad[r], Bd[r], outs[r], sched, dst, [rsig[i] for i in sel],
                        L.Symm.of(r, [x.data_ptr() for x in stages]), L.Symm.of(r, [x.data_ptr() for x in flags]),
                        counters, epoch=epoch, timeout_ns=500_000_000, status=status)
                torch.cuda.synchronize()
                assert status.tolist() == [0, 0, 0, 0]
        for r in range(world):
            assert_gemm_close(outs[r], want[r])
            outs[r].zero_()


def test_full_size_cfg1_local_shape_against_fp32_reference(status):
    """The 1-GPU benchmark shape (per-rank share of AG+GEMM at world 8: [8192,8192] x [3584,8192]^T),
    checked on the device against an fp32 matmul of the same 16-bit inputs."""
    from syncopate_b200.computation.gemm import gemm

    M, N, K = 8192, 3584, 8192
    g = torch.Generator(device="cuda").manual_seed(1000)
    a = torch.randn(M, K, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    b = (torch.randn(N, K, generator=g, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
    c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    sched = E.swizzle_pull_schedule(8, 3, 1024, N)
    flags = torch.ones(7, dtype=torch.int64, device="cuda")
    gemm(a, b, c, cur_wave_sizes=sched["shapes"], wave_offsets=sched["offsets"], signal_ptr=flags,
         signal_offsets=sched["signals"], status=status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        worst = [0.0, 0.0, 0.0]
        for r0 in range(0, M, 2048):  # fp32 reference in row blocks to bound memory
            ref = a[r0 : r0 + 2048].float() @ b.float().t()
            glob, tile, maxabs, allowed = gemm_errors(c[r0 : r0 + 2048], ref)
            worst = [max(worst[0], glob), max(worst[1], tile), max(worst[2], maxabs / allowed)]
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    print(f"cfg1 local shape: relative Frobenius {worst[0]:.2e}, worst 128x256 tile {worst[1]:.2e}, "
          f"max-abs / allowed {worst[2]:.2f}")
    assert worst[0] < TOL and worst[1] < TOL and worst[2] <= 1.0


def test_timed_out_launch_leaves_the_tail_workspace_usable(status):
    """A launch that gives up on a flag (1 ms bound) on a shape whose left-over tiles are split
    along K, then the same shape without the flag: every CTA of a split tile still arrives and
    departs once on the give-up path, so the workspace counters rewind and the next launch is
    exact."""
    from syncopate_b200.computation.gemm import gemm

    M, N, K = 4864, 1024, 2048
    a, b = _seeded(7, (M, K), 1.0, torch.bfloat16).cuda(), _seeded(8, (N, K), 0.02, torch.bfloat16).cuda()
    c = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    flags = torch.zeros(1, dtype=torch.int64, device="cuda")
    st = torch.zeros(4, dtype=torch.int32, device="cuda")
    gemm(a, b, c, BLOCK_SIZE_N=256, cur_wave_sizes=[[M, N]], wave_offsets=[[0, 0]], signal_ptr=flags,
         signal_offsets=[0], timeout_ns=1_000_000, status=st)
    torch.cuda.synchronize()
    assert st.tolist()[0] == 1           # the flag wait ran out
    c.zero_()
    gemm(a, b, c, BLOCK_SIZE_N=256, status=status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    assert_gemm_close(c, a.float() @ b.float().t(), "after a timed-out launch")


@pytest.mark.parametrize("world,rows,K,N,split,comm_pair", [(2, 512, 512, 768, 2, True), (4, 1024, 256, 512, 4, True),
                                                            (2, 384, 256, 256, 3, False)])
def test_fused_ag_gemm_with_split_chunks(world, rows, K, N, split, comm_pair, status):
    """Every remote slab arrives as ``split`` row pieces with flags of their own; with 256-row pieces
    the CTA-pair kernel runs with its comm warps, otherwise the one-CTA kernel."""
    from syncopate_b200 import _lib as L
    from syncopate_b200.computation.gemm import ag_gemm
    from syncopate_b200.operators import plan_all_gather

    dt = torch.bfloat16
    _gen, info, low = plan_all_gather(world, rows, K, dt, "swizzle", chunk_split=split)
    assert info.recv_signal_num == (world - 1) * split
    shards = [_seeded(10 + r, (rows, K), 1.0, dt) for r in range(world)]
    full = torch.cat(shards, 0)
    bufs = []
    for r in range(world):
        buf = torch.full((world * rows, K), float("nan"), dtype=dt, device="cuda")
        buf[r * rows : (r + 1) * rows] = shards[r].cuda()
        bufs.append(buf)
    for r in range(world):
        b = _seeded(20 + r, (N, K), 0.02, dt)
        sched = low[r]["a"]
        assert len(sched.gen_signal_lists()) == 1 + (world - 1) * split
        c = torch.zeros(world * rows, N, dtype=dt, device="cuda")
        flags = torch.zeros(info.recv_signal_num, dtype=torch.int64, device="cuda")
        counters = torch.zeros(130, dtype=torch.int32, device="cuda")
        for epoch in (1, 2):
            bufs[r][:] = float("nan")
            bufs[r][r * rows : (r + 1) * rows] = shards[r].cuda()
            ag_gemm(L.Symm.of(r, [x.data_ptr() for x in bufs]), bufs[r], b.cuda(), c, sched, flags, counters,
                    epoch=epoch, timeout_ns=500_000_000, status=status)
            torch.cuda.synchronize()
            assert status.tolist() == [0, 0, 0, 0]
            assert torch.equal(bufs[r].cpu(), full)              # bytes moved: bit-exact
            assert_gemm_close(c, full.float() @ b.float().t())
            assert flags.tolist() == [epoch] * info.recv_signal_num
            assert int(counters.abs().sum()) == 0


def _rs_phase_schedule(src, rsig, rank, own: bool):
    cols = (src.gen_block_offset_lists(), src.gen_block_shape_lists(), src.gen_signal_lists(),
            src.gen_target_rank_list(), src.gen_dst_offset_lists())
    tgt = cols[3]
    sel = [i for i in range(len(tgt)) if (tgt[i] < 0 or tgt[i] == rank) == own]
    return tuple([col[i] for i in sel] for col in cols), [rsig[i] for i in sel], sel


@pytest.mark.parametrize("world,M,N,Kl,split,transport", [(2, 1024, 512, 256, 2, "push"), (4, 2048, 256, 128, 2, "push"),
                                                          (2, 1024, 512, 256, 2, "local"), (4, 1536, 256, 128, 3, "push")])
@pytest.mark.parametrize("reduce_pass", [False, True])
def test_fused_gemm_rs_with_split_slabs(world, M, N, Kl, split, transport, reduce_pass, status):
    """Every slab leaves as ``split`` row pieces (flags of their own) and the rows kept by a rank are
    reduced piece by piece.  ``push``: the epilogue's TMA stores write the peers' staging slabs;
    ``local``: the epilogue fills the local send buffer and raises the local per-wave flags, and the
    test plays the transport (copy the rows, raise the receiver's flag).  256-row pieces run on the
    CTA-pair kernel, 128-row pieces on the one-CTA kernel.  ``reduce_pass``: the staged partial sums
    are added by the pass behind the kernel instead of the own tiles' epilogue."""
    from syncopate_b200 import _lib as L
    from syncopate_b200.computation.gemm import gemm_rs
    from syncopate_b200.computation.gemm.plan import rs_remote_signals, rs_transport_program
    from syncopate_b200.operators import plan_reduce_scatter

    dt = torch.bfloat16
    slab = M // world
    _gen, info, low = plan_reduce_scatter(world, M, N, dt, "direct", chunk_split=split)
    A = [_seeded(30 + r, (M, Kl), 1.0, dt) for r in range(world)]
    B = [_seeded(40 + r, (N, Kl), 0.02, dt) for r in range(world)]
    scheds = [{"offsets": low[r]["src"].gen_block_offset_lists(), "shapes": low[r]["src"].gen_block_shape_lists()}
              for r in range(world)]
    want = E.gemm_rs(scheds, A, B, out_dtype=torch.float32)
    Ad, Bd = [x.cuda() for x in A], [x.cuda() for x in B]
    stages = [torch.full((2, world, slab, N), float("nan"), dtype=dt, device="cuda") for _ in range(world)]
    flags = [torch.zeros(max(info.recv_signal_num, 1), dtype=torch.int64, device="cuda") for _ in range(world)]
    outs = [torch.zeros(slab, N, dtype=dt, device="cuda") for _ in range(world)]
    counters = torch.zeros(130, dtype=torch.int32, device="cuda")
    stage_symm = lambda r: L.Symm.of(r, [x.data_ptr() for x in stages])
    flag_symm = lambda r: L.Symm.of(r, [x.data_ptr() for x in flags])
    for epoch in (1, 2):
        for own in (False, True):
            for r in range(world):
                src, dst = low[r]["src"], low[r]["dst"]
                rsig = rs_remote_signals(info, r, src)
                sched, sig_sel, sel = _rs_phase_schedule(src, rsig, r, own)
                kw = {}
                if own:
                    kw = dict(out_flags=torch.zeros(split, dtype=torch.int64, device="cuda"), reduce_pass=reduce_pass)
                if transport == "local" and not own:
                    send = torch.full((world, slab, N), float("nan"), dtype=dt, device="cuda")
                    send_flags = torch.zeros(len(sel), dtype=torch.int64, device="cuda")
                    kw = dict(send_buf=send, send_flags=send_flags)
                gemm_rs(Ad[r], Bd[r], outs[r], sched, dst, sig_sel, stage_symm(r), flag_symm(r), counters, epoch=epoch,
                        timeout_ns=500_000_000, status=status, **kw)
                torch.cuda.synchronize()
                assert status.tolist() == [0, 0, 0, 0]
                assert int(counters.abs().sum()) == 0
                if own:
                    assert kw["out_flags"].tolist() == [epoch] * split    # one local flag per reduced row piece
                elif kw:
                    assert send_flags.tolist() == [epoch] * len(sel)   # one local flag per wave
                    # the transport program addresses waves by their index in the schedule it is given
                    class _Sub:
                        gen_block_offset_lists = staticmethod(lambda: sched[0])
                        gen_block_shape_lists = staticmethod(lambda: sched[1])
                        gen_target_rank_list = staticmethod(lambda: sched[3])
                    prog = rs_transport_program(r, world, slab, N * 2, epoch, _Sub, sig_sel, send.data_ptr(),
                                                send_flags.data_ptr(), [x.data_ptr() for x in stages],
                                                [x.data_ptr() for x in flags])
                    assert len(prog) == len(sel)
                    for lflag, src_addr, dst_addr, nbytes, rflag in prog:
                        t = next(i for i in range(world) if stages[i].data_ptr() <= dst_addr < stages[i].data_ptr() + stages[i].numel() * 2)
                        so, do = (src_addr - send.data_ptr()) // 2, (dst_addr - stages[t].data_ptr()) // 2
                        stages[t].view(-1)[do : do + nbytes // 2] = send.view(-1)[so : so + nbytes // 2]
                        flags[t][(rflag - flags[t].data_ptr()) // 8] = epoch
        for r in range(world):
            assert_gemm_close(outs[r], want[r], f"rank {r} epoch {epoch}")
            outs[r].zero_()


def test_reduce_pass_with_a_missing_partial_sum_times_out_cleanly(status):
    """The reduce pass behind the kernel waits with a bound: when a peer's partial sum never
    arrives, the pass records the timeout, leaves the own partial sum in place, and the local
    flag of the piece is still raised, so that nothing downstream is left waiting."""
    from syncopate_b200 import _lib as L
    from syncopate_b200.computation.gemm import gemm_rs
    from syncopate_b200.computation.gemm.plan import rs_remote_signals
    from syncopate_b200.operators import plan_reduce_scatter

    world, M, N, Kl, dt = 2, 512, 256, 128, torch.bfloat16
    slab = M // world
    _gen, info, low = plan_reduce_scatter(world, M, N, dt, "direct")
    src, dst = low[0]["src"], low[0]["dst"]
    rsig = rs_remote_signals(info, 0, src)
    sched, sig_sel, _sel = _rs_phase_schedule(src, rsig, 0, own=True)
    a, b = _seeded(70, (M, Kl), 1.0, dt).cuda(), _seeded(71, (N, Kl), 0.02, dt).cuda()
    stages = [torch.zeros(2, world, slab, N, dtype=dt, device="cuda") for _ in range(world)]
    flags = [torch.zeros(max(info.recv_signal_num, 1), dtype=torch.int64, device="cuda") for _ in range(world)]
    out = torch.zeros(slab, N, dtype=dt, device="cuda")
    out_flags = torch.zeros(1, dtype=torch.int64, device="cuda")
    counters = torch.zeros(130, dtype=torch.int32, device="cuda")
    gemm_rs(a, b, out, sched, dst, sig_sel, L.Symm.of(0, [x.data_ptr() for x in stages]),
            L.Symm.of(0, [x.data_ptr() for x in flags]), counters, epoch=1, timeout_ns=20_000_000, status=status,
            out_flags=out_flags, reduce_pass=True)
    torch.cuda.synchronize()
    got = status.tolist()
    assert got[0] == 1 and got[2] <= -2, got       # flag timeout, in a reduce wait
    assert out_flags.tolist() == [1]
    assert_gemm_close(out, a[:slab].float().cpu() @ b.float().cpu().t(), "own partial sum")
    # the same launch succeeds once the partial sum is there
    status.zero_()
    flags[0].fill_(2)
    gemm_rs(a, b, out, sched, dst, sig_sel, L.Symm.of(0, [x.data_ptr() for x in stages]),
            L.Symm.of(0, [x.data_ptr() for x in flags]), counters, epoch=2, timeout_ns=20_000_000, status=status,
            out_flags=out_flags, reduce_pass=True)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0] and out_flags.tolist() == [2]
