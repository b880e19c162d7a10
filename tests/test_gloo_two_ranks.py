"""Host-side multi-rank logic on CPU: two gloo ranks build the plans, marshal the per-rank kernel
arguments and exchange data the way the GPU ranks do, and the result is checked against the
single-process oracle.  No GPU and no CUDA call is involved."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import emulate as E
        from syncopate_b200.computation.attn.plan import all_to_all_wave_metadata, pull_ops_from_schedule
        from syncopate_b200.computation.gemm.plan import rs_remote_signals
        from syncopate_b200.operators import _plan, plan_all_gather, plan_reduce_scatter
        from syncopate_b200.communication.common_descriptors import build_all_to_all_plan_dim

        dt = torch.bfloat16
        rows, K, N = 64, 32, 48
        # ---- all-gather + GEMM: every rank derives its own schedule; data moves with gloo
        _g, info, low = plan_all_gather(world, rows, K, dt)
        sched = low[rank]["a"]
        g = torch.Generator().manual_seed(100 + rank)
        shard = torch.randn(rows, K, generator=g).to(dt)
        b = (torch.randn(N, K, generator=g) * 0.02).to(dt)
        gathered = [torch.empty_like(shard) for _ in range(world)]
        dist.all_gather(gathered, shard)
        mine = {"offsets": sched.gen_block_offset_lists(), "shapes": sched.gen_block_shape_lists()}
        assert mine["offsets"] == E.swizzle_pull_schedule(world, rank, rows, K)["offsets"]
        full, c = E.ag_gemm(mine, gathered, b, out_dtype=torch.float32)
        assert torch.equal(full, torch.cat(gathered, 0))
        assert torch.equal(c, torch.cat(gathered, 0).float() @ b.float().t())

        # ---- GEMM + reduce-scatter: the flag a sender raises is the flag its receiver waits for
        _g, rs_info, rs_low = plan_reduce_scatter(world, 256, 64, dt, "direct")
        sent = rs_remote_signals(rs_info, rank, rs_low[rank]["src"])
        table = [None] * world
        dist.all_gather_object(table, sent)
        dst = rs_low[rank]["dst"]
        for src_rank, sig in zip(dst.gen_target_rank_list(), dst.gen_signal_lists()):
            if src_rank < 0 or src_rank == rank:
                continue
            src_sched = rs_low[src_rank]["src"]
            wave = src_sched.gen_target_rank_list().index(rank)
            assert table[src_rank][wave] == sig

        # ---- GEMM + reduce-scatter with the slabs moved by somebody else than the kernel: every rank
        # runs its transport program against a byte image of all ranks' staging buffers (addresses are
        # offsets into per-rank arrays here), then the owner sums the staged slabs with its own
        from syncopate_b200.computation.gemm.plan import rs_transport_program

        M, Nn, slab = 256, 64, 256 // world
        slab_bytes = slab * Nn * 2
        g2 = torch.Generator().manual_seed(300 + rank)
        partial = torch.randn(M, Nn, generator=g2).to(dt)             # this rank's partial product
        BASE = 1 << 20                                                 # "address" of a rank's staging / flag arrays
        for epoch in (1, 2):
            prog = rs_transport_program(rank, world, slab, Nn * 2, epoch, rs_low[rank]["src"], sent,
                                        send_ptr=0, send_flags_ptr=0, stage_ptrs=[BASE * (t + 1) for t in range(world)],
                                        flag_ptrs=[BASE * (t + 1) for t in range(world)])
            assert len(prog) == world - 1
            moves = []
            src_targets = rs_low[rank]["src"].gen_target_rank_list()
            for lflag, src_addr, dst_addr, nbytes, rflag in prog:
                tgt = dst_addr // BASE - 1
                assert lflag == 8 * src_targets.index(tgt) and src_addr == tgt * slab_bytes and nbytes == slab_bytes
                slot = (dst_addr - BASE * (tgt + 1)) // slab_bytes
                assert slot == (epoch & 1) * world + rank
                moves.append((tgt, slot, (rflag - BASE * (tgt + 1)) // 8, partial[tgt * slab:(tgt + 1) * slab].clone()))
            everyone = [None] * world
            dist.all_gather_object(everyone, moves)
            staged = {}
            raised = set()
            for src_rank, mv in enumerate(everyone):
                for tgt, slot, flag, data in mv:
                    if tgt == rank:
                        assert slot not in staged      # no two senders share a slot
                        staged[slot] = data
                        raised.add(flag)
            # the flags that were raised here are exactly the ones this rank's owner wave waits for
            waits = {sig for src_rank, sig in zip(dst.gen_target_rank_list(), dst.gen_signal_lists())
                     if src_rank >= 0 and src_rank != rank}
            assert raised == waits
            total = partial[rank * slab:(rank + 1) * slab].float()
            for data in staged.values():
                total = total + data.float()
            parts = [None] * world
            dist.all_gather_object(parts, partial)
            want = sum(p_[rank * slab:(rank + 1) * slab].float() for p_ in parts)
            assert torch.allclose(total, want, atol=1e-6)

        # ---- Ulysses reshard: the comm warps' copy list moves exactly the bytes the plan describes
        shape = (3, 1, 2 * world, 16, 8)
        _g, a2a_info, a2a_low = _plan({
            r: build_all_to_all_plan_dim(shape, dtype=dt, mesh_size=world, rank=r, src_buffer="src", dst_buffer="dst",
                                         src_split_axis=3, dst_split_axis=2, transfer_kind="pull")
            for r in range(world)})
        dst_shape = (3, 1, 2, 16 * world, 8)
        ops = pull_ops_from_schedule(a2a_low[rank]["dst"], rank, world, shape, dst_shape, 4, 0, 1)  # 4-byte elements here
        src = torch.arange(rank * 10000, rank * 10000 + 3 * 2 * world * 16 * 8, dtype=torch.int32).reshape(shape)
        srcs = [torch.empty_like(src) for _ in range(world)]
        dist.all_gather(srcs, src)
        out = torch.zeros(dst_shape, dtype=torch.int32)
        flat_out = out.view(-1).view(torch.uint8)
        for op in ops:
            flat_src = srcs[op.src_rank].reshape(-1).view(torch.uint8)
            for r_ in range(op.rows):
                so, do = op.src_offset + r_ * op.src_pitch, op.dst_offset + r_ * op.dst_pitch
                flat_out[do : do + op.row_bytes] = flat_src[so : so + op.row_bytes]
        want = torch.cat([s[:, :, 2 * rank : 2 * rank + 2] for s in srcs], dim=3)
        assert torch.equal(out, want)
        offs, sizes, sigs, cum = all_to_all_wave_metadata(a2a_low[rank]["dst"], {"batch": 1, "head": 2, "seq": 3})
        assert len(offs) == world * world and cum[-1] == 2 * 16 * world * world
        results[rank] = "ok"
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_gloo_ranks_agree_with_the_oracle():
    world = 2
    port = _free_port()
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert dict(results) == {0: "ok", 1: "ok"}
