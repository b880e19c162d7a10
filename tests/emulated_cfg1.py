"""One fused GEMM launch at the benchmark's per-rank shapes with all eight ranks' buffers on ONE GPU
(``EmulatedWorld``), checked against torch: a stand-alone case for looking at the fused kernels
under a profiler on a one-GPU box (a few GB of device memory, one launch of the kernel of interest).

    python tests/emulated_cfg1.py --op ag    # rank 0 of AG+GEMM: comm warps pull seven 16.8 MB slabs while the tiles run
    python tests/emulated_cfg1.py --op rs    # rank 0 of GEMM+RS, the seven remote waves: the routed epilogue's TMA stores
    python tests/emulated_cfg1.py --op rs-pass      # rank 0's whole GEMM+RS schedule, flags pre-set, reduce pass behind the kernel
    python tests/emulated_cfg1.py --op rs-epilogue  # the same with the reduction in the own tiles' epilogue

Peer buffers live in the same HBM here, so transfer RATES say nothing about NVLink; what the case
shows is what the comm warp and the routed epilogue cost the tensor pipe."""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def seeded(seed, shape, scale):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g, dtype=torch.float32) * scale).to(torch.bfloat16)


def rel(x, ref):
    return ((x.float() - ref).norm() / ref.norm()).item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", choices=["ag", "rs", "rs-pass", "rs-epilogue"], default="ag")
    ap.add_argument("--reps", type=int, default=2)
    args = ap.parse_args()
    from syncopate_b200 import _lib as L
    from syncopate_b200.computation.gemm import gemm_rs
    from syncopate_b200.computation.gemm.plan import rs_remote_signals
    from syncopate_b200.operators import AllGatherGemm, plan_reduce_scatter
    from syncopate_b200.runtime import EmulatedWorld

    W, dt = 8, torch.bfloat16
    ew = EmulatedWorld(W)
    if args.op == "ag":
        rows, K, N = 1024, 8192, 28672 // W
        ops = [AllGatherGemm(c, rows, K, N, dt, comm="sm", timeout_ns=2_000_000_000) for c in ew.contexts]
        shards = [seeded(1000 + r, (rows, K), 1.0).cuda() for r in range(W)]
        for r, op in enumerate(ops):
            op.shard.copy_(shards[r])
        b = seeded(5000, (N, K), 0.02).cuda()
        for _ in range(args.reps):
            c = ops[0](b)
        torch.cuda.synchronize()
        ops[0].ctx.check()
        full = torch.cat(shards, 0)
        assert torch.equal(ops[0].a.local, full)
        err = max(rel(c[r0:r0 + 2048], full[r0:r0 + 2048].float() @ b.float().t()) for r0 in range(0, W * rows, 2048))
        print(f"ag ok: relative Frobenius {err:.2e}")
    else:
        M, N, Kl = 8192, 8192, 28672 // W
        slab = M // W
        _gen, info, low = plan_reduce_scatter(W, M, N, dt, "direct")
        src, dst = low[0]["src"], low[0]["dst"]
        rsig = rs_remote_signals(info, 0, src)
        cols = (src.gen_block_offset_lists(), src.gen_block_shape_lists(), src.gen_signal_lists(),
                src.gen_target_rank_list(), src.gen_dst_offset_lists())
        whole = args.op != "rs"   # the own slab too: its flags are pre-set and the staged slabs hold zeros
        sel = [i for i, t in enumerate(cols[3]) if whole or (t >= 0 and t != 0)]
        sched = tuple([col[i] for i in sel] for col in cols)
        a, b = seeded(2000, (M, Kl), 1.0).cuda(), seeded(3000, (N, Kl), 0.02).cuda()
        stages = [torch.zeros(2, W, slab, N, dtype=dt, device="cuda") for _ in range(W)]
        flags = [torch.full((max(info.recv_signal_num, 1),), (1 << 40) if whole else 0, dtype=torch.int64, device="cuda")
                 for _ in range(W)]
        out = torch.zeros(slab, N, dtype=dt, device="cuda")
        counters = torch.zeros(130, dtype=torch.int32, device="cuda")
        status = torch.zeros(4, dtype=torch.int32, device="cuda")
        for epoch in range(1, args.reps + 1):
            gemm_rs(a, b, out, sched, dst, [rsig[i] for i in sel], L.Symm.of(0, [x.data_ptr() for x in stages]),
                    L.Symm.of(0, [x.data_ptr() for x in flags]), counters, epoch=epoch, timeout_ns=2_000_000_000,
                    status=status, reduce_pass=args.op == "rs-pass")
        torch.cuda.synchronize()
        assert status.tolist() == [0, 0, 0, 0]
        err = 0.0
        for t in range(1, W):  # rank 0's partial rows of slab t sit in slot 0 of rank t's staging half
            ref = a[t * slab:(t + 1) * slab].float() @ b.float().t()
            err = max(err, rel(stages[t][args.reps & 1, 0], ref))
        print(f"rs ok: relative Frobenius of the staged slabs {err:.2e}")
        assert err < 1e-2
        if whole:
            own = rel(out, a[:slab].float() @ b.float().t())
            print(f"own slab (own partial sum + zeros): relative Frobenius {own:.2e}")
            assert own < 1e-2


if __name__ == "__main__":
    main()
