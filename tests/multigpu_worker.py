"""Multi-process worker for the multi-GPU tests: run under torchrun with one rank per GPU.
Checks the fused operators over real peer-mapped memory against a gather-then-operate reference
computed with torch.distributed (test plumbing only)."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")

from syncopate_b200.operators import (  # noqa: E402
    AllGatherGemm,
    AllToAllGemm,
    ContextParallelAttention,
    GemmAllToAllGemm,
    GemmAllReduce,
    GemmReduceScatter,
    UlyssesAttention,
)
from syncopate_b200.runtime import init_from_env  # noqa: E402

TOL = 1e-2


def seeded(seed, shape, scale, dtype, device):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g, dtype=torch.float32) * scale).to(dtype).to(device)


def rel(x, ref):
    return ((x.float() - ref.float()).norm() / ref.float().norm()).item()


def main():
    rank, world, ctx = init_from_env()
    dev = ctx.device
    dt = torch.bfloat16
    failures = []

    def tile_ok(x, ref):
        """relative Frobenius error of the whole output and of its worst 128 x 256 tile"""
        xf, rf = x.float(), ref.float()
        M_, N_ = rf.shape
        pm, pn = (-M_) % 128, (-N_) % 256
        xp = torch.nn.functional.pad(xf, (0, pn, 0, pm))
        rp = torch.nn.functional.pad(rf, (0, pn, 0, pm))
        gm, gn = xp.shape[0] // 128, xp.shape[1] // 256
        d = (xp - rp).reshape(gm, 128, gn, 256).permute(0, 2, 1, 3).reshape(gm, gn, -1)
        r = rp.reshape(gm, 128, gn, 256).permute(0, 2, 1, 3).reshape(gm, gn, -1)
        return rel(x, ref), (d.norm(dim=-1) / r.norm(dim=-1).clamp_min(1e-30)).max().item()

    for kind, comm, rows, K, N, split, lock in (
            ("swizzle", "sm", 256, 512, 512, 1, True), ("ring", "sm", 128, 256, 512, 1, True),
            ("swizzle", "ce", 256, 512, 512, 1, True), ("swizzle", "sm", 512, 512, 512, 2, True),
            ("swizzle", "ce", 512, 256, 768, 4, "pairwise"),
            ("swizzle", "sm", 1024, 8192, 28672 // world, 1, True),
            ("swizzle", "sm", 1024, 8192, 28672 // world, 2, True),
            ("swizzle", "ce", 1024, 8192, 28672 // world, 2, True),
            ("swizzle", "ce", 1024, 8192, 28672 // world, 2, "pairwise")):
        op = AllGatherGemm(ctx, rows, K, N, dt, plan=kind, comm=comm, timeout_ns=2_000_000_000, chunk_split=split,
                           lockstep=lock)
        shards = [seeded(1000 + r, (rows, K), 1.0, dt, dev) for r in range(world)]
        b = seeded(5000 + rank, (N, K), 0.02, dt, dev)
        full = torch.cat(shards, 0)
        ref = full.float() @ b.float().t()
        for it in range(3):
            op.a.local.fill_(float("nan"))
            op.shard.copy_(shards[rank])
            torch.cuda.synchronize()
            ctx.barrier()
            c = op(b)
            ctx.check()
            e, et = tile_ok(c, ref)
            same = torch.equal(op.a.local, full)
            if not (e < TOL and et < TOL and same):
                failures.append(f"ag_gemm {kind}/{comm}/split{split} rows={rows} it={it} rank={rank}: relerr={e:.3e} "
                                f"tile={et:.3e} gathered_ok={same}")
            ctx.barrier()  # nobody may overwrite its shard while a peer still pulls it
            torch.cuda.synchronize()
        del op, ref

    # the shard is rewritten before every call and nothing but the operator synchronises the ranks
    # (leading barrier of every call + sync_after): each call must see the peers' new shards
    for comm in ("sm", "ce"):
        rows, K, N = 256, 512, 512
        op = AllGatherGemm(ctx, rows, K, N, dt, comm=comm, timeout_ns=2_000_000_000, sync_after=True)
        b = seeded(5100 + rank, (N, K), 0.02, dt, dev)
        for it in range(6):
            shards = [seeded(1200 + 10 * it + r, (rows, K), 1.0, dt, dev) for r in range(world)]
            op.shard.copy_(shards[rank])
            c = op(b)
            full = torch.cat(shards, 0)
            ctx.check()
            e = rel(c, full.float() @ b.float().t())
            same = torch.equal(op.a.local, full)
            if not (e < TOL and same):
                failures.append(f"ag_gemm rewrite-loop {comm} it={it} rank={rank}: relerr={e:.3e} gathered_ok={same}")
        del op

    # comm "sm": the epilogue pushes tiles to the peers; "ce": local slabs moved by copy engines
    for kind, M, N, Kl, comm, split, red in (
            ("direct", 256 * world, 512, 256, "sm", 1, "epilogue"), ("a2a", 128 * world, 1024, 512, "sm", 1, "epilogue"),
            ("direct", 8192, 8192, 28672 // world, "sm", 1, "epilogue"),
            ("direct", 256 * world, 512, 256, "ce", 1, "epilogue"), ("a2a", 128 * world, 1024, 512, "ce", 1, "pass"),
            ("direct", 512 * world, 512, 256, "sm", 2, "pass"), ("direct", 512 * world, 512, 256, "ce", 2, "epilogue"),
            ("direct", 8192, 8192, 28672 // world, "sm", 2, "epilogue"),
            ("direct", 8192, 8192, 28672 // world, "ce", 2, "pass"), ("direct", 8192, 8192, 28672 // world, "ce", 1, "pass")):
        if split > 1 and (M // world) % (split * 128):
            continue
        op = GemmReduceScatter(ctx, M, N, dt, plan=kind, timeout_ns=2_000_000_000, comm=comm, chunk_split=split,
                               reduce=red)
        a = seeded(2000 + rank, (M, Kl), 1.0, dt, dev)
        b = seeded(3000 + rank, (N, Kl), 0.02, dt, dev)
        part = a.float() @ b.float().t()
        dist.all_reduce(part)
        ref = part[rank * op.slab : (rank + 1) * op.slab]
        for it in range(3):
            out = op(a, b)
            ctx.check()
            e, et = tile_ok(out, ref)
            if not (e < TOL and et < TOL):
                failures.append(f"gemm_rs {kind}/{comm}/split{split}/{red} M={M} it={it} rank={rank}: relerr={e:.3e} tile={et:.3e}")
        del op, part, ref

    # ---- the same operator called back to back (no host synchronisation between the calls): a rank may
    # be one call ahead of a peer; both reduce modes, one and two copy streams
    M, N, Kl = 8192, 8192, 28672 // world
    a = seeded(2000 + rank, (M, Kl), 1.0, dt, dev)
    b = seeded(3000 + rank, (N, Kl), 0.02, dt, dev)
    part = a.float() @ b.float().t()
    dist.all_reduce(part)
    ref = part[rank * (M // world) : (rank + 1) * (M // world)].clone()
    del part
    for red, streams, comm in (("epilogue", 2, "ce"), ("pass", 2, "ce"), ("pass", 1, "ce"), ("pass", 1, "sm")):
        op = GemmReduceScatter(ctx, M, N, dt, plan="direct", timeout_ns=2_000_000_000, comm=comm, copy_streams=streams,
                               reduce=red)
        outs = [torch.empty(M // world, N, dtype=dt, device=dev) for _ in range(2)]
        for it in range(12):
            op(a, b, outs[it & 1])
        ctx.check()
        for o in outs:
            e, et = tile_ok(o, ref)
            if not (e < TOL and et < TOL):
                failures.append(f"gemm_rs back to back {comm}/{red}/{streams} streams rank={rank}: relerr={e:.3e} tile={et:.3e}")
        del op, outs
    del ref

    # ---- GEMM + all-reduce: reduce-scatter in the kernel, reduced rows all-gathered by copy engines
    for M, N, Kl, splits, pieces, comm, red in (
            (512 * world, 512, 256, 1, 1, "ce", "epilogue"), (1024 * world, 512, 256, 2, 2, "ce", "pass"),
            (512 * world, 768, 128, 2, 1, "sm", "epilogue"), (8192, 8192, 28672 // world, 4, 1, "ce", "epilogue"),
            (8192, 8192, 28672 // world, 1, 1, "ce", "pass")):
        if (M // splits // world) % (pieces * 128):
            continue
        op = GemmAllReduce(ctx, M, N, dt, num_splits=splits, chunk_split=pieces, comm=comm, timeout_ns=2_000_000_000,
                           sync_after=True, reduce=red)
        a = seeded(2500 + rank, (M, Kl), 1.0, dt, dev)
        b = seeded(3500 + rank, (N, Kl), 0.02, dt, dev)
        ref = a.float() @ b.float().t()
        dist.all_reduce(ref)
        for it in range(3):
            op.out.local.fill_(float("nan"))
            torch.cuda.synchronize()
            ctx.barrier()
            out = op(a, b)
            ctx.check()
            e, et = tile_ok(out, ref)
            if not (e < TOL and et < TOL):
                failures.append(f"gemm_ar M={M} splits={splits} pieces={pieces} {comm} {red} it={it} rank={rank}: "
                                f"relerr={e:.3e} tile={et:.3e}")
        del op, ref

    # ---- all-to-all + GEMM: SM copies on a few SMs beside the K-gated consumer GEMM on the others
    for B, S, H, D, N in ((1, 256 * world, 2 * world, 128, 512), (2, 512 * world, 8 * world, 128, 1024)):
        op = AllToAllGemm(ctx, B, S, H, D, N, dt, num_copy_sms=16, timeout_ns=2_000_000_000, sync_after=True)
        x = seeded(4000 + rank, (B, S, H // world, D), 1.0, dt, dev)
        w = seeded(4100, (N, H * D), 0.02, dt, dev)
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x)
        Sl = S // world
        a_ref = torch.cat(parts, dim=2)[:, rank * Sl:(rank + 1) * Sl].reshape(B * Sl, H * D)
        ref = a_ref.float() @ w.float().t()
        for it in range(3):
            op.src.copy_(x)
            out = op(w)
            ctx.check()
            e, et = tile_ok(out, ref)
            same = torch.equal(op.a, a_ref)
            if not (e < TOL and et < TOL and same):
                failures.append(f"a2a_gemm S={S} it={it} rank={rank}: relerr={e:.3e} tile={et:.3e} resharded_ok={same}")
        del op, ref

    # ---- GEMM + all-to-all + GEMM (tensor-parallel MLP without a reduction)
    for M, hidden, ffn in ((256 * world, 512, 256 * world), (1024 * world, 1024, 512 * world)):
        op = GemmAllToAllGemm(ctx, M, hidden, ffn, dt, num_copy_sms=16, timeout_ns=2_000_000_000)
        x = seeded(4200, (M, hidden), 0.1, dt, dev)
        w1 = seeded(4300 + rank, (ffn // world, hidden), 0.1, dt, dev)
        w2 = seeded(4400, (hidden, ffn), 0.1, dt, dev)
        w1s = [torch.empty_like(w1) for _ in range(world)]
        dist.all_gather(w1s, w1)
        rows = slice(rank * (M // world), (rank + 1) * (M // world))
        mid = (x[rows].float() @ torch.cat(w1s, 0).float().t()).to(dt)
        ref = mid.float() @ w2.float().t()
        for it in range(3):
            out = op(x, w1, w2)
            ctx.check()
            e, et = tile_ok(out, ref)
            if not (e < TOL and et < TOL):
                failures.append(f"gemm_a2a_gemm M={M} it={it} rank={rank}: relerr={e:.3e} tile={et:.3e}")
            ctx.barrier()   # the peers' pushes of the next call land in this rank's buffers
            torch.cuda.synchronize()
        del op, ref

    # ---- attention operators (reference: gather with torch.distributed, dense fp32 attention per head)
    def dense(q, k, v, causal, q_pos=None, k_pos=None):
        Hq, Hkv = q.shape[0], k.shape[0]
        out = torch.empty(q.shape, dtype=torch.float32, device=q.device)
        for h in range(Hq):
            s = (q[h].float() @ k[h // (Hq // Hkv)].float().t()) * (q.shape[-1] ** -0.5)
            if causal:
                qp = torch.arange(q.shape[1], device=q.device) if q_pos is None else q_pos
                kp = torch.arange(k.shape[1], device=q.device) if k_pos is None else k_pos
                s = s.masked_fill(kp[None, :] > qp[:, None], float("-inf"))
            out[h] = torch.nan_to_num(torch.softmax(s, -1)) @ v[h // (Hq // Hkv)].float()
        return out

    B, H, Sl = 1, 2 * world, 256
    qkv = seeded(7000 + rank, (3, B, H, Sl, 128), 1.0, dt, dev)
    gathered = [torch.empty_like(qkv) for _ in range(world)]
    dist.all_gather(gathered, qkv)
    full = torch.cat(gathered, dim=3)  # [3, B, H, S, D]
    ref = dense(full[0, 0], full[1, 0], full[2, 0], True)[:, rank * Sl : (rank + 1) * Sl].permute(1, 0, 2)
    for overlap in (True, False):  # the kernel sends finished tiles itself / a copy kernel follows it
        op = UlyssesAttention(ctx, B, H, Sl, 128, dt, causal=True, timeout_ns=2_000_000_000, overlap_out=overlap)
        assert (op.push is not None) == overlap
        for it in range(3):
            op.qkv_src.local.copy_(qkv)
            op.out.local.fill_(float("nan"))
            torch.cuda.synchronize()
            ctx.barrier()
            out = op()
            ctx.check()
            e = (out[0].float() - ref).abs().max().item()
            if not e < 2e-2:
                failures.append(f"ulysses overlap_out={overlap} it={it} rank={rank}: maxabs={e:.3e}")
            ctx.barrier()
            torch.cuda.synchronize()
        del op

    for plan in ("swizzle", "ring", "double_ring"):
        Hq, Hkv = 8, 2
        op = ContextParallelAttention(ctx, 1, Hq, Hkv, Sl, 128, dt, causal=True, zigzag=True, plan=plan,
                                      timeout_ns=2_000_000_000)
        kv = seeded(8000 + rank, (2, 1, Hkv, Sl, 128), 1.0, dt, dev)
        q = seeded(9000 + rank, (1, Hq, Sl, 128), 1.0, dt, dev)
        gathered = [torch.empty_like(kv) for _ in range(world)]
        dist.all_gather(gathered, kv)
        full = torch.cat(gathered, dim=3)
        steps = torch.arange(128, device=dev)
        q_pos = (op.q_pos[:, None] + steps[None, :]).reshape(-1)
        k_pos = (op.kv_pos[:, None] + steps[None, :]).reshape(-1)
        ref = dense(q[0], full[0, 0], full[1, 0], True, q_pos, k_pos)
        for it in range(2):
            op.kv.local.fill_(float("nan"))
            op.kv_shard.copy_(kv)
            torch.cuda.synchronize()
            ctx.barrier()
            out = op(q)
            ctx.check()
            e = (out[0].float() - ref).abs().max().item()
            same = torch.equal(op.kv.local, full)
            if not (e < 2e-2 and same):
                failures.append(f"cp {plan} it={it} rank={rank}: maxabs={e:.3e} gathered_ok={same}")
            ctx.barrier()
            torch.cuda.synchronize()

    torch.cuda.synchronize()
    flag = torch.tensor([len(failures)], device=dev)
    dist.all_reduce(flag)
    for f in failures:
        print("FAIL", f, flush=True)
    if rank == 0:
        print("MULTIGPU_OK" if flag.item() == 0 else f"MULTIGPU_FAILED {flag.item()}", flush=True)
    ctx.close()
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
