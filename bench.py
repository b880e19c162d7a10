"""Benchmark of the fused operators: ``python bench.py --gpus N --steps K --warmup W``.

Workload (the one the headline metric is quoted on): all-gather + GEMM, bf16, per-rank A shard
[1024, 8192] gathered to [1024 * TP, 8192], per-rank B [28672 / TP, 8192] (K-major), fp32
accumulation, bf16 output; TP = N for N > 1 (one process per GPU under torchrun, peers' shards
pulled over NVLink by the kernel's comm warps), and at N = 1 the TP = 8 per-rank shapes with the
eight chunk waves gated by pre-set flags (compute only).  481 GFLOP per rank at every N.

One JSON line on rank 0: whole-job TFLOP/s (``value``), the same through the public API with host
buffers (``e2e``), the tensor roofline of the GEMM kernel, the CPU oracle timed on the host cores,
and GEMM + reduce-scatter on the paired shape under ``other_ops``.  ``--impl reference`` times the
reference's definition of the operator (PyTorch CPU emulation of the plan) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

ROWS, K_DIM, N_TOTAL = 1024, 8192, 28672
RS_M, RS_N, RS_K_TOTAL = 8192, 8192, 28672


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained"),
                "hbm_gbs": d.get("hbm_gbs"), "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        clocks, max_clock, reasons = [], None, set()
        inside = [r for (t, r) in self.rows if t0 - 0.05 <= t <= t1 + 0.15] or [r for (_t, r) in self.rows]
        for row in inside:
            parts = [p.strip() for p in row.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                max_clock = float(parts[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(clocks)}


def seeded(seed, shape, scale, dtype):
    import torch

    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g, dtype=torch.float32) * scale).to(dtype)


# --------------------------------------------------------------------------- reference / CPU arm
def cpu_ag_gemm_sample(tp: int, budget_s: float = 12.0):
    """Times the oracle's chunk-ordered all-gather + GEMM of ONE rank at the benchmark shapes on all
    host cores.  Returns (TFLOP/s, cores, description)."""
    import torch

    from oracle import emulate as E

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    n_local = N_TOTAL // tp
    dt = torch.bfloat16
    shards = [seeded(1000 + r, (ROWS, K_DIM), 1.0, dt) for r in range(tp)]
    b = seeded(5000, (n_local, K_DIM), 0.02, dt)
    sched = E.swizzle_pull_schedule(tp, 0, ROWS, K_DIM)
    flop = 2.0 * ROWS * tp * K_DIM * n_local
    E.ag_gemm({"offsets": sched["offsets"][:1], "shapes": sched["shapes"][:1]}, shards, b)  # warm the thread pool
    times = []
    t_all = time.perf_counter()
    while len(times) < 3 and (time.perf_counter() - t_all) < budget_s:
        t0 = time.perf_counter()
        E.ag_gemm(sched, shards, b)
        times.append(time.perf_counter() - t0)
    best = min(times)
    return flop / best / 1e12, cores, (f"one rank's full operator (gather {tp} x [{ROWS},{K_DIM}] + GEMM with "
                                       f"B [{n_local},{K_DIM}], {flop/1e9:.0f} GFLOP), best of {len(times)}"), times


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tp = args.gpus if args.gpus > 1 else 8
    import torch

    from oracle import emulate as E

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    n_local = N_TOTAL // tp
    dt = torch.bfloat16
    shards = [seeded(1000 + r, (ROWS, K_DIM), 1.0, dt) for r in range(tp)]
    b = seeded(5000, (n_local, K_DIM), 0.02, dt)
    sched = E.swizzle_pull_schedule(tp, 0, ROWS, K_DIM)
    flop = 2.0 * ROWS * tp * K_DIM * n_local
    # each step = one rank's full operator (all ranks do the same amount of work)
    for _ in range(max(args.warmup, 1)):
        E.ag_gemm(sched, shards, b)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        E.ag_gemm(sched, shards, b)
    dt_s = (time.perf_counter() - t0) / args.steps
    per_rank = flop / dt_s / 1e12
    # the host cores are shared by all ranks of the box: the whole job proceeds at this one rate
    value = per_rank
    line = {
        "impl": "reference", "metric": "ag_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt_s * 1e3 * max(args.gpus, 1),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": f"each step = one rank's operator ({flop/1e9:.0f} GFLOP) on all host cores; "
                                   f"the {max(args.gpus,1)} ranks of the job share those cores"},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference GPU kernels are Hopper-only Triton/NVSHMEM code that cannot be installed here; this arm "
                "is the reference's definition of the operator (PyTorch CPU emulation of the lowered plan)",
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus: int):
    tp = n_gpus if n_gpus > 1 else 8
    return {
        "workload": f"cfg1 AG+GEMM bf16 TP={tp}: A shard [{ROWS},{K_DIM}] -> [{ROWS*tp},{K_DIM}], "
                    f"B [{N_TOTAL//tp},{K_DIM}] K-major, C [{ROWS*tp},{N_TOTAL//tp}]"
                    + (" (1 GPU: compute only, chunk flags pre-set)" if n_gpus == 1 else ""),
        "tp": tp, "flop_per_rank": 2.0 * ROWS * tp * K_DIM * (N_TOTAL // tp),
        "l2": "inputs+outputs 250 MB per step exceed the 126 MB L2; no explicit flush",
        "plan": "build_all_gather_plan_1d_swizzle pull",
        "comm": "copy-engine program on a side stream + flag-gated tcgen05 GEMM (--comm ce) or in-kernel comm warps (--comm sm)",
    }


# --------------------------------------------------------------------------- own arm
def run_own_arm(args):
    import torch
    import torch.distributed as dist

    from syncopate_b200.operators import AllGatherGemm, GemmReduceScatter
    from syncopate_b200.runtime import init_from_env

    rank, world, ctx = init_from_env()
    assert world == max(args.gpus, 1), f"--gpus {args.gpus} but WORLD_SIZE={world}"
    dev = ctx.device
    dt = torch.bfloat16
    tp = world if world > 1 else 8
    n_local = N_TOTAL // tp
    M = ROWS * tp
    flop = 2.0 * M * K_DIM * n_local
    peaks = measured_peaks()

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---------------- AG + GEMM, inputs resident
    b = seeded(5000 + rank, (n_local, K_DIM), 0.02, dt).to(dev)
    c = torch.empty(M, n_local, dtype=dt, device=dev)
    if world > 1:
        op = AllGatherGemm(ctx, ROWS, K_DIM, n_local, dt, plan="swizzle", comm=args.comm)
        op.shard.copy_(seeded(1000 + rank, (ROWS, K_DIM), 1.0, dt).to(dev))
        step = lambda: op(b, c)
        a_host_shape = (ROWS, K_DIM)
    else:
        from syncopate_b200.computation.gemm import gemm
        from syncopate_b200.operators import plan_all_gather

        a_full = torch.cat([seeded(1000 + r, (ROWS, K_DIM), 1.0, dt) for r in range(tp)], 0).to(dev)
        a_sched = plan_all_gather(tp, ROWS, K_DIM, dt, "swizzle")[2][0]["a"]  # rank 0 of the TP=8 plan
        wave_offsets = [[o[0], 0] for o in a_sched.gen_block_offset_lists()]
        wave_sizes = [[s[0], n_local] for s in a_sched.gen_block_shape_lists()]
        flags = torch.ones(tp, dtype=torch.int64, device=dev)
        step = lambda: gemm(a_full, b, c, cur_wave_sizes=wave_sizes, wave_offsets=wave_offsets,
                            signal_ptr=flags, signal_offsets=a_sched.gen_signal_lists(), status=ctx.status)
        a_host_shape = (M, K_DIM)

    for _ in range(max(args.warmup, 3)):
        step()
    sync_all()
    sampler = ClockSampler(ctx.device_index)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall0 = time.time()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    sync_all()
    t_wall1 = time.time()
    ms = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    ctx.check()
    per_gpu = flop / (ms * 1e-3) / 1e12
    value = per_gpu * world

    # ---------------- the same GEMM with every chunk already resident (flags pre-set, no transfers),
    # timed while all ranks compute: the non-overlapped share of the fused step is the difference
    compute_only_ms = None
    if world > 1:
        from syncopate_b200.computation.gemm import gemm as _plain_gemm

        ones = torch.full((max(op.info.recv_signal_num, 1),), 1 << 40, dtype=torch.int64, device=dev)
        offs = [[o[0], 0] for o in op.schedule.gen_block_offset_lists()]
        sizes = [[s_[0], n_local] for s_ in op.schedule.gen_block_shape_lists()]
        sigs = op.schedule.gen_signal_lists()
        co_step = lambda: _plain_gemm(op.a.local, b, c, cur_wave_sizes=sizes, wave_offsets=offs, signal_ptr=ones,
                                      signal_offsets=sigs, status=ctx.status)
        for _ in range(3):
            co_step()
        sync_all()
        e0.record()
        for _ in range(args.steps):
            co_step()
        e1.record()
        sync_all()
        compute_only_ms = max_over_ranks(e0.elapsed_time(e1) / args.steps)

    # ---------------- e2e: host buffers in, host result out, through the operator API
    a_host = seeded(1000 + rank, (ROWS, K_DIM), 1.0, dt).pin_memory() if world > 1 else a_full.cpu().pin_memory()
    c_host = torch.empty(M, n_local, dtype=dt).pin_memory()

    def e2e_step():
        op.shard.copy_(a_host, non_blocking=True)
        # peers may only pull the new shard once it has landed: the operator's own device-side
        # barrier at the start of the call takes care of that
        step()
        c_host.copy_(c, non_blocking=True)
        ctx.barrier()  # nobody overwrites its shard while a peer still pulls it

    e2e_steps = max(3, min(args.steps, 10))
    if world > 1:
        e2e_path = "pinned host A -> device shard, device barrier, fused op, C -> pinned host"
        for _ in range(2):
            e2e_step()
        sync_all()
        e0.record()
        for _ in range(e2e_steps):
            e2e_step()
        e1.record()
        sync_all()
    else:
        # One GPU: the same three stages per step (input copy, GEMM call, result copy), each step's
        # copies inside the timed region, but on three streams over two sets of device buffers, so
        # that step i + 1's input copy runs while step i computes and returns its result.
        e2e_path = ("pinned host A -> device, GEMM call, C -> pinned host; three streams and two device buffer sets, "
                    "so consecutive steps overlap; every step's copies are inside the timed region")
        cur = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        a_dev = [a_full, torch.empty_like(a_full)]
        c_dev = [c, torch.empty_like(c)]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_comp = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]
        sig_offsets = a_sched.gen_signal_lists()

        def e2e_run(n):
            for i in range(n):
                k = i & 1
                s_in.wait_event(ev_comp[k])  # the GEMM that last read this input buffer
                with torch.cuda.stream(s_in):
                    a_dev[k].copy_(a_host, non_blocking=True)
                    ev_in[k].record(s_in)
                cur.wait_event(ev_in[k])
                cur.wait_event(ev_out[k])    # the result copy that last read this output buffer
                gemm(a_dev[k], b, c_dev[k], cur_wave_sizes=wave_sizes, wave_offsets=wave_offsets, signal_ptr=flags,
                     signal_offsets=sig_offsets, status=ctx.status)
                ev_comp[k].record(cur)
                s_out.wait_event(ev_comp[k])
                with torch.cuda.stream(s_out):
                    c_host.copy_(c_dev[k], non_blocking=True)
                    ev_out[k].record(s_out)
            cur.wait_stream(s_out)

        e2e_run(2)
        sync_all()
        e0.record()
        e2e_run(e2e_steps)
        e1.record()
        sync_all()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1) / e2e_steps)
    ctx.check()
    e2e_value = flop / (e2e_ms * 1e-3) / 1e12 * world
    h2d = a_host.numel() * 2
    d2h = c_host.numel() * 2

    # ---------------- GEMM + reduce-scatter on the paired shape (reported, not the headline)
    rs_k = RS_K_TOTAL // tp
    rs = GemmReduceScatter(ctx, RS_M, RS_N, dt, plan="direct") if world > 1 else None
    ra = seeded(2000 + rank, (RS_M, rs_k), 1.0, dt).to(dev)
    rb = seeded(3000 + rank, (RS_N, rs_k), 0.02, dt).to(dev)
    if world > 1:
        rout = torch.empty(RS_M // world, RS_N, dtype=dt, device=dev)
        rs_step = lambda: rs(ra, rb, rout)
    else:
        from syncopate_b200.computation.gemm import gemm as _gemm

        rout = torch.empty(RS_M, RS_N, dtype=dt, device=dev)
        rs_step = lambda: _gemm(ra, rb, rout, status=ctx.status)
    for _ in range(3):
        rs_step()
    sync_all()
    e0.record()
    for _ in range(args.steps):
        rs_step()
    e1.record()
    sync_all()
    rs_ms = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    ctx.check()
    rs_flop = 2.0 * RS_M * RS_N * rs_k
    rs_per_gpu = rs_flop / (rs_ms * 1e-3) / 1e12
    rs_compute_only_ms = None
    if world > 1:
        rfull = torch.empty(RS_M, RS_N, dtype=dt, device=dev)
        for _ in range(3):
            _plain_gemm(ra, rb, rfull, status=ctx.status)
        sync_all()
        e0.record()
        for _ in range(args.steps):
            _plain_gemm(ra, rb, rfull, status=ctx.status)
        e1.record()
        sync_all()
        rs_compute_only_ms = max_over_ranks(e0.elapsed_time(e1) / args.steps)
        del rfull

    # ---------------- attention operators at the benchmark shapes (reported, not the headline)
    attn_results = {}
    if not args.skip_attention:
        from syncopate_b200.operators import ContextParallelAttention, UlyssesAttention
        from syncopate_b200.runtime import EmulatedWorld

        def time_op(fn, steps):
            for _ in range(2):
                fn()
            sync_all()
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            sync_all()
            t = max_over_ranks(e0.elapsed_time(e1) / steps)
            ctx.check()
            return t

        a_steps = max(3, min(args.steps, 10))
        # Ulysses: total sequence 32768, 32 heads, D 128, causal; per rank 4 heads over the full sequence
        if world > 1:
            uly = UlyssesAttention(ctx, 1, 32, 32768 // world, 128, dt, causal=True)
            uly.qkv_src.local.copy_(seeded(7000 + rank, (3, 1, 32, 32768 // world, 128), 1.0, dt).to(dev))
            sync_all()
            u_ms = time_op(lambda: uly(), a_steps)
            heads_local = 32 // world
        else:
            from syncopate_b200.computation.attn import AttentionState, attention_forward

            heads_local = 4
            uq = seeded(7000, (3, 1, heads_local, 32768, 128), 1.0, dt).to(dev)
            uo = torch.empty(1, heads_local, 32768, 128, dtype=dt, device=dev)
            ust = AttentionState(1, heads_local, 32768, dev)
            u_ms = time_op(lambda: attention_forward(uq[0], uq[1], uq[2], 128 ** -0.5, uo, causal=True, state=ust,
                                                     status=ctx.status), a_steps)
        u_flop = 4.0 * 32768 * 32768 * 128 * heads_local / 2
        attn_results["ulysses_attn"] = {
            "workload": f"cfg3 Ulysses all2all+attention+all2all bf16: S=32768, 32 heads, D=128, causal; {heads_local} heads per rank"
                        + (" (1 GPU: attention only)" if world == 1 else ""),
            "ms_per_step": u_ms, "per_gpu_tflops_causal": u_flop / (u_ms * 1e-3) / 1e12}
        # context parallel: total sequence 65536, 64 Q heads / 8 KV heads, causal zigzag
        cp_world = world if world > 1 else 8
        s_local = 65536 // cp_world
        if world > 1:
            cp = ContextParallelAttention(ctx, 1, 64, 8, s_local, 128, dt, causal=True, zigzag=True, plan="swizzle")
            cp.kv_shard.copy_(seeded(8000 + rank, (2, 1, 8, s_local, 128), 1.0, dt).to(dev))
        else:
            ew = EmulatedWorld(cp_world)
            cp = ContextParallelAttention(ew.contexts[0], 1, 64, 8, s_local, 128, dt, causal=True, zigzag=True)
            cp.kv.local.copy_(seeded(8000, (2, 1, 8, 65536, 128), 1.0, dt).to(dev))
            cp.ops, cp.comm = [], None  # one GPU: K/V already gathered, flags pre-set
            cp.flags.local.fill_(1 << 40)
        cq = seeded(9000 + rank, (1, 64, s_local, 128), 1.0, dt).to(dev)
        co = torch.empty_like(cq)
        sync_all()
        c_ms = time_op(lambda: cp(cq, co), a_steps)
        if world == 1:
            if cp.ctx.status.tolist()[0] != 0:
                raise RuntimeError(f"context-parallel attention status {cp.ctx.status.tolist()}")
        c_flop = 4.0 * 65536 * 65536 * 128 * 64 / cp_world / 2
        attn_results["cp_attn"] = {
            "workload": f"cfg4 context-parallel all-gather-KV attention bf16: S=65536 ({s_local} Q tokens per rank), "
                        "64 Q / 8 KV heads, D=128, causal zigzag" + (" (1 GPU: rank 0 of 8, K/V resident)" if world == 1 else ""),
            "ms_per_step": c_ms, "per_gpu_tflops_causal": c_flop / (c_ms * 1e-3) / 1e12}

    line = None
    if rank == 0:
        cpu_val, cores, sample, _ = cpu_ag_gemm_sample(tp) if world == 1 else (None, None, None, None)
        peak = peaks["bf16_tflops"]
        nvlink_bytes = (world - 1) * ROWS * K_DIM * 2 if world > 1 else 0
        t_roof_ms = max(flop / (peak * 1e12), nvlink_bytes / 770e9) * 1e3
        line = {
            "metric": "ag_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(world),
            "per_gpu_tflops": per_gpu,
            "compute_only_ms": compute_only_ms,
            "non_overlapped_ms": (ms - compute_only_ms) if compute_only_ms is not None else 0.0,
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms,
                    "path": e2e_path},
            # one GEMM kernel per step; with more than one rank also the operator's lockstep barrier kernel
            "gpu_launches": args.steps * (2 if world > 1 else 1),
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s",
                         "frac": per_gpu / peak,
                         # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on this
                         # workload (ncu capture summarised in profiles/gemm2_kernel_bn256_cfg1_tp8_local.md)
                         "traffic": 610.7e6 if world == 1 else None,
                         "algorithmic_bytes": (M * K_DIM + n_local * K_DIM + M * n_local) * 2,
                         "peak_source": f"{peaks['source']} cuBLAS bf16 burst (MEASURED_PEAKS.json)",
                         "frac_of_sustained": per_gpu / peaks["bf16_tflops_sustained"] if peaks["bf16_tflops_sustained"] else None,
                         "frac_of_nominal_2250": per_gpu / 2250.0,
                         "fused_roofline_ms": t_roof_ms, "frac_of_fused_roofline": t_roof_ms / ms,
                         "nvlink_bytes_in_per_rank": nvlink_bytes},
            "other_ops": {
                "gemm_rs": {"workload": f"cfg2 GEMM+RS bf16 TP={tp}: A [{RS_M},{rs_k}], B [{RS_N},{rs_k}], out "
                                        f"[{RS_M // world if world > 1 else RS_M},{RS_N}]"
                                        + (" (1 GPU: GEMM only)" if world == 1 else ""),
                            "ms_per_step": rs_ms, "per_gpu_tflops": rs_per_gpu, "frac_of_peak": rs_per_gpu / peak,
                            "compute_only_ms": rs_compute_only_ms},
                **attn_results,
            },
        }
        if cpu_val is not None:
            line["cpu_baseline"] = {"value": cpu_val, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                    "sample": sample}
    ctx.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-attention", action="store_true", help="leave the attention operators out of other_ops")
    ap.add_argument("--comm", default="ce", choices=["sm", "ce"],
                    help="who moves the all-gather chunks: the kernel's comm warps (sm) or copy engines (ce)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_own_arm(args)


if __name__ == "__main__":
    main()
