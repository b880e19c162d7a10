"""Benchmark of the fused operators: ``python bench.py --gpus N --steps K --warmup W``.

Workload (the one the headline metric is quoted on): all-gather + GEMM, bf16, per-rank A shard
[1024, 8192] gathered to [1024 * TP, 8192], per-rank B [28672 / TP, 8192] (K-major), fp32
accumulation, bf16 output; TP = N for N > 1 (one process per GPU under torchrun, peers' shards
moved over NVLink while the flag-gated tcgen05 GEMM runs), and at N = 1 the TP = 8 per-rank shapes
with the eight chunk waves gated by pre-set flags (compute only).  481 GFLOP per rank at every N.

Timing: after the warm-up, ``--blocks`` blocks of exactly ``--steps`` steps each are timed with CUDA
events between barriers, the maximum over ranks is taken per block, and the MEDIAN block is
reported (minimum and maximum beside it), so that the figure rests on tens of milliseconds of
device time instead of one short burst.

One JSON line on rank 0: whole-job TFLOP/s (``value``), the same through the public API with host
buffers (``e2e``), the tensor roofline of the GEMM kernel with cuBLAS on the same shape as a
yardstick, the CPU oracle timed on the host cores, the other operators (GEMM + reduce-scatter,
Ulysses attention, context-parallel attention) under ``other_ops``, and - on every N - a ``parity``
block: each operator's result checked on the device against torch on the gathered inputs (outside
the timed regions; the process exits non-zero when one is out of tolerance).  ``--impl reference``
times the reference's definition of the operator (PyTorch CPU emulation of the plan) on the host cores.
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
NVLINK_GBS_NOMINAL = 900.0   # per direction per GPU: the figure the fused roofline is defined with
GEMM_TOL, ATTN_TOL = 1e-2, 2e-2


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained"),
                "hbm_gbs": d.get("hbm_gbs"), "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi (every 20 ms) for the whole run; only
    the samples whose time stamp falls inside a timed region are used."""

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
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self, windows):
        """``windows``: (t0, t1) wall-clock spans of the timed regions."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        clocks, max_clock, reasons = [], None, set()
        inside = [r for (t, r) in self.rows if any(t0 <= t <= t1 + 0.02 for t0, t1 in windows)]
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
                "reasons": sorted(reasons), "samples": len(clocks),
                "note": "nvidia-smi samples every 20 ms whose time stamp falls inside a timed region"}


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
    value = flop / dt_s / 1e12
    line = {
        "impl": "reference", "metric": "ag_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt_s * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.gpus, args.comm, args.chunk_split),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": f"each step = ONE rank's operator ({flop/1e9:.0f} GFLOP) on all host cores, measured; "
                                   f"the {max(args.gpus, 1)} ranks of the job would share those cores"},
        # what the whole job (every rank's operator, one after the other on the same cores) would take
        "whole_job_ms_per_step_extrapolated": dt_s * 1e3 * max(args.gpus, 1),
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference GPU kernels are Hopper-only Triton/NVSHMEM code that cannot be installed here; this arm "
                "is the reference's definition of the operator (PyTorch CPU emulation of the lowered plan)",
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus: int, comm, chunk_split):
    tp = n_gpus if n_gpus > 1 else 8
    cfg = {
        "workload": f"cfg1 AG+GEMM bf16 TP={tp}: A shard [{ROWS},{K_DIM}] -> [{ROWS*tp},{K_DIM}], "
                    f"B [{N_TOTAL//tp},{K_DIM}] K-major, C [{ROWS*tp},{N_TOTAL//tp}]"
                    + (" (1 GPU: compute only, chunk flags pre-set)" if n_gpus == 1 else ""),
        "tp": tp, "flop_per_rank": 2.0 * ROWS * tp * K_DIM * (N_TOTAL // tp),
        "l2": "inputs+outputs 250 MB per step exceed the 126 MB L2; no explicit flush",
        "plan": "build_all_gather_plan_1d_swizzle pull",
    }
    if n_gpus > 1 and comm is not None:
        cfg["comm"] = ("copy-engine program on side streams + flag-gated tcgen05 GEMM" if comm == "ce"
                       else "in-kernel comm warps of the tcgen05 GEMM")
        cfg["comm_mode"] = comm
        cfg["chunk_split"] = chunk_split
    return cfg


# --------------------------------------------------------------------------- parity helpers (device side)
def gemm_parity(c, ref):
    """(global relative Frobenius error, worst 128 x 256 tile's) of ``c`` against ``ref`` (fp32)."""
    import torch

    cf, rf = c.float(), ref.float()
    glob = ((cf - rf).norm() / rf.norm()).item()
    M, N = rf.shape
    tm, tn = 128, 256
    pm, pn = (-M) % tm, (-N) % tn
    if pm or pn:
        cf = torch.nn.functional.pad(cf, (0, pn, 0, pm))
        rf = torch.nn.functional.pad(rf, (0, pn, 0, pm))
    gm, gn = cf.shape[0] // tm, cf.shape[1] // tn
    d = (cf - rf).reshape(gm, tm, gn, tn).permute(0, 2, 1, 3).reshape(gm, gn, -1)
    r = rf.reshape(gm, tm, gn, tn).permute(0, 2, 1, 3).reshape(gm, gn, -1)
    return glob, (d.norm(dim=-1) / r.norm(dim=-1).clamp_min(1e-30)).max().item()


def matmul_blocks(a, b, rows=2048):
    """fp32 product of 16-bit ``a [M, K]`` and ``b [N, K]`` in row blocks (TF32 off)."""
    import torch

    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        bt = b.float().t().contiguous()
        for r0 in range(0, a.shape[0], rows):
            yield r0, a[r0:r0 + rows].float() @ bt
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def attn_rows_error(out_rows, q_rows, k_h, v_h, q_pos, k_pos):
    """max-abs error of some output rows of one head against fp32 dense causal attention."""
    import torch

    s = (q_rows.float() @ k_h.float().t()) * (q_rows.shape[-1] ** -0.5)
    s = s.masked_fill(k_pos[None, :] > q_pos[:, None], float("-inf"))
    ref = torch.softmax(s, dim=-1) @ v_h.float()
    return (out_rows.float() - ref).abs().max().item()


def sample_tiles(n_tiles, seed, extra=2):
    import torch

    g = torch.Generator().manual_seed(seed)
    picks = {0, n_tiles // 2, n_tiles - 1}
    picks.update(int(x) for x in torch.randint(0, n_tiles, (extra,), generator=g))
    return sorted(picks)


# --------------------------------------------------------------------------- own arm
def run_own_arm(args):
    import torch
    import torch.distributed as dist

    from syncopate_b200.computation.gemm import gemm
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
    steps, blocks = args.steps, max(args.blocks, 1)
    warmup = max(args.warmup, 3)
    windows = []       # wall-clock spans of the timed regions, for the clock samples
    launches = [0]     # kernels of this library launched inside the headline's timed region
    parity = {}

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(values):
        if world == 1:
            return list(values)
        t = torch.tensor(list(values), device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn, n_steps=None, n_blocks=None, n_warm=None):
        """Median (and min / max) over blocks of the per-step time, each block timed between
        barriers with CUDA events and reduced with max over ranks."""
        n_steps, n_blocks = n_steps or steps, n_blocks or blocks
        for _ in range(warmup if n_warm is None else n_warm):
            fn()
        per_block = []
        for _ in range(n_blocks):
            sync_all()
            t0 = time.time()
            e0.record()
            for _ in range(n_steps):
                fn()
            e1.record()
            sync_all()
            windows.append((t0, time.time()))
            per_block.append(e0.elapsed_time(e1) / n_steps)
        per_block = max_over_ranks(per_block)
        ctx.check()
        return {"ms": statistics.median(per_block), "ms_min": min(per_block), "ms_max": max(per_block),
                "blocks": n_blocks, "steps_per_block": n_steps}

    def capture_trace(operator, call, rows, signals):
        """Per-wave wait stamps of one call in steady state: four calls back to back without a
        synchronisation in between, the kernel's stamps switched on for the last one (a call made
        on an idle GPU would give its transfers a head start over the kernel).  Returns the rows and
        the kernel's duration (us)."""
        nw = len(rows)
        big = torch.iinfo(torch.int64).max
        tr = torch.zeros(2 + 3 * nw, dtype=torch.int64, device=dev)
        tr[0] = big
        tr[2::3] = big
        sync_all()
        for i in range(4):
            operator.trace = tr if i == 3 else None
            call()
        operator.trace = None
        torch.cuda.synchronize()
        t = tr.tolist()
        out = [{"wave": w, "rows": rows[w], "flag": signals[w],
                "wait_begin_us": (t[2 + 3 * w] - t[0]) / 1e3 if t[2 + 3 * w] != big else None,
                "wait_end_us": (t[3 + 3 * w] - t[0]) / 1e3 if t[3 + 3 * w] else None,
                "summed_wait_us": t[4 + 3 * w] / 1e3} for w in range(nw)]
        return out, (t[1] - t[0]) / 1e3

    sampler = ClockSampler(ctx.device_index)
    if rank == 0:
        sampler.start()

    # ---------------- AG + GEMM, inputs resident
    b = seeded(5000 + rank, (n_local, K_DIM), 0.02, dt).to(dev)
    c = torch.empty(M, n_local, dtype=dt, device=dev)
    shard_seed = lambda r: seeded(1000 + r, (ROWS, K_DIM), 1.0, dt)
    ag_lockstep = "pairwise" if (args.ag_lockstep == "pairwise" and args.comm == "ce" and args.ag_transfer == "pull") else True
    if world > 1:
        op = AllGatherGemm(ctx, ROWS, K_DIM, n_local, dt, plan="swizzle", comm=args.comm, chunk_split=args.chunk_split,
                           copy_streams=args.copy_streams, transfer=args.ag_transfer if args.comm == "ce" else "pull",
                           flag_stream=not args.no_flag_stream, lockstep=ag_lockstep)
        op.shard.copy_(shard_seed(rank).to(dev))
        step = lambda: op(b, c)
        # the GEMM kernel and, with a barrier in front of the transfers, the barrier kernel
        kernels_per_step = 1 if ag_lockstep == "pairwise" else 2
    else:
        from syncopate_b200.operators import plan_all_gather

        a_full = torch.cat([shard_seed(r) for r in range(tp)], 0).to(dev)
        a_sched = plan_all_gather(tp, ROWS, K_DIM, dt, "swizzle")[2][0]["a"]  # rank 0 of the TP=8 plan
        wave_offsets = [[o[0], 0] for o in a_sched.gen_block_offset_lists()]
        wave_sizes = [[s[0], n_local] for s in a_sched.gen_block_shape_lists()]
        flags = torch.ones(tp, dtype=torch.int64, device=dev)
        sig_offsets = a_sched.gen_signal_lists()
        step = lambda: gemm(a_full, b, c, cur_wave_sizes=wave_sizes, wave_offsets=wave_offsets,
                            signal_ptr=flags, signal_offsets=sig_offsets, status=ctx.status)
        kernels_per_step = 1
    head = timed(step)
    ms = head["ms"]
    launches[0] = steps * blocks * kernels_per_step
    per_gpu = flop / (ms * 1e-3) / 1e12
    value = per_gpu * world

    # ---- parity of the headline operator (outside the timed region)
    if world > 1:
        gathered = [torch.empty(ROWS, K_DIM, dtype=dt, device=dev) for _ in range(world)]
        dist.all_gather(gathered, op.shard.contiguous())
        full_a = torch.cat(gathered, 0)
        bit_exact = bool(torch.equal(op.a.local, full_a))
    else:
        full_a, bit_exact = a_full, True
    worst = [0.0, 0.0]
    for r0, ref in matmul_blocks(full_a, b):
        glob, tile = gemm_parity(c[r0:r0 + ref.shape[0]], ref)
        worst = [max(worst[0], glob), max(worst[1], tile)]
    parity["ag_gemm"] = {"rel_frobenius": worst[0], "worst_tile_rel_frobenius": worst[1], "tol": GEMM_TOL}
    parity["gathered_bit_exact"] = bit_exact
    if world > 1:
        del gathered

    # ---- yardstick: cuBLAS (torch.matmul) on the same local shape, in the same run (not on the product path)
    c_ref = torch.empty(M, n_local, dtype=dt, device=dev)
    bt = b.t()
    cublas = timed(lambda: torch.matmul(full_a, bt, out=c_ref), n_blocks=max(3, blocks // 2), n_warm=3)
    del c_ref

    # ---------------- the same GEMM with every chunk already resident (flags pre-set, no transfers),
    # timed while all ranks compute: the non-overlapped share of the fused step is the difference
    compute_only = None
    other_comm = None
    trace_rows = None
    if world > 1:
        ones = torch.full((max(op.info.recv_signal_num, 1),), 1 << 40, dtype=torch.int64, device=dev)
        offs = [[o[0], 0] for o in op.schedule.gen_block_offset_lists()]
        sizes = [[s_[0], n_local] for s_ in op.schedule.gen_block_shape_lists()]
        sigs = op.schedule.gen_signal_lists()
        compute_only = timed(lambda: gemm(op.a.local, b, c, cur_wave_sizes=sizes, wave_offsets=offs, signal_ptr=ones,
                                          signal_offsets=sigs, status=ctx.status), n_blocks=max(3, blocks // 2), n_warm=3)
        # per-wave flag waits of one call (kernel time stamps): where the non-overlapped time sits
        trace_rows, kernel_us = capture_trace(op, step, [s_[0] for s_ in sizes], sigs)
        # the other transport, for the record
        alt = "sm" if args.comm == "ce" else "ce"
        if not args.skip_alt_comm:
            op2 = AllGatherGemm(ctx, ROWS, K_DIM, n_local, dt, plan="swizzle", comm=alt, chunk_split=args.chunk_split,
                                copy_streams=args.copy_streams)
            op2.shard.copy_(shard_seed(rank).to(dev))
            sync_all()
            other_comm = timed(lambda: op2(b, c), n_blocks=max(3, blocks // 2), n_warm=3)
            other_comm["comm_mode"] = alt
            del op2

    # ---------------- e2e: host buffers in, host result out, through the operator API; every step's
    # copies are inside the timed region, consecutive steps overlap over separate streams
    e2e_steps = max(3, min(steps, 10))
    cur = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    c_host = torch.empty(M, n_local, dtype=dt).pin_memory()
    c_dev = [c, torch.empty_like(c)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    if world > 1:
        # Three operator instances: the shard of instance i % 3 is rewritten for step i while step
        # i - 1 computes; by the time step i - 2 has finished here, every peer has entered step i - 2
        # and so finished pulling what step i - 3 left in that shard.
        a_host = shard_seed(rank).pin_memory()
        sets = [op] + [AllGatherGemm(ctx, ROWS, K_DIM, n_local, dt, plan="swizzle", comm=args.comm,
                                     chunk_split=args.chunk_split, copy_streams=args.copy_streams,
                                     transfer=args.ag_transfer if args.comm == "ce" else "pull",
                                     flag_stream=not args.no_flag_stream, lockstep=ag_lockstep) for _ in range(2)]
        ev_in = [torch.cuda.Event() for _ in range(3)]
        ev_comp = [torch.cuda.Event() for _ in range(3)]
        e2e_path = ("pinned host A shard -> symmetric device shard, fused operator, C -> pinned host; three operator "
                    "instances and two result buffers on three streams, so consecutive steps overlap")

        def e2e_run(n):
            for i in range(n):
                k, kc = i % 3, i & 1
                s_in.wait_event(ev_comp[(i + 1) % 3])  # step i - 2 has finished on this rank
                with torch.cuda.stream(s_in):
                    sets[k].shard.copy_(a_host, non_blocking=True)
                    ev_in[k].record(s_in)
                cur.wait_event(ev_in[k])
                cur.wait_event(ev_out[kc])
                sets[k](b, c_dev[kc])
                ev_comp[k].record(cur)
                s_out.wait_event(ev_comp[k])
                with torch.cuda.stream(s_out):
                    c_host.copy_(c_dev[kc], non_blocking=True)
                    ev_out[kc].record(s_out)
            cur.wait_stream(s_out)
    else:
        a_host = a_full.cpu().pin_memory()
        a_dev = [a_full, torch.empty_like(a_full)]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_comp = [torch.cuda.Event() for _ in range(2)]
        e2e_path = ("pinned host A -> device, GEMM call, C -> pinned host; three streams and two device buffer sets, "
                    "so consecutive steps overlap; every step's copies are inside the timed region")

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

    e2e_run(3)
    sync_all()
    e2e = timed(lambda: e2e_run(e2e_steps), n_steps=1, n_blocks=max(3, blocks // 2), n_warm=0)
    e2e_ms = e2e["ms"] / e2e_steps
    e2e_value = flop / (e2e_ms * 1e-3) / 1e12 * world
    h2d = a_host.numel() * 2
    d2h = c_host.numel() * 2
    if world > 1:
        del sets

    # ---------------- GEMM + reduce-scatter on the paired shape (reported, not the headline)
    rs_k = RS_K_TOTAL // tp
    ra = seeded(2000 + rank, (RS_M, rs_k), 1.0, dt).to(dev)
    rb = seeded(3000 + rank, (RS_N, rs_k), 0.02, dt).to(dev)
    rs_other = None
    rs_other_reduce = None
    rs_reduce_mode = None
    rs_compute_only = None
    rs_trace_rows = None
    ar_result = None
    rs_bytes_per_rank = (world - 1) * (RS_M // world) * RS_N * 2 if world > 1 else 0
    if world > 1:
        rs = GemmReduceScatter(ctx, RS_M, RS_N, dt, plan="direct", comm=args.rs_comm, chunk_split=args.rs_split,
                               copy_streams=args.copy_streams, flag_stream=not args.no_flag_stream, reduce=args.rs_reduce)
        rs_reduce_mode = rs.reduce
        rout = torch.empty(RS_M // world, RS_N, dtype=dt, device=dev)
        rs_t = timed(lambda: rs(ra, rb, rout), n_warm=3)
        # parity: fp32 product of this rank's operands, reduce-scattered with torch.distributed
        ref_slab = torch.zeros(RS_M // world, RS_N, dtype=torch.float32, device=dev)
        part = torch.empty(RS_M, RS_N, dtype=torch.float32, device=dev)
        for r0, blk in matmul_blocks(ra, rb):
            part[r0:r0 + blk.shape[0]] = blk
        dist.reduce_scatter_tensor(ref_slab, part)
        del part
        glob, tile = gemm_parity(rout, ref_slab)
        parity["gemm_rs"] = {"rel_frobenius": glob, "worst_tile_rel_frobenius": tile, "tol": GEMM_TOL}
        del ref_slab
        # the kernel walks the remote waves of the plan, then the locally kept slab cut into its row pieces
        rs_rows = [s_[0] for s_, t_ in zip(rs.src_schedule.gen_block_shape_lists(), rs.src_schedule.gen_target_rank_list())
                   if t_ >= 0 and t_ != rank]
        own_pieces = max(args.rs_split, 1)
        rs_rows += [RS_M // world // own_pieces] * own_pieces
        rs_trace_rows, rs_kernel_us = capture_trace(rs, lambda: rs(ra, rb, rout), rs_rows,
                                                    ["remote"] * (len(rs_rows) - own_pieces) + ["reduce"] * own_pieces)
        rfull = torch.empty(RS_M, RS_N, dtype=dt, device=dev)
        rs_compute_only = timed(lambda: gemm(ra, rb, rfull, status=ctx.status), n_blocks=max(3, blocks // 2), n_warm=3)
        del rfull
        # GEMM + all-reduce on the same shape: reduce-scatter in the kernel + all-gather of the reduced rows
        from syncopate_b200.operators import GemmAllReduce

        ar = GemmAllReduce(ctx, RS_M, RS_N, dt, num_splits=args.ar_splits, chunk_split=1, comm=args.rs_comm,
                           copy_streams=args.copy_streams, sync_after=True, reduce=args.rs_reduce)
        ar_t = timed(lambda: ar(ra, rb), n_blocks=max(3, blocks // 2), n_warm=3)
        ar_ref = torch.empty(RS_M, RS_N, dtype=torch.float32, device=dev)
        for r0, blk in matmul_blocks(ra, rb):
            ar_ref[r0:r0 + blk.shape[0]] = blk
        dist.all_reduce(ar_ref)
        glob, tile = gemm_parity(ar.out.local, ar_ref)
        parity["gemm_ar"] = {"rel_frobenius": glob, "worst_tile_rel_frobenius": tile, "tol": GEMM_TOL}
        del ar_ref
        ar_bytes = 2 * rs_bytes_per_rank
        ar_result = {"workload": f"GEMM+AR bf16 TP={tp}: A [{RS_M},{rs_k}], B [{RS_N},{rs_k}], out [{RS_M},{RS_N}] on every rank, "
                                 f"{args.ar_splits} row slices (reduce-scatter in the kernel, all-gather by copy engines; "
                                 "includes the closing barrier that makes the output reusable)",
                     "ms_per_step": ar_t["ms"], "ms_min": ar_t["ms_min"], "ms_max": ar_t["ms_max"],
                     "per_gpu_tflops": 2.0 * RS_M * RS_N * rs_k / (ar_t["ms"] * 1e-3) / 1e12,
                     "nvlink_gbs_achieved": ar_bytes / (ar_t["ms"] * 1e-3) / 1e9,
                     "fused_roofline_ms": max(2.0 * RS_M * RS_N * rs_k / (peaks["bf16_tflops"] * 1e12),
                                              ar_bytes / (NVLINK_GBS_NOMINAL * 1e9)) * 1e3}
        ar_result["frac_of_fused_roofline"] = ar_result["fused_roofline_ms"] / ar_t["ms"]
        del ar
        if not args.skip_alt_comm:
            alt = "sm" if args.rs_comm == "ce" else "ce"
            rs2 = GemmReduceScatter(ctx, RS_M, RS_N, dt, plan="direct", comm=alt, chunk_split=args.rs_split,
                                    copy_streams=args.copy_streams, reduce=args.rs_reduce)
            rs_other = timed(lambda: rs2(ra, rb, rout), n_blocks=max(3, blocks // 2), n_warm=3)
            rs_other["comm_mode"] = alt
            del rs2
            alt_red = "pass" if rs.reduce == "epilogue" else "epilogue"
            rs3 = GemmReduceScatter(ctx, RS_M, RS_N, dt, plan="direct", comm=args.rs_comm, chunk_split=args.rs_split,
                                    copy_streams=args.copy_streams, flag_stream=not args.no_flag_stream, reduce=alt_red)
            rs_other_reduce = timed(lambda: rs3(ra, rb, rout), n_blocks=max(3, blocks // 2), n_warm=3)
            rs_other_reduce["reduce_mode"] = alt_red
            del rs3
    else:
        rout = torch.empty(RS_M, RS_N, dtype=dt, device=dev)
        rs_t = timed(lambda: gemm(ra, rb, rout, status=ctx.status), n_warm=3)
        worst = [0.0, 0.0]
        for r0, ref in matmul_blocks(ra, rb):
            glob, tile = gemm_parity(rout[r0:r0 + ref.shape[0]], ref)
            worst = [max(worst[0], glob), max(worst[1], tile)]
        parity["gemm_rs"] = {"rel_frobenius": worst[0], "worst_tile_rel_frobenius": worst[1], "tol": GEMM_TOL,
                             "note": "1 GPU: the local GEMM of the operator"}
    rs_ms = rs_t["ms"]
    rs_flop = 2.0 * RS_M * RS_N * rs_k
    rs_per_gpu = rs_flop / (rs_ms * 1e-3) / 1e12

    # ---------------- all-to-all + GEMM and GEMM + all-to-all + GEMM (the reference's LLaMA-3.1-70B shapes of
    # tests/test_all2all_gemm.py:200-232 and tests/test_gemm_all2all_gemm.py:213-250; reported, not the headline)
    a2a_results = {}
    if world > 1 and not args.skip_a2a:
        from syncopate_b200.operators import AllToAllGemm, GemmAllToAllGemm

        hidden, heads, hd = 8192, 64, 128
        Bq, Sq = 2, 2048 * world                       # 4096 rows per rank
        ag2 = AllToAllGemm(ctx, Bq, Sq, heads, hd, hidden, dt, num_copy_sms=args.copy_sms)
        xa = seeded(6000 + rank, (Bq, Sq, heads // world, hd), 1.0, dt).to(dev)
        wa = seeded(6100, (hidden, hidden), 0.02, dt).to(dev)
        oa = torch.empty(Bq * Sq // world, hidden, dtype=dt, device=dev)
        ag2.src.copy_(xa)
        sync_all()
        t_a = timed(lambda: ag2(wa, oa), n_blocks=max(3, blocks // 2), n_warm=3)
        parts = [torch.empty_like(xa) for _ in range(world)]
        dist.all_gather(parts, xa)
        Sl = Sq // world
        a_ref = torch.cat(parts, dim=2)[:, rank * Sl:(rank + 1) * Sl].reshape(Bq * Sl, hidden)
        del parts
        worst = [0.0, 0.0]
        for r0, ref in matmul_blocks(a_ref, wa):
            glob, tile = gemm_parity(oa[r0:r0 + ref.shape[0]], ref)
            worst = [max(worst[0], glob), max(worst[1], tile)]
        same = bool(torch.equal(ag2.a, a_ref))
        parity["a2a_gemm"] = {"rel_frobenius": worst[0], "worst_tile_rel_frobenius": worst[1], "tol": GEMM_TOL,
                              "resharded_bit_exact": same}
        fl = 2.0 * (Bq * Sl) * hidden * hidden
        nbytes = (world - 1) * Bq * Sl * (heads // world) * hd * 2
        a2a_results["a2a_gemm"] = {
            "workload": f"all-to-all + GEMM bf16 TP={world}: x [{Bq},{Sq},{heads // world},{hd}] per rank -> [{Bq * Sl},{hidden}] @ W[{hidden},{hidden}]^T; "
                        f"SM copies on {args.copy_sms} SMs, K-gated tcgen05 GEMM on the others",
            "ms_per_step": t_a["ms"], "ms_min": t_a["ms_min"], "ms_max": t_a["ms_max"],
            "per_gpu_tflops": fl / (t_a["ms"] * 1e-3) / 1e12, "frac_of_peak": fl / (t_a["ms"] * 1e-3) / 1e12 / peaks["bf16_tflops"],
            "nvlink_gbs_achieved": nbytes / (t_a["ms"] * 1e-3) / 1e9}
        del ag2, a_ref, xa, oa
        Mm, ffn = 4096 * world, 28672
        mlp = GemmAllToAllGemm(ctx, Mm, hidden, ffn, dt, num_copy_sms=args.copy_sms)
        xm = seeded(6200, (Mm, hidden), 0.1, dt).to(dev)
        w1 = seeded(6300 + rank, (ffn // world, hidden), 0.1, dt).to(dev)
        w2 = seeded(6400, (hidden, ffn), 0.02, dt).to(dev)
        om = torch.empty(Mm // world, hidden, dtype=dt, device=dev)
        sync_all()
        t_m = timed(lambda: mlp(xm, w1, w2, om), n_steps=max(3, min(steps, 10)), n_blocks=max(3, blocks // 2), n_warm=2)
        w1s = [torch.empty_like(w1) for _ in range(world)]
        dist.all_gather(w1s, w1)
        rows = slice(rank * (Mm // world), (rank + 1) * (Mm // world))
        mid = torch.empty(Mm // world, ffn, dtype=dt, device=dev)
        for r0, blk in matmul_blocks(xm[rows], torch.cat(w1s, 0)):
            mid[r0:r0 + blk.shape[0]] = blk.to(dt)
        del w1s
        worst = [0.0, 0.0]
        for r0, ref in matmul_blocks(mid, w2):
            glob, tile = gemm_parity(om[r0:r0 + ref.shape[0]], ref)
            worst = [max(worst[0], glob), max(worst[1], tile)]
        parity["gemm_a2a_gemm"] = {"rel_frobenius": worst[0], "worst_tile_rel_frobenius": worst[1], "tol": GEMM_TOL}
        fl = 2.0 * Mm * (ffn // world) * hidden + 2.0 * (Mm // world) * hidden * ffn
        a2a_results["gemm_a2a_gemm"] = {
            "workload": f"GEMM + all-to-all + GEMM bf16 TP={world}: x [{Mm},{hidden}] @ W1_r[{ffn // world},{hidden}]^T -> all-to-all -> "
                        f"[{Mm // world},{ffn}] @ W2[{hidden},{ffn}]^T; SM copies on {args.copy_sms} SMs",
            "ms_per_step": t_m["ms"], "ms_min": t_m["ms_min"], "ms_max": t_m["ms_max"],
            "per_gpu_tflops": fl / (t_m["ms"] * 1e-3) / 1e12, "frac_of_peak": fl / (t_m["ms"] * 1e-3) / 1e12 / peaks["bf16_tflops"]}
        del mlp, mid, xm, w1, w2, om

    # ---------------- attention operators at the benchmark shapes (reported, not the headline)
    attn_results = {}
    if not args.skip_attention:
        from syncopate_b200.operators import ContextParallelAttention, UlyssesAttention
        from syncopate_b200.runtime import EmulatedWorld

        a_steps = max(3, min(steps, 10))
        a_blocks = max(3, blocks // 2)
        # Ulysses: total sequence 32768, 32 heads, D 128, causal; per rank 4 heads over the full sequence
        S_u = 32768
        if world > 1:
            heads_local = 32 // world
            uly = UlyssesAttention(ctx, 1, 32, S_u // world, 128, dt, causal=True)
            uly.qkv_src.local.copy_(seeded(7000 + rank, (3, 1, 32, S_u // world, 128), 1.0, dt).to(dev))
            sync_all()
            u_t = timed(lambda: uly(), a_steps, a_blocks, 2)
            # parity: sampled rows of this rank's output against dense attention over the gathered sequence
            parts = [torch.empty_like(uly.qkv_src.local) for _ in range(world)]
            dist.all_gather(parts, uly.qkv_src.local)
            full = torch.cat(parts, dim=3)  # [3, 1, 32, S, D]
            del parts
            Sl = S_u // world
            kpos = torch.arange(S_u, device=dev)
            err = 0.0
            for h in (rank % 32, (5 * rank + 3) % 32):
                for t in sample_tiles(Sl // 128, 40 + rank):
                    rows = torch.arange(rank * Sl + t * 128, rank * Sl + (t + 1) * 128, device=dev)
                    err = max(err, attn_rows_error(uly.out.local[0, t * 128:(t + 1) * 128, h], full[0, 0, h, rows],
                                                   full[1, 0, h], full[2, 0, h], rows, kpos))
            del full
        else:
            from syncopate_b200.computation.attn import AttentionState, attention_forward

            heads_local = 4
            uq = seeded(7000, (3, 1, heads_local, S_u, 128), 1.0, dt).to(dev)
            uo = torch.empty(1, heads_local, S_u, 128, dtype=dt, device=dev)
            ust = AttentionState(1, heads_local, S_u, dev)
            u_t = timed(lambda: attention_forward(uq[0], uq[1], uq[2], 128 ** -0.5, uo, causal=True, state=ust,
                                                  status=ctx.status), a_steps, a_blocks, 2)
            kpos = torch.arange(S_u, device=dev)
            err = 0.0
            for h in (0, heads_local - 1):
                for t in sample_tiles(S_u // 128, 40 + h, extra=3):
                    rows = torch.arange(t * 128, (t + 1) * 128, device=dev)
                    err = max(err, attn_rows_error(uo[0, h, rows], uq[0, 0, h, rows], uq[1, 0, h], uq[2, 0, h], rows, kpos))
        parity["ulysses"] = {"max_abs_sampled_rows": max_over_ranks([err])[0], "tol": ATTN_TOL}
        u_flop = 4.0 * S_u * S_u * 128 * heads_local / 2
        attn_results["ulysses_attn"] = {
            "workload": f"cfg3 Ulysses all2all+attention+all2all bf16: S={S_u}, 32 heads, D=128, causal; {heads_local} heads per rank"
                        + (" (1 GPU: attention only)" if world == 1 else ""),
            "ms_per_step": u_t["ms"], "ms_min": u_t["ms_min"], "ms_max": u_t["ms_max"],
            "per_gpu_tflops_causal": u_flop / (u_t["ms"] * 1e-3) / 1e12,
            "frac_of_peak": u_flop / (u_t["ms"] * 1e-3) / 1e12 / peaks["bf16_tflops"]}
        # context parallel: total sequence 65536, 64 Q heads / 8 KV heads, causal zigzag
        cp_world = world if world > 1 else 8
        S_c = 65536
        s_local = S_c // cp_world
        if world > 1:
            cp = ContextParallelAttention(ctx, 1, 64, 8, s_local, 128, dt, causal=True, zigzag=True, plan="swizzle")
            cp.kv_shard.copy_(seeded(8000 + rank, (2, 1, 8, s_local, 128), 1.0, dt).to(dev))
        else:
            ew = EmulatedWorld(cp_world)
            cp = ContextParallelAttention(ew.contexts[0], 1, 64, 8, s_local, 128, dt, causal=True, zigzag=True)
            cp.kv.local.copy_(seeded(8000, (2, 1, 8, S_c, 128), 1.0, dt).to(dev))
            cp.ops, cp.comm = [], None  # one GPU: K/V already gathered, flags pre-set
            cp.flags.local.fill_(1 << 40)
        cq = seeded(9000 + rank, (1, 64, s_local, 128), 1.0, dt).to(dev)
        co = torch.empty_like(cq)
        sync_all()
        c_t = timed(lambda: cp(cq, co), a_steps, a_blocks, 2)
        if world == 1 and cp.ctx.status.tolist()[0] != 0:
            raise RuntimeError(f"context-parallel attention status {cp.ctx.status.tolist()}")
        if world > 1:
            parts = [torch.empty_like(cp.kv_shard.contiguous()) for _ in range(world)]
            dist.all_gather(parts, cp.kv_shard.contiguous())
            full_kv = torch.cat(parts, dim=3)
            del parts
            parity["cp_gathered_bit_exact"] = bool(torch.equal(cp.kv.local, full_kv))
        else:
            full_kv = cp.kv.local
        st = torch.arange(128, device=dev)
        q_pos = (cp.q_pos[:, None] + st[None, :]).reshape(-1)
        k_pos = (cp.kv_pos[:, None] + st[None, :]).reshape(-1)
        err = 0.0
        for h in (rank % 64, (37 + rank) % 64):
            for t in sample_tiles(s_local // 128, 60 + rank):
                rows = torch.arange(t * 128, (t + 1) * 128, device=dev)
                err = max(err, attn_rows_error(co[0, h, rows], cq[0, h, rows], full_kv[0, 0, h // 8], full_kv[1, 0, h // 8],
                                               q_pos[rows], k_pos))
        parity["cp"] = {"max_abs_sampled_rows": max_over_ranks([err])[0], "tol": ATTN_TOL}
        c_flop = 4.0 * S_c * S_c * 128 * 64 / cp_world / 2
        attn_results["cp_attn"] = {
            "workload": f"cfg4 context-parallel all-gather-KV attention bf16: S={S_c} ({s_local} Q tokens per rank), "
                        "64 Q / 8 KV heads, D=128, causal zigzag" + (" (1 GPU: rank 0 of 8, K/V resident)" if world == 1 else ""),
            "ms_per_step": c_t["ms"], "ms_min": c_t["ms_min"], "ms_max": c_t["ms_max"],
            "per_gpu_tflops_causal": c_flop / (c_t["ms"] * 1e-3) / 1e12,
            "frac_of_peak": c_flop / (c_t["ms"] * 1e-3) / 1e12 / peaks["bf16_tflops"]}

    # ---------------- verdict on parity (all ranks agree: the figures above are maxima over ranks)
    for extra in ("a2a_gemm", "gemm_a2a_gemm"):
        if extra in parity:
            v = max_over_ranks([parity[extra]["rel_frobenius"], parity[extra]["worst_tile_rel_frobenius"],
                                0.0 if parity[extra].get("resharded_bit_exact", True) else 1.0])
            parity[extra]["rel_frobenius"], parity[extra]["worst_tile_rel_frobenius"] = v[0], v[1]
            if "resharded_bit_exact" in parity[extra]:
                parity[extra]["resharded_bit_exact"] = v[2] == 0.0
    ar_p = parity.get("gemm_ar", {"rel_frobenius": 0.0, "worst_tile_rel_frobenius": 0.0})
    flat = max_over_ranks([parity["ag_gemm"]["rel_frobenius"], parity["ag_gemm"]["worst_tile_rel_frobenius"],
                           parity["gemm_rs"]["rel_frobenius"], parity["gemm_rs"]["worst_tile_rel_frobenius"],
                           0.0 if parity["gathered_bit_exact"] and parity.get("cp_gathered_bit_exact", True) else 1.0,
                           ar_p["rel_frobenius"], ar_p["worst_tile_rel_frobenius"]])
    if "gemm_ar" in parity:
        parity["gemm_ar"]["rel_frobenius"], parity["gemm_ar"]["worst_tile_rel_frobenius"] = flat[5], flat[6]
    parity["ag_gemm"]["rel_frobenius"], parity["ag_gemm"]["worst_tile_rel_frobenius"] = flat[0], flat[1]
    parity["gemm_rs"]["rel_frobenius"], parity["gemm_rs"]["worst_tile_rel_frobenius"] = flat[2], flat[3]
    parity["gathered_bit_exact"] = flat[4] == 0.0
    ok = (flat[0] < GEMM_TOL and flat[1] < GEMM_TOL and flat[2] < GEMM_TOL and flat[3] < GEMM_TOL and flat[4] == 0.0
          and flat[5] < GEMM_TOL and flat[6] < GEMM_TOL
          and all(parity[k]["max_abs_sampled_rows"] < ATTN_TOL for k in ("ulysses", "cp") if k in parity)
          and all(parity[k]["rel_frobenius"] < GEMM_TOL and parity[k]["worst_tile_rel_frobenius"] < GEMM_TOL
                  and parity[k].get("resharded_bit_exact", True) for k in ("a2a_gemm", "gemm_a2a_gemm") if k in parity))
    parity["ok"] = bool(ok)
    parity["how"] = ("checked on the device after the timed regions: AG+GEMM against an fp32 product of the gathered "
                     "A (torch.distributed all_gather) and the gathered buffer bit for bit; GEMM+RS against fp32 product "
                     "+ reduce_scatter_tensor; attention on sampled query tiles against fp32 dense attention over the "
                     "gathered sequence; maxima over ranks")

    line = None
    if rank == 0:
        clocks = sampler.stop(windows)
        cpu_val, cores, sample, _ = cpu_ag_gemm_sample(tp) if world == 1 else (None, None, None, None)
        peak = peaks["bf16_tflops"]
        nvlink_bytes = (world - 1) * ROWS * K_DIM * 2 if world > 1 else 0
        t_roof_ms = max(flop / (peak * 1e12), nvlink_bytes / (NVLINK_GBS_NOMINAL * 1e9)) * 1e3
        rs_bytes = (world - 1) * (RS_M // world) * RS_N * 2 if world > 1 else 0
        rs_roof_ms = max(rs_flop / (peak * 1e12), rs_bytes / (NVLINK_GBS_NOMINAL * 1e9)) * 1e3
        mhz = clocks.get("sm_mhz") if clocks else None
        line = {
            "metric": "ag_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(world, args.comm, args.chunk_split),
            "timing": {"blocks": head["blocks"], "steps_per_block": steps, "ms_per_step_median": ms,
                       "ms_per_step_min": head["ms_min"], "ms_per_step_max": head["ms_max"],
                       "timed_region_ms_per_block": ms * steps,
                       "ms_x_sm_mhz": ms * mhz if mhz else None},
            "per_gpu_tflops": per_gpu,
            "compute_only_ms": compute_only["ms"] if compute_only else None,
            "non_overlapped_ms": (ms - compute_only["ms"]) if compute_only else 0.0,
            "nvlink_gbs_achieved": nvlink_bytes / (ms * 1e-3) / 1e9 if world > 1 else None,
            "other_comm_mode": other_comm,
            "clocks": clocks,
            "parity": parity,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms, "path": e2e_path},
            # per step: one GEMM kernel; with more than one rank also the operator's lockstep barrier kernel
            "gpu_launches": launches[0],
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s",
                         "frac": per_gpu / peak,
                         # dram__bytes_read.sum + dram__bytes_write.sum of one launch of gemm2_kernel<256,7,0> on
                         # this workload (557.4 MB read + 51.9 MB written, mean of three launches), from an ncu
                         # capture of `bench.py --steps 2 --warmup 3 --skip-attention` with the library as built
                         # from this tree
                         "traffic": 609.4e6 if world == 1 else None,
                         "algorithmic_bytes": (M * K_DIM + n_local * K_DIM + M * n_local) * 2,
                         "peak_source": f"{peaks['source']} cuBLAS bf16 burst (MEASURED_PEAKS.json)",
                         "cublas_same_shape_ms": cublas["ms"],
                         "cublas_same_shape_tflops": flop / (cublas["ms"] * 1e-3) / 1e12,
                         "frac_of_sustained": per_gpu / peaks["bf16_tflops_sustained"] if peaks["bf16_tflops_sustained"] else None,
                         "frac_of_nominal_2250": per_gpu / 2250.0,
                         "fused_roofline_ms": t_roof_ms, "frac_of_fused_roofline": t_roof_ms / ms,
                         "fused_roofline_def": f"max(flop / measured peak, NVLink bytes in / {NVLINK_GBS_NOMINAL:.0f} GB/s)",
                         "nvlink_bytes_in_per_rank": nvlink_bytes},
            "other_ops": {
                "gemm_rs": {"workload": f"cfg2 GEMM+RS bf16 TP={tp}: A [{RS_M},{rs_k}], B [{RS_N},{rs_k}], out "
                                        f"[{RS_M // world if world > 1 else RS_M},{RS_N}]"
                                        + (" (1 GPU: GEMM only)" if world == 1 else ""),
                            "comm_mode": args.rs_comm if world > 1 else None,
                            "chunk_split": args.rs_split if world > 1 else None,
                            "ms_per_step": rs_ms, "ms_min": rs_t["ms_min"], "ms_max": rs_t["ms_max"],
                            "per_gpu_tflops": rs_per_gpu, "frac_of_peak": rs_per_gpu / peak,
                            "fused_roofline_ms": rs_roof_ms, "frac_of_fused_roofline": rs_roof_ms / rs_ms,
                            "nvlink_gbs_achieved": rs_bytes / (rs_ms * 1e-3) / 1e9 if world > 1 else None,
                            "compute_only_ms": rs_compute_only["ms"] if rs_compute_only else None,
                            "reduce_mode": rs_reduce_mode,
                            "other_comm_mode": rs_other, "other_reduce_mode": rs_other_reduce},
                **({"gemm_ar": ar_result} if ar_result is not None else {}),
                **a2a_results,
                **attn_results,
            },
        }
        if trace_rows is not None:
            line["overlap_trace"] = {"kernel_us": kernel_us, "waves": trace_rows,
                                     "note": "one call of the headline operator on rank 0 in steady state (fourth of four "
                                             "back-to-back calls): per wave, earliest flag-wait begin and latest end over "
                                             "CTAs (us from the kernel's start) and the wait summed over CTAs; a wave's "
                                             "latest end is also set by CTAs that reach the wave late"}
        if rs_trace_rows is not None:
            line["other_ops"]["gemm_rs"]["overlap_trace"] = {
                "kernel_us": rs_kernel_us, "waves": rs_trace_rows,
                "note": "one call on rank 0: the reduce waves' waits for the staged partial sums of their rows"}
        if cpu_val is not None:
            line["cpu_baseline"] = {"value": cpu_val, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                    "sample": sample}
    ctx.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line), flush=True)
    if not ok:
        sys.exit(3)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--blocks", type=int, default=10, help="timed blocks of --steps steps; the median block is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-attention", action="store_true", help="leave the attention operators out of other_ops")
    ap.add_argument("--skip-alt-comm", action="store_true", help="do not time the other transport beside the chosen one")
    ap.add_argument("--skip-a2a", action="store_true", help="leave the all-to-all + GEMM operators out of other_ops")
    ap.add_argument("--copy-sms", type=int, default=16, help="SMs of the SM-copy programs beside a GEMM (all-to-all + GEMM)")
    ap.add_argument("--comm", default="ce", choices=["sm", "ce"],
                    help="who moves the all-gather chunks: the kernel's comm warps (sm) or copy engines (ce)")
    ap.add_argument("--chunk-split", type=int, default=2, help="row pieces per remote all-gather slab")
    ap.add_argument("--ag-transfer", default="pull", choices=["pull", "push"],
                    help="copy-engine all-gather: receivers pull, or owners push")
    ap.add_argument("--rs-comm", default="sm", choices=["sm", "ce"],
                    help="GEMM+RS transport: the epilogue's TMA stores (sm) or copy engines (ce)")
    ap.add_argument("--rs-split", type=int, default=1, help="row pieces per reduce-scatter slab")
    ap.add_argument("--rs-reduce", default="auto", choices=["auto", "epilogue", "pass"],
                    help="GEMM+RS / GEMM+AR: staged partial sums added in the own tiles' epilogue, or by a pass behind the kernel")
    ap.add_argument("--ar-splits", type=int, default=1, help="row slices of GEMM+AR (separate launches)")
    ap.add_argument("--copy-streams", type=int, default=1)
    ap.add_argument("--ag-lockstep", default="barrier", choices=["barrier", "pairwise"],
                    help="AG+GEMM by copy-engine pulls: a barrier in front of the transfers, or one 'entered' word per peer")
    ap.add_argument("--no-flag-stream", action="store_true",
                    help="write each chunk's flag on its copy stream instead of a separate flag stream")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_own_arm(args)


if __name__ == "__main__":
    main()
