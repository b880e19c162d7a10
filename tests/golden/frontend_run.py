"""Runs one front-end case through a given implementation (module root ``pkg``) and returns its
canonical form.  ``pkg`` is ``"syncopate"`` (the reference) or ``"syncopate_b200"``."""
import importlib
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import canon  # noqa: E402


def run_case(pkg, builder, world, kwargs, codegen, num_splits=None):
    cd = importlib.import_module(f"{pkg}.communication.common_descriptors")
    rs = importlib.import_module(f"{pkg}.communication.common_descriptors.reduce_scatter")
    cg = importlib.import_module(f"{pkg}.communication.code_gen")
    lw = importlib.import_module(f"{pkg}.interface.lowering")
    fn = getattr(cd, builder, None) or getattr(rs, builder)
    plans = {r: fn(rank=r, mesh_size=world, **kwargs) for r in range(world)}
    if num_splits is not None:
        plans = {r: p.split_xfers(num_splits) for r, p in plans.items()}
    out = {"plans_before": {str(r): canon.device_plan(p) for r, p in plans.items()}}
    gen = cg.CommGenerator(plans)
    gen.plan_signals(plan_compute_signals=True)
    out["signals"] = gen.visualize_signals()
    out["counters"] = [gen.receive_signal_counters, gen.transit_signal_counters, gen.compute_signal_counters]
    out["counters"] = [{str(k): v for k, v in c.items()} for c in out["counters"]]
    if codegen is not None:
        try:
            info = gen.generate_code_for_plan(cg.CodeGenOptions(copy_engine=(codegen == "ce")))
            out["comm_info"] = canon.comm_info(info)
        except Exception as exc:  # the reference's codegen rejects some plans: the error is the contract
            out["comm_info_error"] = [type(exc).__name__, str(exc)]
    try:
        low = lw.lower_comm_plan_to_raw_schedules(gen)
        out["lowered"] = canon.lowered(low)
    except ValueError as exc:  # e.g. byte-split regions lose their axes: the error is the contract
        out["lowered_error"] = [type(exc).__name__, str(exc)]
    out["plans_after"] = {str(r): canon.device_plan(p) for r, p in gen.device_plans.items()}
    return out


def compact(full, inline_limit=20000):
    """Golden record of one case: a digest of the complete canonical form, the parts the kernels
    consume (lowered schedules, flag counts, op program) inline, and everything inline when small."""
    import hashlib
    import json

    blob = json.dumps(full, sort_keys=True, separators=(",", ":"))
    rec = {"sha256": hashlib.sha256(blob.encode()).hexdigest()}
    if len(blob) <= inline_limit:
        rec["full"] = full
        return rec
    for key in ("lowered", "lowered_error", "counters", "comm_info", "comm_info_error"):
        if key in full:
            rec[key] = full[key]
    rec["signals_sha256"] = hashlib.sha256(full["signals"].encode()).hexdigest()
    return rec
