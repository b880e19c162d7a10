"""The plan grid that pins the front end: every hot-path builder at the benchmark shapes and at
small shapes, with the code-generation options each operator uses.  Shared by
``make_frontend_golden.py`` (runs the reference) and ``tests/test_frontend_golden.py`` (runs this
package); each case is ``(name, builder_name, world, kwargs_without_rank, codegen)`` where codegen
is ``None`` (plan + signals + lowering only), ``"ce"`` (copy engine) or ``"sm"`` (N-D slice ops)."""
import torch

BF16, FP16, FP32 = torch.bfloat16, torch.float16, torch.float32


def cases():
    out = []

    def add(name, builder, world, codegen, **kw):
        out.append((name, builder, world, kw, codegen))

    # ---- all-gather + GEMM
    add("ag_readme_w4", "build_all_gather_plan_1d_swizzle", 4, "ce", shape=(1024, 512), dtype=FP16, axis=0,
        buffer_name="a", transfer_kind="pull")
    add("ag_cfg0_w4", "build_all_gather_plan_1d_swizzle", 4, "ce", shape=(4096, 512), dtype=FP16, axis=0,
        buffer_name="a", transfer_kind="pull")
    for w in (2, 4, 8):
        add(f"ag_cfg1_w{w}", "build_all_gather_plan_1d_swizzle", w, "ce", shape=(1024 * w, 8192), dtype=BF16,
            axis=0, buffer_name="a", transfer_kind="pull")
    add("ag_cfg1_w8_sm", "build_all_gather_plan_1d_swizzle", 8, "sm", shape=(8192, 8192), dtype=BF16, axis=0,
        buffer_name="a", transfer_kind="pull")
    add("ag_push_w4", "build_all_gather_plan_1d_swizzle", 4, "ce", shape=(512, 64), dtype=BF16, axis=0,
        buffer_name="a", transfer_kind="push")
    add("ag_axis1_w4", "build_all_gather_plan_1d_swizzle", 4, "ce", shape=(8, 64), dtype=FP32, axis=1,
        buffer_name="buffer", transfer_kind="pull")
    add("ag_neg_axis_w2", "build_all_gather_plan_1d_swizzle", 2, "sm", shape=(4, 6, 8), dtype=FP16, axis=-2,
        buffer_name="x", transfer_kind="pull")
    # ---- GEMM + reduce-scatter
    for w in (2, 4, 8):
        add(f"rs_direct_cfg2_w{w}", "build_reduce_scatter_direct_reduce_plan", w, "sm", shape=(8192, 8192),
            dtype=BF16, axis=0, src_buffer="src", dst_buffer="dst")
        add(f"rs_a2a_cfg2_w{w}", "build_all_to_all_plan", w, "sm", shape=(8192, 8192), dtype=BF16,
            src_buffer="src", dst_buffer="dst", transfer_kind="push", compute_producer=True)
    add("rs_direct_pull_w4", "build_reduce_scatter_direct_reduce_plan", 4, "sm", shape=(512, 256), dtype=BF16,
        axis=0, src_buffer="src", dst_buffer="dst", transfer_kind="pull")
    add("rs_a2a_ce_w4", "build_all_to_all_plan", 4, "ce", shape=(512, 256), dtype=FP16, src_buffer="src",
        dst_buffer="dst", transfer_kind="push", compute_producer=True)
    add("a2a_pull_w4", "build_all_to_all_plan", 4, "ce", shape=(64, 16), dtype=FP32, src_buffer="s",
        dst_buffer="d", transfer_kind="pull", compute_producer=False)
    add("a2a_pull_cp_w4", "build_all_to_all_plan", 4, "sm", shape=(64, 16), dtype=FP32, src_buffer="s",
        dst_buffer="d", transfer_kind="pull", compute_producer=True)
    add("rs_coll_w4", "build_reduce_scatter_collective_plan", 4, "sm", shape=(512, 256), dtype=BF16, axis=0,
        split_axis=1, src_buffer="src", dst_buffer="dst", num_reduce_scatters=4, compute_producer=True)
    add("rs_coll_default_w2", "build_reduce_scatter_collective_plan", 2, "sm", shape=(64, 32), dtype=FP16, axis=0,
        src_buffer="src", dst_buffer="dst")
    # ---- Ulysses
    add("uly_in_cfg3_w8", "build_all_to_all_plan_dim", 8, "sm", shape=(3, 1, 32, 4096, 128), dtype=BF16,
        src_buffer="src", dst_buffer="dst", src_split_axis=3, dst_split_axis=2, transfer_kind="pull")
    add("uly_out_cfg3_w8", "build_all_to_all_plan_dim", 8, "sm", shape=(1, 32768, 4, 128), dtype=BF16,
        src_buffer="src", dst_buffer="dst", src_split_axis=2, dst_split_axis=1, transfer_kind="push",
        compute_producer=True)
    add("uly_in_small_w2_ce", "build_all_to_all_plan_dim", 2, "ce", shape=(3, 1, 4, 256, 64), dtype=BF16,
        src_buffer="src", dst_buffer="dst", src_split_axis=3, dst_split_axis=2, transfer_kind="pull")
    add("uly_in_ccw_w4", "build_all_to_all_plan_dim", 4, "sm", shape=(2, 8, 128, 64), dtype=BF16,
        src_buffer="src", dst_buffer="dst", src_split_axis=2, dst_split_axis=1, transfer_kind="push",
        peer_order="counter-clockwise")
    add("uly_waves_w4", "build_all_to_all_plan_dim_waves", 4, "sm", shape=(2, 8, 128, 64), dtype=BF16,
        src_buffer="src", dst_buffer="dst", src_split_axis=2, dst_split_axis=1, num_waves=2,
        transfer_kind="pull")
    add("uly_waves_push_cp_w2", "build_all_to_all_plan_dim_waves", 2, "sm", shape=(4, 64, 32), dtype=FP16,
        src_buffer="src", dst_buffer="dst", src_split_axis=0, dst_split_axis=1, num_waves=4,
        transfer_kind="push", compute_producer=True)
    add("a2a_axis_w4", "build_all_to_all_plan_axis", 4, "sm", shape=(4, 64, 32), dtype=FP16, src_buffer="src",
        dst_buffer="dst", split_axis=1, transfer_kind="push")
    add("a2a_axis_pull_cp_w2", "build_all_to_all_plan_axis", 2, "ce", shape=(8, 32), dtype=FP32,
        src_buffer="src", dst_buffer="dst", split_axis=0, transfer_kind="pull", compute_producer=True)
    # ---- context-parallel KV gather
    kv = dict(shape=(2, 1, 8, 65536, 128), dtype=BF16, axis=3, buffer_name="kv")
    add("cp_swizzle_cfg4_w8", "build_all_gather_plan_1d_swizzle", 8, "sm", transfer_kind="pull", **kv)
    add("cp_ring_cfg4_w8", "build_ring_all_gather_plan", 8, "sm", **kv)
    add("cp_dring2_cfg4_w8", "build_double_ring_all_gather_plan", 8, "sm", inner_mesh_size=2, **kv)
    add("cp_dring4_cfg4_w8", "build_double_ring_all_gather_plan", 8, "sm", inner_mesh_size=4, **kv)
    add("ring_small_w4_ce", "build_ring_all_gather_plan", 4, "ce", shape=(64, 8), dtype=FP16, axis=0,
        buffer_name="buf")
    add("dring_small_w4_g1", "build_double_ring_all_gather_plan", 4, "sm", shape=(64, 8), dtype=FP16, axis=0,
        inner_mesh_size=1, buffer_name="buf")
    add("dring_small_w4_g4", "build_double_ring_all_gather_plan", 4, "sm", shape=(64, 8), dtype=FP16, axis=0,
        inner_mesh_size=4, buffer_name="buf")
    add("ring_w1", "build_ring_all_gather_plan", 1, None, shape=(8, 8), dtype=FP16, axis=0, buffer_name="buf")
    # ---- GEMM + all-reduce
    add("ar_cfg2_w8_split4", "build_all_reduce_plan", 8, "sm", shape=(8192, 8192), dtype=BF16, buffer_name="c",
        num_all_reduces=4, split_axis=0, compute_producer=True)
    add("ar_plain_w2", "build_all_reduce_plan", 2, "sm", shape=(64, 32), dtype=FP16, buffer_name="c")
    add("ar_axis1_w4", "build_all_reduce_plan", 4, "ce", shape=(16, 64), dtype=FP32, buffer_name="c",
        num_all_reduces=2, split_axis=-1, compute_producer=False)
    add("ar_nvsharp_w4", "build_all_reduce_nvsharp_plan", 4, "sm", shape=(512, 256), dtype=BF16, src_name="src",
        dst_name="dst", num_all_reduces=2, split_axis=0, compute_producer=True)
    return out


def split_cases():
    """(name, builder, world, kwargs, num_splits): DevicePlan.split_xfers before signal planning."""
    return [
        ("ag_split2_w4", "build_all_gather_plan_1d_swizzle", 4,
         dict(shape=(1024, 512), dtype=FP16, axis=0, buffer_name="a", transfer_kind="pull"), 2),
        ("ag_axis1_split3_w2", "build_all_gather_plan_1d_swizzle", 2,
         dict(shape=(6, 64), dtype=FP32, axis=1, buffer_name="a", transfer_kind="pull"), 3),
        ("rs_coll_split2_w2", "build_reduce_scatter_collective_plan", 2,
         dict(shape=(64, 32), dtype=FP16, axis=0, src_buffer="src", dst_buffer="dst"), 2),
    ]
