"""Pins the CPU oracle: its schedule closed forms against the reference-generated golden vectors,
and its chunk-ordered arithmetic against the un-chunked gather-then-operate definition that the
reference's own GPU tests use as golden output."""
import json
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle import emulate as E  # noqa: E402

GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "frontend_golden.json")))


def _lowered(case, rank, buf):
    rec = GOLDEN[case]
    low = rec["full"]["lowered"] if "full" in rec else rec["lowered"]
    return low[str(rank)][buf]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_swizzle_closed_form_matches_reference_golden(world):
    for rank in range(world):
        want = _lowered(f"ag_cfg1_w{world}", rank, "a")
        got = E.swizzle_pull_schedule(world, rank, 1024, 8192)
        assert got["offsets"] == want["offsets"]
        assert got["shapes"] == want["shapes"]
        assert got["signals"] == want["signals"]
        assert got["targets"] == want["targets"]


def test_readme_hello_world_vector():
    # rank 2 of 4, shape (1024, 512): offsets [[512,0],[768,0],[0,0],[256,0]], signals [-1,0,1,2]
    got = E.swizzle_pull_schedule(4, 2, 256, 512)
    assert got["offsets"] == [[512, 0], [768, 0], [0, 0], [256, 0]]
    assert got["signals"] == [-1, 0, 1, 2]
    assert got["targets"] == [2, 3, 0, 1]
    assert got == {k: _lowered("ag_readme_w4", 2, "a")[k] for k in got}


@pytest.mark.parametrize("world", [2, 4, 8])
def test_direct_reduce_closed_form_matches_reference_golden(world):
    for rank in range(world):
        want = _lowered(f"rs_direct_cfg2_w{world}", rank, "src")
        got = E.direct_reduce_schedule(world, rank, 8192 // world, 8192)
        for key in ("offsets", "shapes", "signals", "targets"):
            assert got[key] == want[key], key


def test_ring_closed_form_matches_reference_golden():
    for rank in range(4):
        want = _lowered("ring_small_w4_ce", rank, "buf")
        got = E.ring_push_schedule(4, rank, 16, 8)
        for key in ("offsets", "shapes", "signals", "targets"):
            assert got[key] == want[key], key


def _inputs(cfg, world, rows, K, N, dtype):
    shards, bs = [], []
    for r in range(world):
        g = torch.Generator().manual_seed(1000 * cfg + r)
        shards.append(torch.randn(rows, K, generator=g, dtype=torch.float32).to(dtype))
        bs.append((torch.randn(N, K, generator=g, dtype=torch.float32) * 0.02).to(dtype))
    return shards, bs


def test_cfg0_chunk_ordered_ag_gemm_equals_unchunked():
    """BASELINE configs[0]: W=4, per-rank A [1024,512] fp16, B [512,1024] fp16 -> C [4096,1024]."""
    world, rows, K, N = 4, 1024, 512, 1024
    shards, bs = _inputs(0, world, rows, K, N, torch.float16)
    full = torch.cat(shards, 0)
    for rank in range(world):
        sched = _lowered("ag_cfg0_w4", rank, "a")
        gathered, c = E.ag_gemm(sched, shards, bs[rank], out_dtype=torch.float32)
        assert torch.equal(gathered, full)
        ref = full.float() @ bs[rank].float().t()
        assert c.shape == (4096, 1024)
        assert (c - ref).abs().max().item() == 0.0


def test_gemm_rs_oracle_equals_matmul_then_reduce_scatter():
    world, M, N, K = 4, 512, 256, 128
    a, b = [], []
    for r in range(world):
        g = torch.Generator().manual_seed(2000 + r)
        a.append(torch.randn(M, K, generator=g).to(torch.bfloat16))
        b.append((torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16))
    scheds = [E.direct_reduce_schedule(world, r, M // world, N) for r in range(world)]
    outs = E.gemm_rs(scheds, a, b, out_dtype=torch.float32)
    partials = [x.float() @ y.float().t() for x, y in zip(a, b)]
    for r in range(world):
        # same addends in the same (rank) order for every output row => bit-equal fp32 sums
        want = torch.zeros(M // world, N)
        for src in range(world):
            want += partials[src][r * (M // world) : (r + 1) * (M // world)]
        assert torch.equal(outs[r], want)


def test_attention_blocks_match_dense_noncausal_and_causal():
    torch.manual_seed(0)
    h, s, d = 2, 256, 64
    q, k, v = (torch.randn(h, s, d).to(torch.bfloat16) for _ in range(3))
    for causal in (False, True):
        dense, lse = E.attention_dense(q, k, v, d ** -0.5, causal=causal)
        blocks = [(ql, 128, kl, 64) for kl in (64, 0, 192, 128) for ql in (128, 0)]
        out, lse_b = E.attention_by_blocks(q, k, v, d ** -0.5, blocks, causal=causal)
        assert torch.allclose(out, dense, atol=2e-6, rtol=1e-5)
        assert torch.allclose(lse_b, lse, atol=1e-5, rtol=1e-5)


def test_attention_dense_matches_torch_sdpa():
    torch.manual_seed(1)
    h, s, d = 3, 128, 32
    q, k, v = (torch.randn(h, s, d) for _ in range(3))
    for causal in (False, True):
        want = torch.nn.functional.scaled_dot_product_attention(q[None], k[None], v[None], is_causal=causal)[0]
        got, _ = E.attention_dense(q, k, v, d ** -0.5, causal=causal)
        assert torch.allclose(got, want, atol=1e-5, rtol=1e-5)


def test_gqa_and_zigzag_positions():
    assert E.zigzag_positions(4, 1, 2).tolist() == [2, 3, 12, 13]
    torch.manual_seed(2)
    q = torch.randn(4, 16, 8)
    k, v = torch.randn(2, 16, 8), torch.randn(2, 16, 8)
    got, _ = E.attention_dense(q, k, v, 1.0)
    want, _ = E.attention_dense(q, k.repeat_interleave(2, 0), v.repeat_interleave(2, 0), 1.0)
    assert torch.equal(got, want)
