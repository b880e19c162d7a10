"""GPU parity of the attention kernel and of the two attention operators against the CPU oracle
(fp32 dense attention of the same seeded inputs).  Tolerance: max-abs error <= 2e-2 on bf16
outputs of O(1) magnitude (the bound the operators are specified to); ~8e-3 is what 16-bit P and
output rounding give."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle import emulate as E  # noqa: E402

pytestmark = pytest.mark.gpu
TOL = 2e-2
DT = torch.bfloat16


@pytest.fixture(autouse=True, params=["one_tile", "two_tile"])
def kernel_choice(request, monkeypatch):
    """Every test runs once with the one-tile kernel and once with the two-tile kernel forced
    (the library would pick by problem size; the test shapes are small).  The benchmark-shape
    tests at the end of the file run once, with the kernel the library picks for them."""
    monkeypatch.setenv("SYNCOPATE_B200_ATTN_TWO_TILE", "0" if request.param == "one_tile" else "2")
    return request.param


def _seeded(seed, shape):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32).to(DT)


def _dense(q, k, v, causal, q_pos=None, k_pos=None):
    """Oracle for [Z, H, S, D] tensors."""
    return torch.stack([E.attention_dense(q[z], k[z], v[z], q.shape[-1] ** -0.5, q_pos, k_pos, causal)[0]
                        for z in range(q.shape[0])])


@pytest.mark.parametrize(
    "Z,Hq,Hkv,Sq,Skv,causal",
    [
        (1, 1, 1, 128, 128, False),
        (1, 2, 2, 256, 512, False),
        (1, 2, 2, 512, 512, True),
        (2, 8, 2, 384, 640, False),   # grouped-query heads, sizes that are not powers of two
        (1, 4, 1, 256, 256, True),
        (1, 2, 2, 384, 384, True),    # odd number of query tiles: the last pair has one tile
        (1, 2, 1, 300, 256, False),   # ragged last tile
        (1, 3, 3, 1280, 1280, True),  # several units per CTA at 148 SMs only when planned per unit
    ],
)
def test_attention_matches_oracle(Z, Hq, Hkv, Sq, Skv, causal):
    from syncopate_b200.computation.attn import attention_forward

    q, k, v = _seeded(1, (Z, Hq, Sq, 128)), _seeded(2, (Z, Hkv, Skv, 128)), _seeded(3, (Z, Hkv, Skv, 128))
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    o = attention_forward(q.cuda(), k.cuda(), v.cuda(), 128 ** -0.5, causal=causal, status=status,
                          timeout_ns=300_000_000)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    assert (o.float().cpu() - _dense(q, k, v, causal)).abs().max().item() < TOL


def test_waves_merge_partial_results_and_lse():
    """Four (Q half, KV half) waves in a scrambled order: rows visited twice are merged; the stored
    LSE (log2 domain) matches the oracle's natural-log LSE."""
    from syncopate_b200.computation.attn import AttentionState, attention_forward

    Z, H, S = 1, 4, 1024
    q, k, v = _seeded(4, (Z, H, S, 128)), _seeded(5, (Z, H, S, 128)), _seeded(6, (Z, H, S, 128))
    offs = [[0, 0, 512, 512], [0, 0, 0, 0], [0, 0, 512, 0], [0, 0, 0, 512]]
    sizes = [[1, 4, 512, 512]] * 4
    st = AttentionState(Z, H, S, "cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    for causal in (False, True):
        o = attention_forward(q.cuda(), k.cuda(), v.cuda(), 128 ** -0.5, wave_offsets=offs, wave_sizes=sizes,
                              causal=causal, state=st, status=status, timeout_ns=300_000_000)
        torch.cuda.synchronize()
        assert status.tolist() == [0, 0, 0, 0]
        want, lse = E.attention_dense(q[0], k[0], v[0], 128 ** -0.5, causal=causal)
        assert (o[0].float().cpu() - want).abs().max().item() < TOL
        assert torch.allclose(st.lse[0].cpu() * 0.6931471805599453, lse, atol=2e-3, rtol=1e-4)


def test_waves_that_start_on_odd_tiles():
    """Waves whose query ranges start or end inside a tile pair: each tile of a pair takes part
    only in the waves that cover it."""
    from syncopate_b200.computation.attn import AttentionState, attention_forward

    Z, H, S = 1, 2, 512
    q, k, v = _seeded(14, (Z, H, S, 128)), _seeded(15, (Z, H, S, 128)), _seeded(16, (Z, H, S, 128))
    offs = [[0, 0, 128, 0], [0, 0, 0, 0], [0, 0, 384, 0]]
    sizes = [[1, 2, 256, 512], [1, 2, 128, 512], [1, 2, 128, 512]]
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    o = attention_forward(q.cuda(), k.cuda(), v.cuda(), 128 ** -0.5, wave_offsets=offs, wave_sizes=sizes,
                          causal=True, state=AttentionState(Z, H, S, "cuda"), status=status, timeout_ns=300_000_000)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    assert (o.float().cpu() - _dense(q, k, v, True)).abs().max().item() < TOL


def test_planned_and_arithmetic_ownership_agree():
    from syncopate_b200.computation.attn import attention_forward

    q, k, v = (_seeded(20 + i, (1, 4, 1024, 128)).cuda() for i in range(3))
    a = attention_forward(q, k, v, 128 ** -0.5, causal=True, balance=True, timeout_ns=300_000_000)
    b = attention_forward(q, k, v, 128 ** -0.5, causal=True, balance=False, timeout_ns=300_000_000)
    torch.cuda.synchronize()
    assert torch.equal(a, b)   # same arithmetic per row whoever owns the tile


def test_strided_layouts_and_output_buffer():
    """BSHD inputs (head stride < sequence stride) and a caller-provided BSHD output."""
    from syncopate_b200.computation.attn import attention_forward

    B, S, H = 2, 256, 3
    qkv = _seeded(7, (3, B, S, H, 128)).cuda()
    out = torch.zeros(B, S, H, 128, dtype=DT, device="cuda")
    q, k, v = (qkv[i].permute(0, 2, 1, 3) for i in range(3))
    res = attention_forward(q, k, v, 128 ** -0.5, out.permute(0, 2, 1, 3), causal=True, timeout_ns=300_000_000)
    torch.cuda.synchronize()
    assert res.data_ptr() == out.data_ptr()
    want = _dense(q.cpu(), k.cpu(), v.cpu(), True)
    assert (out.permute(0, 2, 1, 3).float().cpu() - want).abs().max().item() < TOL


def test_flag_gated_wave_times_out_cleanly():
    from syncopate_b200.computation.attn import attention_forward

    q = torch.zeros(1, 1, 256, 128, dtype=DT, device="cuda")
    flags = torch.zeros(1, dtype=torch.int64, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    attention_forward(q, q, q, 1.0, wave_offsets=[[0, 0, 0, 0]], wave_sizes=[[1, 1, 256, 256]], signal_ptr=flags,
                      signal_offsets=[0], status=status, timeout_ns=1_000_000)
    torch.cuda.synchronize()
    assert status.tolist()[:3] == [1, 0, 0]   # flag timeout on wave 0 / flag 0, nothing hung


def test_rejects_unsupported_shapes():
    from syncopate_b200 import _lib as L
    from syncopate_b200.computation.attn import attention_forward

    q = torch.zeros(1, 1, 128, 64, dtype=DT, device="cuda")
    with pytest.raises(L.SynError, match="SYN_ERR_UNSUPPORTED"):
        attention_forward(q, q, q, 1.0)
    q = torch.zeros(1, 1, 256, 128, dtype=DT, device="cuda")
    with pytest.raises(L.SynError, match="SYN_ERR_SHAPE"):
        attention_forward(q, q, q, 1.0, wave_offsets=[[0, 0, 64, 0]], wave_sizes=[[1, 1, 128, 256]])


@pytest.mark.parametrize("world,B,H,S_local,causal", [(2, 1, 4, 256, True), (4, 2, 4, 128, False)])
@pytest.mark.parametrize("join", [False, True])
def test_ulysses_operator_emulated_ranks(world, B, H, S_local, causal, join):
    """All ranks on one GPU: inbound all-to-all inside the attention kernel, outbound by the SM
    copy kernel; every rank's [B, S/W, H, D] result equals dense attention over the full sequence."""
    from syncopate_b200.operators import UlyssesAttention
    from syncopate_b200.runtime import EmulatedWorld

    ew = EmulatedWorld(world)
    ops = [UlyssesAttention(c, B, H, S_local, 128, DT, causal=causal, timeout_ns=500_000_000, join_waves=join)
           for c in ew.contexts]
    qkv = [_seeded(20 + r, (3, B, H, S_local, 128)) for r in range(world)]
    for r in range(world):
        ops[r].qkv_src.local.copy_(qkv[r].cuda())
    full = torch.cat(qkv, dim=3)
    want = torch.stack([E.attention_dense(full[0, b], full[1, b], full[2, b], 128 ** -0.5, causal=causal)[0]
                        for b in range(B)])  # [B, H, S, D]
    for _it in range(2):
        for op in ops:
            op.launch_attention()
        torch.cuda.synchronize()
        for op in ops:
            op.launch_scatter()
        torch.cuda.synchronize()
        for r, op in enumerate(ops):
            op.wait_output()
            op.ctx.check()
            # the gathered Q/K/V of this rank's heads are bit-exact copies
            heads = slice(r * (H // world), (r + 1) * (H // world))
            assert torch.equal(op.qkv_dst.cpu(), full[:, :, heads])
            got = op.out.local.float().cpu()  # [B, S/W, H, D]
            ref = want[:, :, r * S_local : (r + 1) * S_local].permute(0, 2, 1, 3)
            assert (got - ref).abs().max().item() < TOL
            op.out.local.zero_()


@pytest.mark.parametrize("world,Hq,Hkv,plan,zigzag", [(2, 4, 2, "swizzle", True), (4, 8, 2, "ring", True),
                                                       (4, 4, 4, "double_ring", False)])
@pytest.mark.parametrize("merge", [-1, 1])
def test_context_parallel_operator_emulated_ranks(world, Hq, Hkv, plan, zigzag, merge):
    """``merge`` = 1: the waves behind the first are joined where their key ranges are adjacent
    (one flag, the last chunk's, gates the joined wave)."""
    from syncopate_b200.operators import ContextParallelAttention
    from syncopate_b200.runtime import EmulatedWorld

    B, S_local = 1, 256
    ew = EmulatedWorld(world)
    ops = [ContextParallelAttention(c, B, Hq, Hkv, S_local, 128, DT, causal=True, zigzag=zigzag, plan=plan,
                                    timeout_ns=500_000_000, merge_waves_after=merge) for c in ew.contexts]
    if merge >= 1 and world > 2:
        assert any(len(op.waves[0]) < world for op in ops)   # something was joined
    kv = [_seeded(40 + r, (2, B, Hkv, S_local, 128)) for r in range(world)]
    q = [_seeded(60 + r, (B, Hq, S_local, 128)) for r in range(world)]
    full = torch.cat(kv, dim=3)
    steps = torch.arange(128)
    for _it in range(2):
        for r, op in enumerate(ops):
            op.kv.local.fill_(float("nan"))
            op.kv_shard.copy_(kv[r].cuda())
        outs = [op(q[r].cuda()) for r, op in enumerate(ops)]
        torch.cuda.synchronize()
        for r, op in enumerate(ops):
            op.ctx.check()
            assert torch.equal(op.kv.local.cpu(), full)   # gathered K/V: bit-exact
            q_pos = (op.q_pos.cpu()[:, None] + steps[None, :]).reshape(-1)
            k_pos = (op.kv_pos.cpu()[:, None] + steps[None, :]).reshape(-1) if op.kv_pos is not None else None
            want = _dense(q[r], full[0], full[1], True, q_pos, k_pos)
            assert (outs[r].float().cpu() - want).abs().max().item() < TOL


# ----------------------------------------------------------------------------------------------
# the shapes the benchmark times
# ----------------------------------------------------------------------------------------------
def _sampled_rows_error(out_h, q_h, k_h, v_h, rows, q_pos=None, k_pos=None):
    """max-abs error of ``out_h[rows]`` (one head, [S, D]) against fp32 dense causal attention of those
    query rows over all keys, computed on the device."""
    qs = q_h[rows].float()
    s = (qs @ k_h.float().t()) * (q_h.shape[-1] ** -0.5)
    qp = rows if q_pos is None else q_pos[rows]
    kp = torch.arange(k_h.shape[0], device=k_h.device) if k_pos is None else k_pos
    s = s.masked_fill(kp[None, :] > qp[:, None], float("-inf"))
    ref = torch.softmax(s, dim=-1) @ v_h.float()
    return (out_h[rows].float() - ref).abs().max().item()


def _sample_tiles(n_tiles: int, seed: int, extra: int = 3):
    g = torch.Generator().manual_seed(seed)
    picks = {0, 1, n_tiles // 2, n_tiles // 2 + 1, n_tiles - 2, n_tiles - 1}
    picks.update(int(x) for x in torch.randint(0, n_tiles, (extra,), generator=g))
    return sorted(picks)


@pytest.mark.parametrize("kernel_choice", ["two_tile"], indirect=True)
def test_cfg3_local_shape_sampled_rows(kernel_choice):
    """The per-rank attention of the Ulysses benchmark (4 heads over the full 32768-token sequence,
    causal, planned ownership: 256 key blocks per row, so the lazy rescale of O runs many times):
    sampled query tiles of two heads against fp32 dense attention."""
    from syncopate_b200.computation.attn import AttentionState, attention_forward

    S, H = 32768, 4
    g = torch.Generator(device="cuda").manual_seed(7000)
    qkv = torch.randn(3, 1, H, S, 128, generator=g, device="cuda", dtype=torch.float32).to(DT)
    out = torch.empty(1, H, S, 128, dtype=DT, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    attention_forward(qkv[0], qkv[1], qkv[2], 128 ** -0.5, out, causal=True, state=AttentionState(1, H, S, "cuda"),
                      status=status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    worst = 0.0
    for h in (0, 3):
        for t in _sample_tiles(S // 128, 11 + h):
            rows = torch.arange(t * 128, (t + 1) * 128, device="cuda")
            worst = max(worst, _sampled_rows_error(out[0, h], qkv[0, 0, h], qkv[1, 0, h], qkv[2, 0, h], rows))
    print(f"cfg3 local attention, sampled tiles: max-abs {worst:.2e}")
    assert worst < TOL


@pytest.mark.parametrize("kernel_choice", ["two_tile"], indirect=True)
@pytest.mark.parametrize("join", [False, True])
def test_cfg3_ulysses_world8_emulated_sampled_rows(kernel_choice, join):
    """The Ulysses benchmark configuration itself on eight emulated ranks (32 heads, 4096 tokens per
    rank): 64 (Q slab, KV slab) waves per rank - or, joined, the 8 to 14 waves of contiguous key and
    query ranges that the causal mask leaves - gated by the in-kernel all-to-all, the outbound
    all-to-all, and every rank's sampled output rows against fp32 dense attention over the full
    sequence."""
    from syncopate_b200.operators import UlyssesAttention
    from syncopate_b200.runtime import EmulatedWorld

    W, H, Sl = 8, 32, 4096
    ew = EmulatedWorld(W)
    ops = [UlyssesAttention(c, 1, H, Sl, 128, DT, causal=True, timeout_ns=2_000_000_000, join_waves=join)
           for c in ew.contexts]
    assert all((len(op.waves[0]) == 64) != join for op in ops)
    g = torch.Generator(device="cuda").manual_seed(7100)
    for op in ops:
        op.qkv_src.local.copy_(torch.randn(3, 1, H, Sl, 128, generator=g, device="cuda", dtype=torch.float32).to(DT))
    for op in ops:
        op.launch_attention()
    torch.cuda.synchronize()
    for op in ops:
        op.launch_scatter()
    torch.cuda.synchronize()
    full = torch.cat([op.qkv_src.local for op in ops], dim=3)  # [3, 1, H, S, D]
    worst = 0.0
    for r, op in enumerate(ops):
        op.wait_output()
        op.ctx.check()
        got = op.out.local  # [1, S/W, H, D]
        for h in (r, (r * 5 + 3) % H):
            for t in _sample_tiles(Sl // 128, 100 + r, extra=1)[::2]:
                rows = torch.arange(r * Sl + t * 128, r * Sl + (t + 1) * 128, device="cuda")
                qs = full[0, 0, h, rows].float()
                s = (qs @ full[1, 0, h].float().t()) * (128 ** -0.5)
                s = s.masked_fill(torch.arange(W * Sl, device="cuda")[None, :] > rows[:, None], float("-inf"))
                ref = torch.softmax(s, dim=-1) @ full[2, 0, h].float()
                worst = max(worst, (got[0, t * 128 : (t + 1) * 128, h].float() - ref).abs().max().item())
    print(f"cfg3 Ulysses on 8 emulated ranks, sampled tiles: max-abs {worst:.2e}")
    assert worst < TOL


@pytest.mark.parametrize("kernel_choice", ["two_tile"], indirect=True)
@pytest.mark.parametrize("merge", [-1, 3])
def test_cfg4_rank0_sampled_rows(kernel_choice, merge):
    """Rank 0 of the context-parallel benchmark (64 query / 8 KV heads, 8192 local queries against
    65536 keys, zigzag positions, eight waves gated by the in-kernel K/V gather from eight emulated
    ranks): gathered K/V bit-exact, sampled query tiles against fp32 dense attention with the true
    positions."""
    from syncopate_b200.operators import ContextParallelAttention
    from syncopate_b200.runtime import EmulatedWorld

    W, Hq, Hkv, Sl = 8, 64, 8, 8192
    ew = EmulatedWorld(W)
    g = torch.Generator(device="cuda").manual_seed(8000)
    ops = [ContextParallelAttention(c, 1, Hq, Hkv, Sl, 128, DT, causal=True, zigzag=True, plan="swizzle",
                                    timeout_ns=2_000_000_000, merge_waves_after=merge) for c in ew.contexts]
    for op in ops:
        op.kv.local.fill_(float("nan"))
        op.kv_shard.copy_(torch.randn(2, 1, Hkv, Sl, 128, generator=g, device="cuda", dtype=torch.float32).to(DT))
    q = torch.randn(1, Hq, Sl, 128, generator=g, device="cuda", dtype=torch.float32).to(DT)
    op = ops[0]
    out = op(q)
    torch.cuda.synchronize()
    op.ctx.check()
    full = torch.cat([o.kv_shard for o in ops], dim=3)  # [2, 1, Hkv, S, D]
    assert torch.equal(op.kv.local, full)
    steps = torch.arange(128, device="cuda")
    q_pos = (op.q_pos[:, None] + steps[None, :]).reshape(-1)
    k_pos = (op.kv_pos[:, None] + steps[None, :]).reshape(-1)
    worst = 0.0
    for h in (0, 37, 63):
        for t in _sample_tiles(Sl // 128, 200 + h, extra=2):
            rows = torch.arange(t * 128, (t + 1) * 128, device="cuda")
            worst = max(worst, _sampled_rows_error(out[0, h], q[0, h], full[0, 0, h // (Hq // Hkv)],
                                                   full[1, 0, h // (Hq // Hkv)], rows, q_pos, k_pos))
    print(f"cfg4 rank 0 ({len(op.waves[0])} waves per row), sampled tiles: max-abs {worst:.2e}")
    assert worst < TOL


@pytest.mark.parametrize("kernel_choice", ["two_tile"], indirect=True)
@pytest.mark.parametrize("world,B,H,S_local,causal,num_sms", [(2, 1, 4, 256, True, 0), (4, 2, 4, 128, False, 0),
                                                              (2, 1, 2, 512, True, 3), (4, 1, 8, 256, True, 0)])
def test_ulysses_operator_pushes_finished_tiles(kernel_choice, world, B, H, S_local, causal, num_sms, monkeypatch):
    """The attention kernel in its producer role: every query tile's final rows go straight to the
    rank that owns them, at the tile's last visit (earlier visits merge through the local buffer),
    and a slab's flag is raised by the tile that completes it.  All ranks run one after the other on
    one GPU; with three CTAs a CTA owns several tile pairs, which it visits wave after wave."""
    from syncopate_b200.operators import UlyssesAttention
    from syncopate_b200.runtime import EmulatedWorld
    import syncopate_b200.computation.attn as attn_mod

    if num_sms:
        real = attn_mod.attention_forward
        monkeypatch.setattr("syncopate_b200.operators.attention_forward",
                            lambda *a, **kw: real(*a, **{**kw, "num_sms": num_sms}))
    ew = EmulatedWorld(world)
    ops = [UlyssesAttention(c, B, H, S_local, 128, DT, causal=causal, timeout_ns=500_000_000, overlap_out=True)
           for c in ew.contexts]
    assert all(op.push is not None for op in ops)
    qkv = [_seeded(80 + r, (3, B, H, S_local, 128)) for r in range(world)]
    for r in range(world):
        ops[r].qkv_src.local.copy_(qkv[r].cuda())
    full = torch.cat(qkv, dim=3)
    want = torch.stack([E.attention_dense(full[0, b], full[1, b], full[2, b], 128 ** -0.5, causal=causal)[0]
                        for b in range(B)])  # [B, H, S, D]
    for it in range(2):
        for op in ops:
            op.out.local.fill_(float("nan"))
        for op in ops:
            op.launch_attention(push=True)      # no copy kernel behind it
        torch.cuda.synchronize()
        for r, op in enumerate(ops):
            op.ctx.check()
            assert op.out_flags.local[:op.out_info.recv_signal_num].tolist() == [it + 1] * op.out_info.recv_signal_num
            assert int(op.push_counters.abs().sum()) == 0
            got = op.out.local.float().cpu()  # [B, S/W, H, D]
            ref = want[:, :, r * S_local : (r + 1) * S_local].permute(0, 2, 1, 3)
            assert (got - ref).abs().max().item() < TOL
