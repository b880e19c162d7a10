"""The host model of the kernel's wave dispatch reproduces the known-answer tile orders of the
reference's dispatch simulator (tests/computation/transform/test_transform_pass.py:210-319)."""
import pytest

from syncopate_b200.computation.gemm.plan import tile_order


def _grouped(tile_id, num_pid_m, num_pid_n, group):
    in_group = group * num_pid_n
    gid = tile_id // in_group
    first = gid * group
    gsz = min(num_pid_m - first, group)
    return first + (tile_id % in_group) % gsz, (tile_id % in_group) // gsz


@pytest.mark.parametrize("m,n,g", [(5, 7, 4), (3, 2, 2), (64, 14, 8), (8, 16, 8)])
def test_single_wave_is_the_grouped_raster(m, n, g):
    got = tile_order([(0, 0)], [(m * 128, n * 256)], 128, 256, g)
    assert got == [_grouped(t, m, n, g) for t in range(m * n)]
    assert sorted(got) == [(i, j) for i in range(m) for j in range(n)]


def test_known_answer_one_wave():
    got = tile_order([(0, 0)], [(4, 2)], 1, 1, 8)
    assert got == [(0, 0), (1, 0), (2, 0), (3, 0), (0, 1), (1, 1), (2, 1), (3, 1)]


def test_known_answer_two_waves():
    got = tile_order([(0, 0), (2, 0)], [(2, 2), (2, 2)], 1, 1, 8)
    assert got == [(0, 0), (1, 0), (0, 1), (1, 1), (2, 0), (3, 0), (2, 1), (3, 1)]


def test_merge_wave_tail_joins_adjacent_key_ranges():
    """Wave list of rank 2 of 8 in swizzled order (chunks 2, 3, ..., 7, 0, 1): behind the first
    ``keep`` waves, chunks that are adjacent in the buffer become one wave gated by the last flag."""
    from syncopate_b200.computation.attn.plan import merge_wave_tail

    rows = 8192
    order = (2, 3, 4, 5, 6, 7, 0, 1)
    offs = [[0, 0, 0, r * rows] for r in order]
    shapes = [[1, 64, rows, rows] for _ in order]
    sigs = [-1, 0, 1, 2, 3, 4, 5, 6]
    cum = list(range(1, 9))
    waves = (offs, shapes, sigs, cum)
    assert merge_wave_tail(waves, -1) is waves
    assert merge_wave_tail(waves, 7) is waves
    o, s, g, c = merge_wave_tail(waves, 3)
    assert [x[3] for x in o] == [2 * rows, 3 * rows, 4 * rows, 5 * rows, 0]
    assert [x[3] for x in s] == [rows, rows, rows, 3 * rows, 2 * rows]
    assert g == [-1, 0, 1, 4, 6] and c == [1, 2, 3, 6, 8]
    # every key of every chunk is still covered exactly once
    covered = sorted((x[3], x[3] + y[3]) for x, y in zip(o, s))
    assert covered[0][0] == 0 and covered[-1][1] == 8 * rows
    assert all(a[1] == b[0] for a, b in zip(covered, covered[1:]))
    # a different query box is never joined
    shapes2 = [list(x) for x in shapes]
    shapes2[5][1] = 32
    o2, _s2, _g2, _c2 = merge_wave_tail((offs, shapes2, sigs, cum), 3)
    assert len(o2) == 6


@pytest.mark.parametrize("order", [(0, 1, 2, 3, 4, 5, 6, 7), (2, 3, 4, 5, 6, 7, 0, 1), (7, 0, 1, 2, 3, 4, 5, 6), (1, 0)])
def test_causal_all_to_all_waves_cover_every_visible_pair_once(order):
    """The joined causal waves of the Ulysses operator: whatever the arrival order of the slabs,
    every (query slab, key slab at or below it) pair is covered exactly once, no wave covers a pair
    without a visible key, a wave is gated by the flag of the slab that arrives last among those it
    touches, and there are far fewer waves than slab pairs."""
    from syncopate_b200.computation.attn.plan import all_to_all_wave_metadata

    rows = 4096

    class Schedule:
        def gen_block_offset_lists(self):
            return [[0, 0, 0, r * rows, 0] for r in order]

        def gen_block_shape_lists(self):
            return [[3, 1, 4, rows, 128] for _ in order]

        def gen_signal_lists(self):
            return list(range(len(order)))

    axes = {"batch": 1, "head": 2, "seq": 3}
    offs, shapes, sigs, cum = all_to_all_wave_metadata(Schedule(), axes, causal=True)
    arrival = {slab: step for step, slab in enumerate(order)}
    seen = {}
    for o, s, g in zip(offs, shapes, sigs):
        assert o[:2] == [0, 0] and s[:2] == [1, 4]
        touched = set()
        for q in range(o[2] // rows, (o[2] + s[2]) // rows):
            for k in range(o[3] // rows, (o[3] + s[3]) // rows):
                seen[(q, k)] = seen.get((q, k), 0) + 1
                touched |= {q, k}
        assert g == max(arrival[t] for t in touched)
    n = len(order)
    assert seen == {(q, k): 1 for q in range(n) for k in range(q + 1)}
    assert len(offs) <= 2 * n and cum[-1] == sum(s[0] * s[1] * s[2] for s in shapes)
    # the un-joined form: one wave per ordered pair of slabs
    assert len(all_to_all_wave_metadata(Schedule(), axes)[0]) == n * n


@pytest.mark.parametrize("order", [(0, 1, 2, 3), (2, 3, 0, 1), (1, 3, 0, 2)])
def test_joined_all_to_all_waves_without_a_mask_cover_every_pair_once(order):
    from syncopate_b200.computation.attn.plan import all_to_all_wave_metadata

    rows = 512

    class Schedule:
        def gen_block_offset_lists(self):
            return [[0, 0, 0, r * rows, 0] for r in order]

        def gen_block_shape_lists(self):
            return [[3, 2, 4, rows, 128] for _ in order]

        def gen_signal_lists(self):
            return list(range(len(order)))

    offs, shapes, sigs, _cum = all_to_all_wave_metadata(Schedule(), {"batch": 1, "head": 2, "seq": 3}, join=True)
    arrival = {slab: step for step, slab in enumerate(order)}
    seen = {}
    for o, s, g in zip(offs, shapes, sigs):
        touched = set()
        for q in range(o[2] // rows, (o[2] + s[2]) // rows):
            for k in range(o[3] // rows, (o[3] + s[3]) // rows):
                seen[(q, k)] = seen.get((q, k), 0) + 1
                touched |= {q, k}
        assert g == max(arrival[t] for t in touched)
    n = len(order)
    assert seen == {(q, k): 1 for q in range(n) for k in range(n)}
    assert len(offs) < n * n
