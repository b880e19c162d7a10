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
