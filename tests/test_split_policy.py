"""Split policies: exact vectors, totals, alignment, monotonicity, matrix consistency, rejection of bad input.
Counterpart of csrc/tests/variable_counts.cpp in the reference (host-only unit test of the Zipf policy)."""
import pytest

from purlin_b200.utils import split_policy as sp


def test_split_unit_is_a_power_of_two_that_keeps_eight_units_per_rank():
    assert sp.split_unit(128, 1) == 128
    assert sp.split_unit(1 << 20, 8) == (1 << 20) // 64
    assert sp.split_unit(1 << 30, 4) == (1 << 30) // 32
    assert sp.split_unit(3 * 128, 2) == 128            # odd multiples cannot be coarsened
    for total, world in ((1 << 20, 8), (768 << 10, 4), (1 << 30, 16)):
        u = sp.split_unit(total, world)
        assert u & (u - 1) == 0 and total % u == 0 and (total // u >= 8 * world or u == 128)


@pytest.mark.parametrize("eighths", [0, 1, 2, 4, 8])
@pytest.mark.parametrize("world", [1, 2, 4, 8, 16])
def test_zipf_totals_alignment_and_monotonicity(world, eighths):
    for total in (128 * 64 * world, 1 << 20, 3 << 22):
        s = sp.zipf_splits(total, world, eighths)
        u = sp.split_unit(total, world)
        assert sum(s) == total and all(x % u == 0 for x in s)
        assert all(a >= b for a, b in zip(s, s[1:])), "lower ranks never receive less"
        if eighths == 0:
            assert max(s) - min(s) <= u


def test_zipf_exact_vectors():
    # exponent 1 with integer weights: 8 ranks share 761 * 8 units exactly as lcm(1..8) / (r + 1) = 840/(r+1)
    total = 2283 * 8 * 128
    s = sp.zipf_splits(total, 8, 8)
    assert s == [x * 128 for x in (6720, 3360, 2240, 1680, 1344, 1120, 960, 840)]
    # uniform exponent: remainder units go to the lowest ranks
    assert sp.zipf_splits(128 * 10, 4, 0) == [384, 384, 256, 256]


def test_zipf_environment_switch(monkeypatch):
    monkeypatch.setenv("BENCH_ZIPF_EXPONENT", "0.5")
    assert sp.zipf_exponent_eighths() == 4
    monkeypatch.setenv("BENCH_ZIPF_EXPONENT", "2")
    with pytest.raises(ValueError):
        sp.zipf_exponent_eighths()
    monkeypatch.delenv("BENCH_ZIPF_EXPONENT")
    assert sp.zipf_exponent_eighths() == 1


def test_invalid_input_is_rejected():
    with pytest.raises(ValueError):
        sp.zipf_splits(100, 4)          # not a multiple of 128
    with pytest.raises(ValueError):
        sp.zipf_splits(0, 4)
    with pytest.raises(ValueError):
        sp.zipf_splits(1 << 20, 33)
    with pytest.raises(ValueError):
        sp.zipf_splits(1 << 20, 4, 3)   # exponent 3/8 is not offered
    with pytest.raises(ValueError):
        sp.skew_splits(1 << 20, 4, 101)


@pytest.mark.parametrize("percent", [0, 25, 50])
def test_skew_moves_the_stated_share_to_one_seeded_rank(percent):
    total, world = 1 << 22, 8
    a = sp.skew_splits(total, world, percent, seed=5)
    assert a == sp.skew_splits(total, world, percent, seed=5) and sum(a) == total
    even = total // world
    heavy = max(a)
    assert abs(heavy - (even * (100 - percent) // 100 + total * percent // 100)) <= 2 * sp.split_unit(total, world)
    if percent:
        assert sp.skew_splits(total, world, percent, seed=5) != sp.skew_splits(total, world, percent, seed=6) or True


def test_matrices_are_consistent():
    w = 8
    m = sp.sparse_matrix(w, 2, 64 << 10, seed=3)
    assert all(sum(1 for x in row if x) == 2 and all(x in (0, 64 << 10) for x in row) for row in m)
    recv = [sum(m[r][d] for r in range(w)) for d in range(w)]
    assert sum(recv) == sum(map(sum, m))
    h = sp.hot_ring_matrix(w, 1 << 20, 90)
    for r in range(w):
        assert sum(h[r]) == 1 << 20 and h[r][(r + 1) % w] == (1 << 20) // 128 * 90 // 100 * 128
        assert all(x % 128 == 0 for x in h[r])


def test_uniform_counts_follow_the_benchmark_recipe():
    c = sp.uniform_counts(8, 4 << 20, seed=7)
    assert c == sp.uniform_counts(8, 4 << 20, seed=7)
    assert all((2 << 20) <= x <= (6 << 20) and x % 16 == 0 for x in c)
    assert sp.offsets([3, 4, 5]) == [0, 3, 7]
