"""How a decode launch is cut over the grid (host logic, no device): one
contiguous run of 128-key units a block, even in units plus a few virtual
units at the head of every (sequence, KV head) pair."""
import numpy as np
import pytest

from ttsxabe_b200 import InvalidArgument, decode_cut


def units(tk, kv):
    return sum(-(-t // 128) * kv for t in tk)


@pytest.mark.parametrize("tk,kv,hd", [
    ([131072] * 8, 8, 128),
    ([16384] * 8, 8, 128),
    ([3000, 2048, 4096, 2500] * 4, 8, 128),
    ([1500], 20, 64),
    ([100] * 32, 64, 64),
    ([37], 1, 128),
    ([129], 8, 128),
])
def test_runs_are_contiguous_increasing_and_cover_every_unit(tk, kv, hd):
    cut = decode_cut(tk, kv, hd, 148)
    w = units(tk, kv)
    grid = len(cut) - 1
    # never fewer than four units a block - unless that is fewer blocks than pairs
    assert grid == min(148, max(1, w // 4, len(tk) * kv))
    assert cut[0] == 0 and cut[-1] == w
    assert all(a < b for a, b in zip(cut, cut[1:])), "every block gets at least one unit"


def test_a_run_that_crosses_a_pair_boundary_carries_fewer_keys():
    tk, kv = [16384] * 8, 8                      # 64 pairs of 128 units over 148 blocks
    cut = decode_cut(tk, kv, 128, 148)
    sizes = np.diff(cut)
    crossing = np.array([(a // 128) != ((b - 1) // 128) for a, b in zip(cut, cut[1:])])
    assert crossing.any() and (~crossing).any()
    # five virtual units at the head of a long pair: the runs that swallow them are shorter
    assert sizes[crossing].max() < np.median(sizes[~crossing])
    assert 4.0 <= sizes[~crossing].mean() - sizes[crossing].mean() <= 6.0
    # short pairs (24 units each) carry three
    cut = decode_cut([3072] * 16, kv, 128, 148)
    sizes = np.diff(cut)
    crossing = np.array([(a // 24) != ((b - 1) // 24) for a, b in zip(cut, cut[1:])])
    assert 1.0 <= sizes[~crossing].mean() - sizes[crossing].mean() <= 4.0
    assert sizes.max() - sizes.min() <= 4


def test_ragged_contexts_are_laid_end_to_end():
    tk, kv = [1000, 130, 4096], 2
    cut = decode_cut(tk, kv, 128, 148)
    assert cut[-1] == (8 + 2 + 32) * kv
    # fewer SMs, fewer blocks; never more blocks than a quarter of the units or the pairs
    assert len(decode_cut(tk, kv, 128, 8)) - 1 == 8
    assert len(decode_cut([128], 1, 128, 148)) - 1 == 1


def test_refusals():
    with pytest.raises(InvalidArgument):
        decode_cut([0], 8, 128)
    with pytest.raises(InvalidArgument):
        decode_cut([128], 8, 96)
    with pytest.raises(InvalidArgument):
        decode_cut([128] * 33, 8, 128)


def test_the_plan_of_a_launch():
    """Which cut a launch takes, on a B200's figures (148 SMs; 74 / 33 / 15
    clusters of 2 / 4 / 8 blocks of the head_dim-128 kernel resident at once,
    148 / 71 / 33 of the head_dim-64 one)."""
    from ttsxabe_b200 import decode_plan

    def plan(tk, kv=8, rows=4, hd=128, **kw):
        return decode_plan(tk, kv, rows, hd, **kw)

    # the benchmark's step: long pairs, cut by work over every SM
    mode, cut = plan([131072] * 8)
    assert mode == 0 and len(cut) - 1 == 148
    # a rank of eight's share of it: 64 equal pairs of 128 units, two blocks a pair
    mode, cut = plan([16384] * 8)
    assert mode == 2 and len(cut) - 1 == 128
    assert all(b - a == 64 for a, b in zip(cut, cut[1:]))
    # one short sequence: eight blocks a pair, three units each
    mode, cut = plan([3000])
    assert mode == 8 and len(cut) - 1 == 64 and cut[-1] == 8 * 24
    assert all(b - a == 3 for a, b in zip(cut, cut[1:]))
    # sixteen pairs' clusters of eight are one too many to be resident at once: four a pair
    assert plan([3000] * 2)[0] == 4
    assert plan([3000] * 2, resident=(74, 36, 16))[0] == 8
    assert plan([3000] * 4)[0] == 4 and plan([700] * 8)[0] == 2
    # one unit a pair: nothing to cut, a block a pair by the cut by work
    mode, cut = plan([100])
    assert mode == 0 and cut == list(range(9))
    # unequal lengths: a cluster a pair only while the longest run stays at eight units
    assert plan([600, 1000, 800, 520])[0] == 4
    assert plan([2048, 4096, 3000, 2500, 2100, 3900, 2300, 4000])[0] == 0
    # Whisper cross-attention (20 heads of 64; two blocks of the narrower kernel fit an
    # SM): 1 and 8 rows by clusters of eight, the 80 pairs of 32 rows by clusters of two
    assert plan([1500], kv=20, rows=1, hd=64)[0] == 8
    assert plan([1500], kv=20, rows=8, hd=64)[0] == 8
    mode, cut = plan([1500], kv=20, rows=32, hd=64)
    assert mode == 2 and len(cut) - 1 == 160 and all(b - a == 6 for a, b in zip(cut, cut[1:]))
    # on a device that held one such block an SM: 80 pairs outnumber half the SMs, and are
    # short: a block a pair
    mode, cut = plan([1500], kv=20, rows=32, hd=64, resident=(74, 33, 15))
    assert mode == 1 and len(cut) - 1 == 80 and all(b - a == 12 for a, b in zip(cut, cut[1:]))
    # 128 equal pairs of 16 units: a block a pair; 96 pairs of 24 units leave too many SMs
    # idle for too long that way: cut by work
    assert plan([2048] * 16)[0] == 1 and plan([3072] * 12)[0] == 0
    # every cut covers every unit once, in order
    for tk, kw in (([3000], {}), ([600, 1000, 800, 520], {}), ([1500], dict(kv=20, rows=32, hd=64)),
                   ([2048] * 16, {}), ([777, 5000, 31], {})):
        mode, cut = plan(tk, **kw)
        kv, rows = kw.get("kv", 8), kw.get("rows", 4)
        assert cut[0] == 0 and cut[-1] == sum(-(-t // 128) for t in tk) * kv * -(-rows // 8)
        assert all(a < b for a, b in zip(cut, cut[1:]))
