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
