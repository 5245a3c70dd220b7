"""Keeping a conversation's cache between completions
(crates/llmtie-chat/src/generate.rs:258-283, :139-141;
crates/llmtie-chat/tests/prefix.rs).

The CPU tests cover the bookkeeping; the GPU test is the reference's own
check at the level this library works at: a prompt prefilled on top of a kept,
truncated prefix against the same prompt prefilled cold into an empty cache.
"""
import numpy as np
import pytest

from oracle import oracle as O


class FakeCache:
    def __init__(self):
        self.len = 0

    def truncate(self, n):
        self.len = min(self.len, n)

    def clear(self):
        self.len = 0


def test_shared_prefix_never_keeps_the_whole_prompt():
    from ttsxabe_b200 import shared_prefix

    assert shared_prefix([1, 2, 3, 4], [1, 2, 9, 9, 9]) == 2
    assert shared_prefix([1, 2, 3, 4], [1, 2, 3, 4]) == 3      # the last token is always run
    assert shared_prefix([1, 2, 3, 4], [1, 2, 3, 4, 5]) == 4
    assert shared_prefix([], [7, 8]) == 0
    assert shared_prefix([7, 8], [5]) == 0
    assert shared_prefix([5], [5]) == 0


def test_prefix_cuts_every_layers_cache_to_what_is_shared():
    from ttsxabe_b200 import Prefix

    caches = [FakeCache(), FakeCache()]
    p = Prefix(caches)
    first = [1, 10, 11, 12, 20, 21]
    assert p.keep(first) == 0
    for c in caches:
        c.len = len(first) + 1          # the prompt and one decoded token
    p.extend(first + [99])
    assert len(p) == 7 and p.shared_with([1, 10, 11, 12, 30]) == 4
    assert p.keep([1, 10, 11, 12, 30, 31]) == 4
    assert [c.len for c in caches] == [4, 4] and p.held == [1, 10, 11, 12]
    p.reset()
    assert len(p) == 0 and [c.len for c in caches] == [0, 0]


@pytest.mark.gpu
def test_a_tail_prefilled_after_a_truncated_cache_matches_the_whole_prompt(gpu):
    """Two prompts share an opening. The first is prefilled and one more token
    decoded on top (so the cache holds more than the second shares with it);
    the cache is cut back to the shared run and the second prompt's tail
    prefilled from there. Its rows must be what a cold prefill of the whole
    second prompt gives - within 1e-3 of the output span (the reference allows
    its logits 2 %), and against the oracle - and the cache must hold the
    second prompt's keys and values bit for bit."""
    from ttsxabe_b200 import KvCache, Prefix

    heads, kv, hd = 8, 2, 128
    scale = float(np.float32(hd) ** np.float32(-0.5))
    rng = np.random.default_rng(77)
    vocab = 500
    # a token's projections depend on the token alone: shared tokens, shared rows
    tq_, tk_, tv_ = (O.through_f16(rng.standard_normal((vocab, n)).astype(np.float32).reshape(-1))
                     .reshape(vocab, n) for n in (heads * hd, kv * hd, kv * hd))
    opening = list(rng.integers(0, vocab, size=300))
    a = opening + list(rng.integers(0, vocab, size=90))
    b = opening + list(rng.integers(0, vocab, size=141))
    b[300] = (a[300] + 1) % vocab          # they differ from there on

    def prefill(cache, ids, past):
        n = len(ids)
        cache.reserve(n)
        out = gpu.prefill_varlen(gpu.upload(tq_[ids].reshape(-1)), gpu.upload(tk_[ids].reshape(-1)),
                                 gpu.upload(tv_[ids].reshape(-1)), [0, n], [cache.k], [cache.v],
                                 [past], [cache.cap], None, heads, kv, hd, 10000.0, scale)
        cache.len = past + n
        return gpu.download(out).reshape(n, heads * hd)

    cold = KvCache(gpu, kv, hd, 4096)
    whole = prefill(cold, b, 0)

    warm = KvCache(gpu, kv, hd, 4096)
    prefix = Prefix([warm])
    assert prefix.keep(a) == 0
    prefill(warm, a, 0)
    prefix.extend(a)
    prefill(warm, [a[1]], warm.len)        # a decoded token on top
    prefix.extend([a[1]])
    shared = prefix.keep(b)
    assert shared == 300 and warm.len == 300
    tail = prefill(warm, b[shared:], shared)
    prefix.extend(b[shared:])
    assert warm.len == len(b) == len(prefix)

    span = float(whole.max() - whole.min())
    assert np.abs(whole[shared:] - tail).max() <= 1e-3 * span
    # the kept cache is the cold one wherever either is live
    live = len(b)
    assert warm.cap == cold.cap
    kw = gpu.download_u16(warm.k).reshape(kv, warm.cap, hd)[:, :live]
    kc = gpu.download_u16(cold.k).reshape(kv, cold.cap, hd)[:, :live]
    vw = gpu.download_u16(warm.v).reshape(kv, hd, warm.cap)[:, :, :live]
    vc = gpu.download_u16(cold.v).reshape(kv, hd, cold.cap)[:, :, :live]
    assert np.array_equal(kw, kc) and np.array_equal(vw, vc)
    # and the oracle agrees with the tail
    qr = O.rope(tq_[b[shared:]].reshape(-1), len(b) - shared, heads, hd, 10000.0, shared)
    want = O.prefill(qr, gpu.download_u16(warm.k), gpu.download_u16(warm.v), len(b) - shared,
                     shared, heads, kv, hd, warm.cap, scale, True, fast=True)
    from tests.helpers import assert_parity
    assert_parity("tail over a kept prefix", want, tail.reshape(-1))
