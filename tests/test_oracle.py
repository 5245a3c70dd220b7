"""The CPU oracle against an independent numpy restatement, against analytic
known answers, and against the committed golden fixtures.

The reference holds no golden vectors for this path, so these are what pin
the oracle (it stays "parity unpinned" in the strict sense; see oracle.h).
"""
import os

import numpy as np
import pytest

from oracle import oracle as O
from oracle import oracle_np as N
from tests.helpers import lay_caches

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attention_golden.npz")


def test_seq_generator_is_the_reference_xorshift():
    a = O.seq(2000, 71)
    assert np.array_equal(a, N.seq(2000, 71))
    # (s >> 40) / 2^23 * 4 - 2 lies in [-2, 6)
    assert a.min() >= -2.0 and a.max() < 6.0 and abs(float(a.mean()) - 2.0) < 0.1
    assert not np.array_equal(O.seq(16, 1), O.seq(16, 2))


def test_f16_rounding_is_ieee_nearest_even():
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(200000) * 10.0 ** rng.integers(-9, 6, 200000)).astype(np.float32)
    x = np.concatenate([x, np.float32([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, 5.96e-8,
                                       2.98e-8, 2.99e-8, np.inf, -np.inf])])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(O.round_f16(x), want)
    every = np.arange(65536, dtype=np.uint16)
    finite = np.isfinite(every.view(np.float16))
    assert np.array_equal(O.widen_f16(every)[finite],
                          every.view(np.float16).astype(np.float32)[finite])
    assert np.array_equal(O.round_f16(O.widen_f16(every))[finite], every[finite])


@pytest.mark.parametrize("first", [0, 1, 17, 4095])
def test_rope_c_equals_numpy(first):
    t, heads, hd = 5, 3, 128
    x = O.seq(t * heads * hd, 75)
    a = O.rope(x, t, heads, hd, 10000.0, first)
    b = N.rope(x, t, heads, hd, 10000.0, first)
    assert np.abs(a - b).max() <= 1e-6 * 4


def test_rope_known_answers():
    x = O.seq(2 * 3 * 64, 5)
    # position zero is the identity
    assert np.array_equal(O.rope(x, 1, 6, 64, 10000.0, 0), x)
    # a rotation keeps each pair's norm
    y = O.rope(x, 2, 3, 64, 10000.0, 1234).reshape(2, 3, 2, 32)
    x4 = x.reshape(2, 3, 2, 32)
    assert np.allclose((y ** 2).sum(axis=2), (x4 ** 2).sum(axis=2), rtol=1e-5)
    # pair (0, hd/2) has inv_freq 1: angle = position
    one = np.zeros(64, np.float32)
    one[0] = 1.0
    r = O.rope(one, 1, 1, 64, 10000.0, 3)
    assert abs(r[0] - np.cos(3.0)) < 1e-6 and abs(r[32] - np.sin(3.0)) < 1e-6
    # a divisor of 2 on every pair halves the angle of pair 0
    r2 = O.rope(one, 1, 1, 64, 10000.0, 3, np.full(32, 2.0, np.float32))
    assert abs(r2[0] - np.cos(1.5)) < 1e-6 and abs(r2[32] - np.sin(1.5)) < 1e-6


@pytest.mark.parametrize("case", [(4, 2, 128, True, 70, 33, 160), (4, 4, 64, False, 70, 33, 160),
                                  (8, 1, 128, True, 90, 17, 128), (4, 2, 128, True, 130, 5, 138)])
def test_prefill_c_equals_numpy(case):
    heads, kv, hd, causal, tq, past, cap = case
    tk = past + tq
    scale = float(np.float32(hd) ** np.float32(-0.5))
    q = O.seq(tq * heads * hd, 71) * np.float32(100.0)
    kc, vc = lay_caches(O.seq(kv * tk * hd, 72), O.seq(kv * tk * hd, 73), kv, tk, hd, cap)
    a = O.prefill(q, kc, vc, tq, past, heads, kv, hd, cap, scale, causal)
    b = N.prefill(q, kc, vc, tq, past, heads, kv, hd, cap, scale, causal)
    assert np.abs(a - b).max() < 1e-6
    # an f16 cache holding the same roundings gives the same bits
    c = O.prefill(q, O.round_f16(kc), O.round_f16(vc), tq, past, heads, kv, hd, cap, scale, causal)
    assert np.array_equal(a, c)
    # scale folded onto q (the encoder's convention) at a power-of-two scale is exact
    if hd == 64:
        d = O.prefill(q, kc, vc, tq, past, heads, kv, hd, cap, 0.125, causal, scale_q=True)
        e = O.prefill(q, kc, vc, tq, past, heads, kv, hd, cap, 0.125, causal, scale_q=False)
        assert np.abs(d - e).max() < 1e-6
    # the timed variant computes the same function at f32
    f = O.prefill(q, O.round_f16(kc), O.round_f16(vc), tq, past, heads, kv, hd, cap, scale,
                  causal, fast=True, threads=2)
    assert np.abs(a - f).max() < 5e-3 * max(1.0, float(np.abs(a).max()))


def test_prefill_known_answers():
    heads, kv, hd, tq, cap = 4, 2, 64, 6, 8
    rng = np.random.default_rng(1)
    v = rng.standard_normal((kv, tq, hd)).astype(np.float32)
    v16 = O.through_f16(v).reshape(kv, tq, hd)
    kc, vc = lay_caches(np.zeros((kv, tq, hd), np.float32), v, kv, tq, hd, cap)
    q = rng.standard_normal(tq * heads * hd).astype(np.float32)
    out = O.prefill(q, kc, vc, tq, 0, heads, kv, hd, cap, 0.5, True).reshape(tq, heads, hd)
    # zero keys: uniform weights, so a causal row is the running mean of the values
    for r in range(tq):
        for h in range(heads):
            p = O.through_f16(np.full(r + 1, 1.0 / 1.0, np.float32))   # e = 1, l = r + 1
            want = (p[:, None] * v16[h // 2, :r + 1, :]).sum(axis=0) / (r + 1)
            assert np.abs(out[r, h] - want).max() < 1e-6
    # row zero attends to key zero only
    assert np.abs(out[0, 3] - v16[1, 0]).max() < 1e-7
    # non-causal: every row is the mean of all values
    full = O.prefill(q, kc, vc, tq, 0, heads, kv, hd, cap, 0.5, False).reshape(tq, heads, hd)
    assert np.abs(full[2, 0] - v16[0].mean(axis=0)).max() < 1e-6


@pytest.mark.parametrize("case", [(8, 2, 128, 65, 256, False), (6, 6, 64, 1499, 1500, True),
                                  (32, 8, 128, 777, 1024, False)])
def test_decode_variants_agree(case):
    heads, kv, hd, tk, cap, scale_q = case
    q = O.seq(heads * hd, 300)
    k0, v0 = O.seq(kv * cap * hd, 301), O.seq(kv * hd * cap, 302)
    k, v = O.through_f16(k0), O.through_f16(v0)
    kb, vb = O.round_f16(k0), O.round_f16(v0)
    f32 = O.decode_f32(q, k, v, heads, kv, hd, tk, cap, 0.11, scale_q)
    f64 = O.decode_f64(q, kb, vb, heads, kv, hd, 0, tk, cap, 0.11, scale_q)
    npy = N.decode(q, k, v, heads, kv, hd, tk, cap, 0.11, scale_q)
    fast, threads = O.decode_fast(q, kb, vb, heads, kv, hd, tk, cap, 0.11, scale_q, threads=3)
    full = max(float(np.abs(f64).max()), 1e-6)
    assert np.abs(f64 - npy).max() / full < 1e-6
    assert np.abs(f64 - f32).max() / full < 2e-5
    assert np.abs(f64 - fast).max() / full < 2e-5 and threads == 3


def test_partials_merge_to_the_whole():
    """(o, m, l) of key slices merged by log-sum-exp equals the whole
    (crates/llmtie-cuda/src/kernels.rs:5836-5879), including an empty slice's
    m = -inf."""
    heads, kv, hd, tk, cap = 8, 2, 64, 1000, 1024
    q = O.seq(heads * hd, 1)
    kb, vb = O.round_f16(O.seq(kv * cap * hd, 2)), O.round_f16(O.seq(kv * cap * hd, 3))
    whole = O.decode_f64(q, kb, vb, heads, kv, hd, 0, tk, cap, 0.3, False)
    cuts = [0, 137, 137, 600, 1000]
    os_, ms, ls = [], [], []
    for a, b in zip(cuts[:-1], cuts[1:]):
        _, o, m, l = O.decode_f64(q, kb, vb, heads, kv, hd, a, b, cap, 0.3, False, triple=True)
        os_.append(o), ms.append(m), ls.append(l)
    assert np.isneginf(ms[1]).all() and not ls[1].any()
    merged = O.lse_merge(np.stack(os_), np.stack(ms), np.stack(ls), len(os_), heads, hd)
    # the triples travel as f32, so the merge is good to f32 rounding of full scale
    assert np.abs(merged - whole).max() / np.abs(whole).max() < 2e-6


def test_cache_movers():
    n, kv, hd, cap, past = 5, 3, 4, 16, 2
    src = O.seq(n * kv * hd, 9)
    k = np.zeros(kv * cap * hd, np.uint16)
    v = np.zeros(kv * cap * hd, np.uint16)
    O.cache_append_f16(src, k, n, kv, hd, cap, past, False)
    O.cache_append_f16(src, v, n, kv, hd, cap, past, True)
    s16 = O.round_f16(src).reshape(n, kv, hd)
    assert np.array_equal(k.reshape(kv, cap, hd)[:, past:past + n, :], s16.transpose(1, 0, 2))
    assert np.array_equal(v.reshape(kv, hd, cap)[:, :, past:past + n], s16.transpose(1, 2, 0))
    assert not k.reshape(kv, cap, hd)[:, :past].any() and not v.reshape(kv, hd, cap)[:, :, past + n:].any()
    big_k = np.zeros(kv * 32 * hd, np.uint16)
    O.cache_grow(k, big_k, kv, hd, cap, 32, past + n, False)
    direct = np.zeros(kv * 32 * hd, np.uint16)
    O.cache_append_f16(src, direct, n, kv, hd, 32, past, False)
    assert np.array_equal(big_k, direct)
    big_v = np.zeros(kv * 32 * hd, np.uint16)
    O.cache_grow(v, big_v, kv, hd, cap, 32, past + n, True)
    direct = np.zeros(kv * 32 * hd, np.uint16)
    O.cache_append_f16(src, direct, n, kv, hd, 32, past, True)
    assert np.array_equal(big_v, direct)


def test_rope_cache_is_rope_then_append():
    heads, kv, hd, cap, pos = 8, 2, 128, 64, 37
    q, k, v = O.seq(heads * hd, 1), O.seq(kv * hd, 2), O.seq(kv * hd, 3)
    kc = np.zeros(kv * cap * hd, np.uint16)
    vc = np.zeros(kv * cap * hd, np.uint16)
    rq = O.rope_cache_f16(q, k, v, None, heads, kv, hd, 10000.0, pos, kc, vc, cap)
    assert np.array_equal(rq, O.rope(q, 1, heads, hd, 10000.0, pos))
    kc2 = np.zeros(kv * cap * hd, np.uint16)
    vc2 = np.zeros(kv * cap * hd, np.uint16)
    O.cache_append_f16(O.rope(k, 1, kv, hd, 10000.0, pos), kc2, 1, kv, hd, cap, pos, False)
    O.cache_append_f16(v, vc2, 1, kv, hd, cap, pos, True)
    assert np.array_equal(kc, kc2) and np.array_equal(vc, vc2)


def test_golden_fixtures():
    """Inputs are regenerated from their seeds; outputs must match the
    committed vectors (made by tests/golden/make_golden.py from this oracle)."""
    from tests.golden.make_golden import CASES, run_case

    g = np.load(GOLDEN)
    for name, spec in CASES.items():
        got = run_case(spec)
        want = g[name]
        assert got.shape == want.shape
        assert np.abs(got - want).max() <= 1e-6, name


def test_quantize_q8_known_answers_and_numpy_twin():
    """The activation quantiser behind the decode twin (kernels.rs:693-719):
    the group maximum maps to +-127 exactly, an all-zero group to zero codes and
    a zero scale, halves round to even, and the C and numpy restatements agree
    bit for bit on the reference's generator."""
    from oracle import oracle_np as N

    x = np.zeros(96, dtype=np.float32)
    x[0:32] = np.linspace(-1.0, 1.0, 32, dtype=np.float32)
    x[32] = 254.0
    x[33], x[34], x[35] = 1.0, 3.0, -5.0       # scale 2: 0.5, 1.5, -2.5 -> 0, 2, -2
    codes, scales = O.quantize_q8(x)
    assert codes[0] == -127 and codes[31] == 127
    assert scales[0] == np.float32(1.0) * np.float32(1.0 / 127.0)
    assert codes[32] == 127 and scales[1] == np.float32(254.0) * np.float32(1.0 / 127.0)
    assert list(codes[33:36]) == [0, 2, -2]
    assert not codes[64:].any() and scales[2] == 0.0
    y = O.seq(32 * 257, 33)
    c1, s1 = O.quantize_q8(y)
    c2, s2 = N.quantize_q8(y)
    assert np.array_equal(c1, c2) and np.array_equal(s1, s2)
    back = c1.reshape(-1, 32).astype(np.float32) * s1[:, None]
    assert np.abs(back.reshape(-1) - y).max() <= 0.5 * s1.max() * 1.0001


def test_split_heads_is_a_reshape_with_rounding():
    """The cross-attention cache builders (crates/llmtie-cuda/src/kernels.rs:
    5089-5139) against numpy: [t][heads*hd] (+ bias) -> [heads][cap][hd] and
    [heads][hd][cap], f16, zero past t."""
    t, heads, hd, cap = 11, 3, 8, 16
    x = O.seq(t * heads * hd, 5)
    bias = O.seq(heads * hd, 6)
    y = (x.reshape(t, heads * hd) + bias[None, :]).astype(np.float16).reshape(t, heads, hd)
    k = np.zeros((heads, cap, hd), np.float16)
    k[:, :t, :] = y.transpose(1, 0, 2)
    v = np.zeros((heads, hd, cap), np.float16)
    v[:, :, :t] = y.transpose(1, 2, 0)
    assert np.array_equal(O.split_heads_f16(x, bias, t, heads, hd, cap=cap), k.view(np.uint16).reshape(-1))
    assert np.array_equal(O.split_heads_f16(x, bias, t, heads, hd, cap=cap, transposed=True),
                          v.view(np.uint16).reshape(-1))
