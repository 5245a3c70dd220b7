"""RoPE and the KV-cache movers through the C ABI against the CPU oracle.

Cases and bounds follow the reference's kernel tests
(crates/llmtie-cuda/tests/kernels.rs:1443-1538, :1841-2225).
"""
import numpy as np
import pytest

from oracle import oracle as O
from tests.helpers import assert_close_to

pytestmark = pytest.mark.gpu
EPS = float(np.finfo(np.float32).eps)

LLAMA3_DIV = np.array(
    [1.0] * 29 + [1.207484, 1.553415, 2.026313, 2.69453, 3.684253, 5.257327] + [8.0] * 29,
    dtype=np.float32)


@pytest.mark.parametrize("first", [0, 1, 17, 4095])
def test_rope_matches_at_every_offset(gpu, first):
    t, heads, hd = 5, 3, 128
    x = O.seq(t * heads * hd, 75)
    want = O.rope(x, t, heads, hd, 10000.0, first)
    dev = gpu.upload(x)
    gpu.rope(dev, 0, t, heads, hd, 10000.0, first)
    assert_close_to(f"rope first={first}", want, gpu.download(dev), 1e-5 + first * EPS)


@pytest.mark.parametrize("first", [0, 1, 4095])
def test_scaled_rope_with_llama3_factors(gpu, first):
    t, heads, hd = 4, 3, 128
    x = O.seq(t * heads * hd, 91)
    want = O.rope(x, t, heads, hd, 500000.0, first, LLAMA3_DIV)
    dev = gpu.upload(x)
    gpu.rope_scaled(dev, 0, gpu.upload(LLAMA3_DIV), t, heads, hd, 500000.0, first)
    assert_close_to(f"rope_scaled first={first}", want, gpu.download(dev), 1e-5 + first * EPS)


def test_scaled_rope_with_no_divisor_is_the_unscaled_one(gpu):
    t, heads, hd = 3, 2, 64
    x = O.seq(t * heads * hd, 12)
    a, b = gpu.upload(x), gpu.upload(x)
    gpu.rope(a, 0, t, heads, hd, 10000.0, 7)
    gpu.rope_scaled(b, 0, None, t, heads, hd, 10000.0, 7)
    assert np.array_equal(gpu.download(a), gpu.download(b))


def test_rope_at_an_offset_rotates_that_block_only(gpu):
    t, heads, hd = 5, 3, 64
    span = t * heads * hd
    allv = O.seq(3 * span, 77)
    off = span
    dev = gpu.upload(allv)
    gpu.rope(dev, off, t, heads, hd, 10000.0, 11)
    got = gpu.download(dev)
    want = O.rope(allv[off:off + span], t, heads, hd, 10000.0, 11)
    assert_close_to("rope at an offset", want, got[off:off + span], 1e-5)
    assert np.array_equal(got[:off], allv[:off]), "wrote before the block"
    assert np.array_equal(got[off + span:], allv[off + span:]), "wrote after the block"
    alone = gpu.upload(allv[off:off + span])
    gpu.rope(alone, 0, t, heads, hd, 10000.0, 11)
    assert np.array_equal(gpu.download(alone), got[off:off + span])


@pytest.mark.parametrize("transposed", [False, True])
def test_cache_append_reads_its_own_block(gpu, transposed):
    n, kv, hd, cap, past = 4, 2, 8, 16, 3
    span = n * kv * hd
    allv = O.seq(3 * span, 41)
    off = 2 * span
    src = gpu.upload(allv)
    fused = gpu.zeros(cap * kv * hd)
    gpu.cache_append(src, off, fused, n, kv, hd, cap, past, transposed)
    lone = gpu.upload(allv[off:off + span])
    apart = gpu.zeros(cap * kv * hd)
    gpu.cache_append(lone, 0, apart, n, kv, hd, cap, past, transposed)
    a = gpu.download(fused)
    assert np.array_equal(a, gpu.download(apart))
    want = np.zeros(cap * kv * hd, np.float32)
    O.cache_append_f32(allv[off:off + span], want, n, kv, hd, cap, past, transposed)
    assert np.array_equal(a, want)


@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("shape", [(4, 2, 8, 16, 3), (300, 8, 128, 512, 37), (33, 3, 64, 138, 5)])
def test_cache_append_f16_is_the_oracle_bit_for_bit(gpu, shape, transposed):
    n, kv, hd, cap, past = shape
    src = O.seq(n * kv * hd, 43)
    dst = gpu.upload_u16(np.full(cap * kv * hd, 0x1234, np.uint16))
    gpu.cache_append_f16(gpu.upload(src), 0, dst, n, kv, hd, cap, past, transposed)
    want = np.full(cap * kv * hd, 0x1234, np.uint16)
    O.cache_append_f16(src, want, n, kv, hd, cap, past, transposed)
    assert np.array_equal(gpu.download_u16(dst), want)


def test_rope_cache_f16_is_the_four_launch_chain(gpu):
    """The fused decode-step kernel equals rope twice and cache_append_f16
    twice at t = 1, bit for bit, with q and k at offsets of one buffer and
    pre-filled caches (crates/llmtie-cuda/tests/kernels.rs:1919-2063)."""
    heads, kv, hd, cap, pos = 8, 2, 128, 64, 37
    nq, nk = heads * hd, kv * hd
    buf = O.seq(7 + nq + 5 + nk + 3, 51)
    q_off, k_off = 7, 7 + nq + 5
    vsrc = O.seq(nk + 9, 52)
    v_off = 9
    pattern_k = O.round_f16(O.seq(kv * cap * hd, 53))
    pattern_v = O.round_f16(O.seq(kv * cap * hd, 54))
    for div in (None, LLAMA3_DIV):
        ddiv = None if div is None else gpu.upload(div)
        # fused
        proj = [gpu.upload(buf), gpu.upload(vsrc)]
        kc, vc = gpu.upload_u16(pattern_k), gpu.upload_u16(pattern_v)
        gpu.rope_cache_f16(proj, (0, q_off), (0, k_off), (1, v_off), ddiv, heads, kv, hd,
                           500000.0, pos, kc, vc, cap)
        # the chain
        b2, v2 = gpu.upload(buf), gpu.upload(vsrc)
        kc2, vc2 = gpu.upload_u16(pattern_k), gpu.upload_u16(pattern_v)
        gpu.rope_scaled(b2, q_off, ddiv, 1, heads, hd, 500000.0, pos)
        gpu.rope_scaled(b2, k_off, ddiv, 1, kv, hd, 500000.0, pos)
        gpu.cache_append_f16(b2, k_off, kc2, 1, kv, hd, cap, pos, False)
        gpu.cache_append_f16(v2, v_off, vc2, 1, kv, hd, cap, pos, True)
        fused_buf, chain_buf = gpu.download(proj[0]), gpu.download(b2)
        assert np.array_equal(fused_buf[q_off:q_off + nq], chain_buf[q_off:q_off + nq])
        assert np.array_equal(gpu.download_u16(kc), gpu.download_u16(kc2))
        assert np.array_equal(gpu.download_u16(vc), gpu.download_u16(vc2))
        # the rotated key is never written back to the projection buffer
        assert np.array_equal(fused_buf[k_off:k_off + nk], buf[k_off:k_off + nk])
        assert np.array_equal(fused_buf[:q_off], buf[:q_off])
        # and against the oracle
        okc, ovc = pattern_k.copy(), pattern_v.copy()
        oq = O.rope_cache_f16(buf[q_off:q_off + nq], buf[k_off:k_off + nk],
                              vsrc[v_off:v_off + nk], div, heads, kv, hd, 500000.0, pos, okc,
                              ovc, cap)
        assert_close_to("fused q", oq, fused_buf[q_off:q_off + nq], 1e-5 + pos * EPS)
        assert np.array_equal(gpu.download_u16(vc), ovc)
        dk = O.widen_f16(gpu.download_u16(kc))
        assert np.abs(dk - O.widen_f16(okc)).max() <= 2e-3   # one f16 ulp at |x| < 4


def test_batched_rope_cache_is_the_single_sequence_entry_bit_for_bit(gpu):
    """One launch over several sequences with their own caches, positions and
    capacities equals one rope_cache_f16 call per sequence
    (the loop of crates/llmtie-translate/src/model.rs:824-846)."""
    heads, kv, hd = 8, 2, 64
    nq, nk = heads * hd, kv * hd
    caps, poss = [32, 64, 48, 16], [31, 0, 17, 9]
    batch = len(caps)
    q, k, v = O.seq(batch * nq, 61), O.seq(batch * nk, 62), O.seq(batch * nk, 63)
    pats = [(O.round_f16(O.seq(kv * c * hd, 70 + i)), O.round_f16(O.seq(kv * c * hd, 80 + i)))
            for i, c in enumerate(caps)]
    for div in (None, LLAMA3_DIV[:hd // 2]):
        ddiv = None if div is None else gpu.upload(div)
        dq, dk, dv = gpu.upload(q), gpu.upload(k), gpu.upload(v)
        kcs = [gpu.upload_u16(p[0]) for p in pats]
        vcs = [gpu.upload_u16(p[1]) for p in pats]
        gpu.rope_cache_batched(dq, dk, dv, ddiv, heads, kv, hd, 10000.0, poss, kcs, vcs, caps)
        one = [gpu.upload(q), gpu.upload(k), gpu.upload(v)]
        kcs1 = [gpu.upload_u16(p[0]) for p in pats]
        vcs1 = [gpu.upload_u16(p[1]) for p in pats]
        for b in range(batch):
            gpu.rope_cache_f16(one, (0, b * nq), (1, b * nk), (2, b * nk), ddiv, heads, kv, hd,
                               10000.0, poss[b], kcs1[b], vcs1[b], caps[b])
        assert np.array_equal(gpu.download(dq), gpu.download(one[0]))
        assert np.array_equal(gpu.download(dk), k)      # keys are not rotated in place
        for b in range(batch):
            assert np.array_equal(gpu.download_u16(kcs[b]), gpu.download_u16(kcs1[b]))
            assert np.array_equal(gpu.download_u16(vcs[b]), gpu.download_u16(vcs1[b]))
    with pytest.raises(Exception):
        gpu.rope_cache_batched(dq, dk, dv, None, heads, kv, hd, 10000.0, [32, 0, 0, 0], kcs, vcs,
                               caps)


@pytest.mark.parametrize("transposed", [False, True])
def test_growing_a_cache_restrides_every_head(gpu, transposed):
    live, kv, hd, small, large = 5, 3, 4, 8, 16
    src = O.seq(live * kv * hd, 7)
    up = gpu.upload(src)
    grew = gpu.zeros(small * kv * hd)
    gpu.cache_append(up, 0, grew, live, kv, hd, small, 0, transposed)
    moved = gpu.zeros(large * kv * hd)
    gpu.cache_grow(grew, moved, kv, hd, small, large, live, transposed)
    direct = gpu.zeros(large * kv * hd)
    gpu.cache_append(up, 0, direct, live, kv, hd, large, 0, transposed)
    assert np.array_equal(gpu.download(moved), gpu.download(direct))
    # f16 twin
    grew16 = gpu.zeros_f16(small * kv * hd)
    gpu.cache_append_f16(up, 0, grew16, live, kv, hd, small, 0, transposed)
    moved16 = gpu.zeros_f16(large * kv * hd)
    gpu.cache_grow_f16(grew16, moved16, kv, hd, small, large, live, transposed)
    direct16 = gpu.zeros_f16(large * kv * hd)
    gpu.cache_append_f16(up, 0, direct16, live, kv, hd, large, 0, transposed)
    assert np.array_equal(gpu.download_u16(moved16), gpu.download_u16(direct16))
    want = np.zeros(large * kv * hd, np.uint16)
    O.cache_grow(gpu.download_u16(grew16), want, kv, hd, small, large, live, transposed)
    assert np.array_equal(gpu.download_u16(moved16), want)


def test_refusals(gpu):
    from ttsxabe_b200 import CacheOverrun, OddCacheCapacity, OddHeadDim, SliceOverrun

    kv, hd, small, large = 2, 4, 8, 16
    src = gpu.zeros(small * kv * hd)
    dst = gpu.zeros(large * kv * hd)
    with pytest.raises(CacheOverrun):
        gpu.cache_grow(src, dst, kv, hd, small, large, small + 1, False)
    with pytest.raises(CacheOverrun):
        gpu.cache_grow(src, gpu.zeros(small * kv * hd), kv, hd, large, small, 4, False)
    t, heads, hd8 = 2, 2, 8
    x = gpu.zeros(t * heads * hd8)
    with pytest.raises(SliceOverrun):
        gpu.rope(x, 1, t, heads, hd8, 10000.0, 0)
    with pytest.raises(OddHeadDim):
        gpu.rope(gpu.zeros(2 * 2 * 7), 0, 2, 2, 7, 10000.0, 0)
    with pytest.raises(SliceOverrun):
        gpu.cache_append(x, 1, gpu.zeros(8 * heads * hd8), t, heads, hd8, 8, 0, False)
    with pytest.raises(CacheOverrun):
        gpu.cache_append(x, 0, gpu.zeros(8 * heads * hd8), t, heads, hd8, 8, 7, False)
    with pytest.raises(OddCacheCapacity):
        gpu.cache_append_f16(x, 0, gpu.zeros_f16(7 * heads * hd8), t, heads, hd8, 7, 0, False)
    kc = gpu.zeros_f16(8 * 2 * 8)
    with pytest.raises(CacheOverrun):
        gpu.rope_cache_f16([gpu.zeros(64)], (0, 0), (0, 32), (0, 48), None, 4, 2, 8, 1e4, 8, kc,
                           kc, 8)


def test_kv_cache_grows_as_the_model_crates_do(gpu):
    """Capacity doubling with re-stride (crates/llmtie-chat/src/model.rs:714-747):
    a prompt of 300, single tokens, and a second prompt across the 1024 boundary."""
    from ttsxabe_b200 import KvCache

    kv, hd = 2, 64
    cache = KvCache(gpu, kv, hd, max_positions=8192)
    rng = np.random.default_rng(5)
    host_k = np.zeros((kv, 0, hd), np.float32)
    host_v = np.zeros((kv, 0, hd), np.float32)
    caps = []
    for n in [300] + [1] * 3 + [500] + [1] * 2 + [250]:
        k = rng.standard_normal((n, kv, hd)).astype(np.float32)
        v = rng.standard_normal((n, kv, hd)).astype(np.float32)
        cache.append(gpu.upload(k), gpu.upload(v), 0, 0, n)
        host_k = np.concatenate([host_k, k.transpose(1, 0, 2)], axis=1)
        host_v = np.concatenate([host_v, v.transpose(1, 0, 2)], axis=1)
        caps.append(cache.cap)
    assert caps == [1024] * 7 + [2048]
    assert cache.len == host_k.shape[1]
    gk = gpu.download_u16(cache.k).reshape(kv, cache.cap, hd)
    gv = gpu.download_u16(cache.v).reshape(kv, hd, cache.cap)
    assert np.array_equal(gk[:, :cache.len, :], O.round_f16(host_k).reshape(kv, -1, hd))
    assert np.array_equal(gv[:, :, :cache.len],
                          O.round_f16(host_v.transpose(0, 2, 1)).reshape(kv, hd, -1))
    assert not gk[:, cache.len:, :].any() and not gv[:, :, cache.len:].any()
    cache.truncate(10)
    assert cache.len == 10 and cache.cap == 2048
