"""Seeded random shapes through the decode and prefill entry points against the
oracle: odd lengths, ragged batches, capacities whose value rows are 16-, 8-
or only 4-byte aligned, every head grouping the entries take, the live length
anywhere inside the capacity with NaN bits poisoning what lies beyond."""
import numpy as np
import pytest

from oracle import oracle as O
from tests.helpers import (assert_close_to, assert_parity, lay_caches, normal_f16,
                           poison_f16_bits)

pytestmark = pytest.mark.gpu

GROUPS_128 = [(4, 4), (8, 2), (32, 8), (12, 4), (4, 1), (6, 3)]
GROUPS_64 = [(20, 20), (14, 2), (16, 2), (6, 6), (12, 4), (8, 1)]


def _capacity(rng, tk, step):
    return int(-(-(tk + int(rng.integers(0, 40))) // step) * step)


@pytest.mark.parametrize("seed", range(48))
def test_random_decode_cases(gpu, seed):
    from ttsxabe_b200 import DecodeScratch

    rng = np.random.default_rng(1000 + seed)
    hd = int(rng.choice([64, 128]))
    heads, kv = (GROUPS_128 if hd == 128 else GROUPS_64)[int(rng.integers(0, 6))]
    tk = int(rng.choice([1, 2, 31, 127, 128, 129, 500, 1027, 2999, 6000])) + int(rng.integers(0, 3))
    cap = _capacity(rng, tk, int(rng.choice([4, 8, 8, 16])))
    scale_q = bool(rng.integers(0, 2))
    scale = float(np.float32(hd) ** np.float32(-0.5))
    q = normal_f16(rng, heads * hd)
    kc, vc = lay_caches(normal_f16(rng, kv * tk * hd), normal_f16(rng, kv * tk * hd), kv, tk, hd,
                        cap)
    kbits = poison_f16_bits(O.round_f16(kc), kv, tk, hd, cap, False)
    vbits = poison_f16_bits(O.round_f16(vc), kv, tk, hd, cap, True)
    scratch = DecodeScratch()
    got = gpu.download(gpu.attn_decode_f16(gpu.upload(q), gpu.upload_u16(kbits),
                                           gpu.upload_u16(vbits), heads, kv, hd, tk, cap, scale,
                                           scale_q, scratch))
    want = O.decode_f64(q, O.round_f16(kc), O.round_f16(vc), heads, kv, hd, 0, tk, cap, scale,
                        scale_q)
    name = f"decode {heads}/{kv} hd {hd} tk {tk} cap {cap} scale_q {scale_q}"
    assert_close_to(name, want, got, 2e-5)
    assert_parity(name, want, got)


@pytest.mark.parametrize("seed", range(24))
def test_random_ragged_decode_batches(gpu, seed):
    from ttsxabe_b200 import DecodeScratch

    rng = np.random.default_rng(2000 + seed)
    hd = int(rng.choice([64, 128]))
    heads, kv = (GROUPS_128 if hd == 128 else GROUPS_64)[int(rng.integers(0, 6))]
    batch = int(rng.integers(1, 7))
    tks = [int(rng.integers(1, 2500)) for _ in range(batch)]
    if seed % 3 == 2:
        # every sequence the same length: the cuts that give a pair a cluster or a block
        batch = int(rng.choice([1, 2, 4, 12, 16]))
        tks = [int(rng.choice([130, 700, 1500, 2300]))] * batch
    step = 4 if seed % 4 == 1 else 8     # value rows 8-byte or 16-byte aligned
    caps = [_capacity(rng, t, step) for t in tks]
    scale = float(np.float32(hd) ** np.float32(-0.5))
    q = normal_f16(rng, batch * heads * hd)
    ks, vs, host = [], [], []
    for t, c in zip(tks, caps):
        kc, vc = lay_caches(normal_f16(rng, kv * t * hd), normal_f16(rng, kv * t * hd), kv, t, hd, c)
        host.append((O.round_f16(kc), O.round_f16(vc)))
        ks.append(gpu.upload_u16(poison_f16_bits(host[-1][0], kv, t, hd, c, False)))
        vs.append(gpu.upload_u16(poison_f16_bits(host[-1][1], kv, t, hd, c, True)))
    got = gpu.download(gpu.decode_batched(gpu.upload(q), ks, vs, tks, caps, heads, kv, hd, scale,
                                          False, DecodeScratch())).reshape(batch, -1)
    for b in range(batch):
        want = O.decode_f64(q.reshape(batch, -1)[b], host[b][0], host[b][1], heads, kv, hd, 0,
                            tks[b], caps[b], scale, False)
        assert_close_to(f"batch {tks} sequence {b}", want, got[b], 2e-5)


@pytest.mark.parametrize("seed", range(36))
def test_random_prefill_cases(gpu, seed):
    rng = np.random.default_rng(3000 + seed)
    half = bool(rng.integers(0, 2))
    hd = 128 if half else int(rng.choice([64, 128]))   # f16 caches: 128 only, as the reference
    heads, kv = (GROUPS_128 if hd == 128 else GROUPS_64)[int(rng.integers(0, 6))]
    causal = bool(rng.integers(0, 4)) or half
    tq = int(rng.choice([1, 7, 64, 127, 128, 129, 200, 300])) + int(rng.integers(0, 2))
    past = int(rng.choice([0, 0, 1, 33, 128, 200]))
    tk = past + tq
    cap = _capacity(rng, tk, int(rng.choice([2, 8])))
    scale = float(np.float32(hd) ** np.float32(-0.5))
    q = normal_f16(rng, tq * heads * hd)
    kc, vc = lay_caches(normal_f16(rng, kv * tk * hd), normal_f16(rng, kv * tk * hd), kv, tk, hd,
                        cap)
    if half:
        out = gpu.flash_attn_f16(gpu.upload(q), gpu.upload_f16(kc), gpu.upload_f16(vc), tq, past,
                                 heads, kv, hd, cap, scale, causal)
    else:
        out = gpu.flash_attn(gpu.upload(q), gpu.upload(kc), gpu.upload(vc), tq, past, heads, kv, hd,
                             cap, scale, causal)
    want = O.prefill(q, kc, vc, tq, past, heads, kv, hd, cap, scale, causal)
    assert_parity(f"prefill {heads}/{kv} hd {hd} tq {tq} past {past} cap {cap} causal {causal} "
                  f"f16 {half}", want, gpu.download(out))


@pytest.mark.parametrize("seed", range(10))
def test_random_ragged_prefill_batches(gpu, seed):
    """llmtie_prefill_varlen over a random batch - empty sequences, single
    tokens, prompts on a kept prefix, more sequences than one attention launch
    carries - gives every sequence the bits it gets when prefilled alone, in
    the output and in both caches; one sequence is held to the oracle."""
    rng = np.random.default_rng(4000 + seed)
    heads, kv = GROUPS_128[int(rng.integers(0, 6))]
    hd, cap = 128, 512
    batch = int(rng.choice([1, 2, 3, 5, 9, 12]))
    lens = [int(rng.choice([0, 1, 2, 17, 64, 127, 128, 129, 200, 300])) for _ in range(batch)]
    pasts = [int(rng.choice([0, 0, 1, 33, 128, 200])) for _ in range(batch)]
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    total = int(cu[-1])
    scale = float(np.float32(hd) ** np.float32(-0.5))
    q = normal_f16(rng, max(total, 1) * heads * hd)
    k = normal_f16(rng, max(total, 1) * kv * hd)
    v = normal_f16(rng, max(total, 1) * kv * hd)
    olds = [(O.round_f16(normal_f16(rng, kv * cap * hd)), O.round_f16(normal_f16(rng, kv * cap * hd)))
            for _ in range(batch)]
    kcs = [gpu.upload_u16(a) for a, _ in olds]
    vcs = [gpu.upload_u16(b) for _, b in olds]
    got = gpu.download(gpu.prefill_varlen(gpu.upload(q), gpu.upload(k), gpu.upload(v), cu, kcs, vcs,
                                          pasts, [cap] * batch, None, heads, kv, hd, 10000.0, scale))
    got = got[:total * heads * hd].reshape(total, -1)
    checked = False
    for b in range(batch):
        n, r0 = lens[b], int(cu[b])
        if n == 0:
            assert np.array_equal(gpu.download_u16(kcs[b]), olds[b][0]), f"seed {seed} sequence {b}"
            continue
        kc1, vc1 = gpu.upload_u16(olds[b][0]), gpu.upload_u16(olds[b][1])
        rows = lambda x, w: gpu.upload(x[:total * w].reshape(total, w)[r0:r0 + n].reshape(-1))
        alone = gpu.download(gpu.prefill_varlen(rows(q, heads * hd), rows(k, kv * hd), rows(v, kv * hd),
                                                [0, n], [kc1], [vc1], [pasts[b]], [cap], None, heads,
                                                kv, hd, 10000.0, scale))
        name = f"seed {seed} lens {lens} pasts {pasts} sequence {b}"
        assert np.array_equal(got[r0:r0 + n].reshape(-1), alone), name
        assert np.array_equal(gpu.download_u16(kcs[b]), gpu.download_u16(kc1)), name
        assert np.array_equal(gpu.download_u16(vcs[b]), gpu.download_u16(vc1)), name
        if not checked:
            checked = True
            qr = O.rope(q[:total * heads * hd].reshape(total, -1)[r0:r0 + n].reshape(-1), n, heads, hd,
                        10000.0, pasts[b])
            want = O.prefill(qr, gpu.download_u16(kc1), gpu.download_u16(vc1), n, pasts[b], heads, kv,
                             hd, cap, scale, True)
            assert_parity(name + " (oracle)", want, alone)


@pytest.mark.parametrize("seed", range(10))
def test_random_encoder_rows_and_cross_attention(gpu, seed):
    """The two Whisper entries at random sizes: flash_attn_rows over t frames
    (one frame, either side of a 128-row tile, ragged last tiles) against the
    oracle's non-causal prefill; cross-attention of n query rows over tk keys
    in caches of a capacity whose value rows are 16- or only 8-byte aligned,
    against the oracle's decode row by row."""
    from ttsxabe_b200 import DecodeScratch

    rng = np.random.default_rng(5000 + seed)
    heads, hd = int(rng.choice([4, 6, 20])), 64
    d = heads * hd
    t = int(rng.choice([1, 7, 127, 128, 129, 300, 700]))
    qkv = normal_f16(rng, t * 3 * d).reshape(t, 3 * d)
    got = O.widen_f16(gpu.download_u16(gpu.flash_attn_rows(gpu.upload(qkv), t, heads, hd, 0.125)))
    kc, vc = lay_caches(qkv[:, d:2 * d].reshape(t, heads, hd).transpose(1, 0, 2),
                        qkv[:, 2 * d:].reshape(t, heads, hd).transpose(1, 0, 2), heads, t, hd, t)
    want = O.prefill(np.ascontiguousarray(qkv[:, :d]), kc, vc, t, 0, heads, heads, hd, t, 0.125,
                     False, scale_q=True, fast=True)
    assert np.abs(want - got).max() <= 2e-3 + 2.0 ** -11 * np.abs(want).max(), f"rows t {t} heads {heads}"

    n = int(rng.choice([1, 2, 5, 8, 13, 32]))
    tk = int(rng.choice([1, 31, 130, 1000, 1500]))
    cap = _capacity(rng, tk, int(rng.choice([4, 8])))
    q = normal_f16(rng, n * d)
    kc, vc = lay_caches(normal_f16(rng, heads * tk * hd), normal_f16(rng, heads * tk * hd), heads, tk,
                        hd, cap)
    kbits = poison_f16_bits(O.round_f16(kc), heads, tk, hd, cap, False)
    vbits = poison_f16_bits(O.round_f16(vc), heads, tk, hd, cap, True)
    out = gpu.download(gpu.cross_attn(gpu.upload(q), gpu.upload_u16(kbits), gpu.upload_u16(vbits), n,
                                      heads, hd, tk, cap, 0.125, DecodeScratch())).reshape(n, -1)
    for r in range(n):
        want = O.decode_f64(q.reshape(n, -1)[r], O.round_f16(kc), O.round_f16(vc), heads, heads, hd, 0,
                            tk, cap, 0.125, True)
        assert_close_to(f"cross n {n} tk {tk} cap {cap} row {r}", want, out[r], 2e-5)


@pytest.mark.parametrize("seed", range(12))
def test_random_decode_off_f32_caches(gpu, seed):
    """attn_decode over f32 caches (head_dim 64): one key to a few thousand,
    so one block a head, a few, and eight of several chunks each; twice through
    one scratch; NaN in the capacity past the live keys."""
    from ttsxabe_b200 import DecodeScratch

    rng = np.random.default_rng(6000 + seed)
    heads, kv = GROUPS_64[int(rng.integers(0, 6))]
    hd = 64
    tk = int(rng.choice([1, 2, 63, 64, 65, 200, 448, 513, 1500, 4000])) + int(rng.integers(0, 2))
    cap = _capacity(rng, tk, 2)
    scale_q = bool(rng.integers(0, 2))
    q = normal_f16(rng, heads * hd)
    kc, vc = lay_caches(normal_f16(rng, kv * tk * hd), normal_f16(rng, kv * tk * hd), kv, tk, hd, cap,
                        fill=np.nan)
    want = O.decode_f32(q, np.nan_to_num(kc), np.nan_to_num(vc), heads, kv, hd, tk, cap, 0.125, scale_q)
    dq, dk, dv = gpu.upload(q), gpu.upload(kc), gpu.upload(vc)
    scratch = DecodeScratch()
    a = gpu.download(gpu.attn_decode(dq, dk, dv, heads, kv, hd, tk, cap, 0.125, scale_q, scratch))
    b = gpu.download(gpu.attn_decode(dq, dk, dv, heads, kv, hd, tk, cap, 0.125, scale_q, scratch))
    name = f"f32 decode {heads}/{kv} tk {tk} cap {cap} scale_q {scale_q}"
    assert np.array_equal(a, b), name
    assert_close_to(name, want, a, 2e-5)
