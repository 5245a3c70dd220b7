"""Decode attention through the C ABI against the CPU oracle.

The cases, salts and the 2e-5-of-full-scale bound are those of the
reference's `the_fused_decode_attention_matches_the_chain`
(crates/llmtie-cuda/tests/kernels.rs:2782-2932).
"""
import numpy as np
import pytest

from oracle import oracle as O
from tests.helpers import assert_close_to, assert_parity, normal_f16, poison_f16_bits

pytestmark = pytest.mark.gpu

# (heads, kv_heads, hd, tk, cap, f16 cache, scale on the query)
CASES = [
    (8, 2, 128, 1, 256, True, False),
    (8, 2, 128, 63, 256, True, False),
    (8, 2, 128, 64, 256, True, False),
    (8, 2, 128, 65, 256, True, False),
    (8, 2, 128, 200, 256, True, False),
    (8, 2, 128, 256, 256, True, False),
    (4, 4, 128, 130, 512, True, False),
    (6, 6, 64, 1500, 1500, True, True),
    (6, 6, 64, 1499, 1500, True, True),
    (6, 6, 64, 37, 448, False, True),
    (6, 6, 64, 129, 448, False, True),
    (6, 6, 64, 448, 448, False, True),
    (4, 2, 128, 16500, 16512, True, False),
    (32, 8, 128, 4096, 4096, True, False),
    (32, 8, 128, 8192, 8192, True, False),
    (32, 8, 128, 7777, 8192, True, False),
    (40, 40, 128, 1500, 1536, True, False),
    (20, 20, 64, 1500, 1500, True, True),
    (8, 8, 64, 5000, 5056, False, True),
    # groups that are not powers of two, and the widest a 64-wide head takes:
    # the speech LM of crates/llmtie-cosy (14 query / 2 KV heads: group 7,
    # src/llm.rs:448-475) and its neighbours
    (14, 2, 64, 700, 1024, True, False),
    (16, 2, 64, 333, 512, True, False),
    (12, 4, 128, 500, 512, True, False),
    (14, 2, 64, 9000, 9004, True, True),
    # the first keys of a conversation: one key, and either side of a 32-key block
    (32, 8, 128, 1, 256, True, False),
    (32, 8, 128, 2, 256, True, False),
    (32, 8, 128, 31, 256, True, False),
    (32, 8, 128, 33, 256, True, False),
    (20, 20, 64, 1, 448, True, True),
    (20, 20, 64, 1, 448, False, True),
    (20, 20, 64, 65, 448, False, True),
]


@pytest.mark.parametrize("i,case", list(enumerate(CASES)))
def test_fused_decode_matches_the_chain(gpu, i, case):
    from ttsxabe_b200 import DecodeScratch

    heads, kv, hd, tk, cap, half, scale_q = case
    salt = 300 + 3 * i
    q = O.seq(heads * hd, salt)
    k0 = O.seq(kv * cap * hd, salt + 1)
    v0 = O.seq(kv * hd * cap, salt + 2)
    scale = 0.11
    scratch = DecodeScratch()
    dq = gpu.upload(q)
    name = f"attn_decode heads {heads} kv {kv} hd {hd} tk {tk} f16 {half}"
    if half:
        k, v = O.through_f16(k0), O.through_f16(v0)
        want = O.decode_f32(q, k, v, heads, kv, hd, tk, cap, scale, scale_q)
        dk, dv = gpu.upload_f16(k0), gpu.upload_f16(v0)
        first = gpu.attn_decode_f16(dq, dk, dv, heads, kv, hd, tk, cap, scale, scale_q, scratch)
        again = gpu.attn_decode_f16(dq, dk, dv, heads, kv, hd, tk, cap, scale, scale_q, scratch)
    else:
        want = O.decode_f32(q, k0, v0, heads, kv, hd, tk, cap, scale, scale_q)
        dk, dv = gpu.upload(k0), gpu.upload(v0)
        first = gpu.attn_decode(dq, dk, dv, heads, kv, hd, tk, cap, scale, scale_q, scratch)
        again = gpu.attn_decode(dq, dk, dv, heads, kv, hd, tk, cap, scale, scale_q, scratch)
    a, b = gpu.download(first), gpu.download(again)
    # twice through one scratch: a counter left dirty would merge early or never
    assert np.array_equal(a, b), f"{name}: not reproducible through one scratch"
    assert_close_to(name, want, a, 2e-5)
    if half:
        tight = O.decode_f64(q, O.round_f16(k0), O.round_f16(v0), heads, kv, hd, 0, tk, cap,
                             scale, scale_q)
        assert_close_to(name + " (f64 oracle)", tight, a, 2e-5)


def test_decode_refusals(gpu):
    """The shapes it refuses, by name rather than by wrong answer
    (crates/llmtie-cuda/tests/kernels.rs:2910-2932)."""
    from ttsxabe_b200 import CacheOverrun, DecodeScratch, UnsupportedAttention

    scratch = DecodeScratch()
    dq = gpu.upload(O.seq(8 * 128, 1))
    dk = gpu.upload_f16(O.seq(2 * 256 * 128, 2))
    with pytest.raises(UnsupportedAttention):   # a head width it is not instantiated at
        gpu.attn_decode_f16(dq, dk, dk, 8, 2, 96, 10, 256, 1.0, False, scratch)
    with pytest.raises(CacheOverrun):           # more keys than the cache holds
        gpu.attn_decode_f16(dq, dk, dk, 8, 2, 128, 257, 256, 1.0, False, scratch)
    with pytest.raises(CacheOverrun):           # no keys at all
        gpu.attn_decode_f16(dq, dk, dk, 8, 2, 128, 0, 256, 1.0, False, scratch)
    with pytest.raises(UnsupportedAttention):   # a group wider than the kernel carries
        gpu.attn_decode_f16(dq, dk, dk, 10, 2, 128, 10, 256, 1.0, False, scratch)


def test_row_variant_equals_single(gpu):
    """`attn_decode_f16_q_row` writes row `row` of a shared output and reads q
    at an offset; same kernel, same bits (kernels.rs tests :3339-3440)."""
    from ttsxabe_b200 import DecodeScratch

    heads, kv, hd, tk, cap = 32, 8, 128, 777, 1024
    rows = 3
    scratch = DecodeScratch()
    qs = O.seq(rows * heads * hd, 11)
    dq_all = gpu.upload(qs)
    dk = gpu.upload_f16(O.seq(kv * cap * hd, 12))
    dv = gpu.upload_f16(O.seq(kv * cap * hd, 13))
    out = gpu.zeros(rows * heads * hd)
    for r in range(rows):
        gpu.attn_decode_f16_row(dq_all, r * heads * hd, dk, dv, heads, kv, hd, tk, cap, 0.09,
                                False, scratch, out, r)
    got = gpu.download(out).reshape(rows, -1)
    for r in range(rows):
        dq = gpu.upload(qs[r * heads * hd:(r + 1) * heads * hd])
        single = gpu.download(
            gpu.attn_decode_f16(dq, dk, dv, heads, kv, hd, tk, cap, 0.09, False, scratch))
        assert np.array_equal(single, got[r])


@pytest.mark.parametrize("batch", [1, 2, 4, 16])
def test_config3_batched_decode(gpu, batch):
    """BASELINE config 3: one query per sequence, context seeded uniform in
    [2048, 4096], 32 Q / 8 KV heads, hd 128, f16 cache and N(0,1) query, RoPE
    on the query at position = context length; bar max-abs 2e-3, rel-L2 1e-3.
    (Batches 2 and 4 are few and short enough for the cut that gives each
    pair a cluster of blocks, with sequences of unequal length.)"""
    from ttsxabe_b200 import DecodeScratch

    heads, kv, hd = 32, 8, 128
    rng = np.random.default_rng(3000 + batch)
    tks = rng.integers(2048, 4097, size=batch)
    scale = float(np.float32(hd) ** np.float32(-0.5))
    scratch = DecodeScratch()
    ks, vs, caps, wants, qs = [], [], [], [], []
    for b in range(batch):
        tk = int(tks[b])
        cap = 4096
        q = normal_f16(rng, heads * hd)
        q = O.rope(q, 1, heads, hd, 10000.0, tk)
        kb = O.round_f16(normal_f16(rng, kv * cap * hd))
        vb = O.round_f16(normal_f16(rng, kv * hd * cap))
        # what lies past the live keys must not matter: poison it
        kb = poison_f16_bits(kb, kv, tk, hd, cap, False)
        vb = poison_f16_bits(vb, kv, tk, hd, cap, True)
        wants.append(O.decode_f64(q, kb, vb, heads, kv, hd, 0, tk, cap, scale, False))
        ks.append(gpu.upload_u16(kb))
        vs.append(gpu.upload_u16(vb))
        caps.append(cap)
        qs.append(q)
    dq = gpu.upload(np.concatenate(qs))
    out = gpu.decode_batched(dq, ks, vs, tks, caps, heads, kv, hd, scale, False, scratch)
    got = gpu.download(out).reshape(batch, -1)
    for b in range(batch):
        assert_parity(f"config 3 batch {batch} seq {b} tk {tks[b]}", wants[b], got[b])
        # the reference's loop of single-sequence calls gives the same bits
    single = gpu.download(gpu.attn_decode_f16(gpu.upload(qs[0]), ks[0], vs[0], heads, kv, hd,
                                              int(tks[0]), caps[0], scale, False, scratch))
    assert_parity("single vs oracle", wants[0], single)


def test_partial_triples_merge_to_the_whole(gpu):
    """Splitting the keys over `parts` caches, taking un-normalised
    (o, m, l) from each and merging equals decoding the whole cache: the
    algebra the multi-GPU path rests on (kernels.rs:5836-5879)."""
    from ttsxabe_b200 import DecodeScratch

    heads, kv, hd, parts, per = 32, 8, 128, 4, 1024
    rng = np.random.default_rng(77)
    scale = float(np.float32(hd) ** np.float32(-0.5))
    q = normal_f16(rng, heads * hd)
    kv_all = normal_f16(rng, kv * parts * per * hd).reshape(kv, parts * per, hd)
    vv_all = normal_f16(rng, kv * parts * per * hd).reshape(kv, parts * per, hd)
    scratch = DecodeScratch()
    dq = gpu.upload(q)
    bufs = []
    for p in range(parts):
        kc = np.ascontiguousarray(kv_all[:, p * per:(p + 1) * per, :])
        vc = np.ascontiguousarray(vv_all[:, p * per:(p + 1) * per, :].transpose(0, 2, 1))
        dk, dv = gpu.upload_u16(O.round_f16(kc)), gpu.upload_u16(O.round_f16(vc))
        part = gpu.decode_batched(dq, [dk], [dv], [per], [per], heads, kv, hd, scale, False,
                                  scratch, partial=True)
        trip = gpu.download(part).reshape(heads, hd + 2)
        _, o_un, m, l = O.decode_f64(q, O.round_f16(kc), O.round_f16(vc), heads, kv, hd, 0, per,
                                     per, scale, False, triple=True)
        assert_close_to("partial m", m, trip[:, hd], 1e-5)
        assert_close_to("partial l", l, trip[:, hd + 1], 1e-4)
        assert_close_to("partial o", o_un, trip[:, :hd].reshape(-1), 1e-4)
        bufs.append(part)
    import torch

    with torch.cuda.stream(gpu.stream):
        gathered = torch.cat(bufs)
    merged = gpu.download(gpu.lse_merge(gathered, parts, heads, hd))
    kc = np.ascontiguousarray(kv_all)
    vc = np.ascontiguousarray(vv_all.transpose(0, 2, 1))
    want = O.decode_f64(q, O.round_f16(kc), O.round_f16(vc), heads, kv, hd, 0, parts * per,
                        parts * per, scale, False)
    assert_parity("merged partials", want, merged)
    assert_close_to("merged partials", want, merged, 2e-5)


@pytest.mark.parametrize("mode", ["push", "pairs", "push-clusters", "push-wide-clusters"])
def test_peer_push_exchange_on_one_device(gpu, mode):
    """The fused multi-GPU exchange, with both "ranks" on one device: each rank
    decodes its slice of the keys and pushes its triples into every rank's
    gather buffer (here: two buffers in the same memory), then each rank's
    waiting merge runs. The kernels are enqueued one after another on one
    stream, so every flag a merge waits for was raised by a kernel that has
    already finished (or, for the merge launched as a programmatic dependent
    in "pairs" mode, by a kernel all of whose blocks have at least started).
    "push" raises one flag a rank, "pairs" one a (sequence, KV head) pair. Two
    steps, to use both gather buffers."""
    import torch

    from ttsxabe_b200 import DecodeScratch, Exchange

    heads, kv, hd, batch, world = 32, 8, 128, 3, 2
    per = [1000, 1536]                     # keys held by rank 0 and rank 1
    caps = [1024, 1536]
    if mode == "push-clusters":
        # 64 pairs of equal length a rank: the launch that goes pair by cluster
        batch, per, caps, mode = 8, [2048, 2304], [2048, 2304], "push"
    if mode == "push-wide-clusters":
        # 8 short pairs a rank: eight blocks a pair, the leading one fetches and pushes
        batch, per, caps, mode = 1, [3000, 2944], [3008, 2944], "push"
    rows = batch * heads
    rng = np.random.default_rng(91)
    scale = float(np.float32(hd) ** np.float32(-0.5))
    kfull = [normal_f16(rng, kv * sum(per) * hd).reshape(kv, sum(per), hd) for _ in range(batch)]
    vfull = [normal_f16(rng, kv * sum(per) * hd).reshape(kv, sum(per), hd) for _ in range(batch)]
    with torch.cuda.stream(gpu.stream):
        gathers = [torch.zeros(2 * world * rows * (hd + 2), dtype=torch.float32, device=gpu.device)
                   for _ in range(world)]
        flags = [torch.zeros(64, dtype=torch.int32, device=gpu.device) for _ in range(world)]
        steps = [torch.zeros(1, dtype=torch.int32, device=gpu.device) for _ in range(world)]
        msteps = [torch.zeros(2, dtype=torch.int32, device=gpu.device) for _ in range(world)]
        pflags = [torch.zeros(batch * kv * world, dtype=torch.int32, device=gpu.device)
                  for _ in range(world)]
    xchs = [Exchange(world, r, [g_.data_ptr() for g_ in gathers], [f.data_ptr() for f in flags],
                     steps[r].data_ptr(), [f.data_ptr() for f in pflags]) for r in range(world)]
    caches = []
    for r in range(world):
        t0 = sum(per[:r])
        ks, vs = [], []
        for b in range(batch):
            kc = np.zeros((kv, caps[r], hd), np.float32)
            vc = np.zeros((kv, hd, caps[r]), np.float32)
            kc[:, :per[r], :] = kfull[b][:, t0:t0 + per[r], :]
            vc[:, :, :per[r]] = vfull[b][:, t0:t0 + per[r], :].transpose(0, 2, 1)
            ks.append(gpu.upload_u16(O.round_f16(kc)))
            vs.append(gpu.upload_u16(O.round_f16(vc)))
        caches.append((ks, vs))
    scratch = [DecodeScratch() for _ in range(world)]
    for step in range(2):
        q = normal_f16(rng, batch * heads * hd)
        dq = gpu.upload(q)
        for r in range(world):
            push = gpu.decode_batched_push if mode == "push" else gpu.decode_batched_signal
            push(dq, caches[r][0], caches[r][1], [per[r]] * batch, [caps[r]] * batch, heads, kv, hd,
                 scale, False, scratch[r], xchs[r])
        if mode == "push":
            outs = [gpu.download(gpu.lse_merge_wait(xchs[r], rows, hd)) for r in range(world)]
        else:
            outs = [gpu.download(gpu.lse_merge_pairs(xchs[r], msteps[r], rows, heads // kv, hd))
                    for r in range(world)]
            assert all(int(m[0].item()) == step + 1 and int(m[1].item()) == 0 for m in msteps)
        assert np.array_equal(outs[0], outs[1]), "both ranks must merge to the same context"
        for b in range(batch):
            kc = np.ascontiguousarray(kfull[b])
            vc = np.ascontiguousarray(vfull[b].transpose(0, 2, 1))
            want = O.decode_f64(q.reshape(batch, -1)[b], O.round_f16(kc), O.round_f16(vc), heads,
                                kv, hd, 0, sum(per), sum(per), scale, False)
            assert_parity(f"peer push step {step} sequence {b}", want,
                          outs[0].reshape(batch, -1)[b])
            assert_close_to(f"peer push step {step} sequence {b}", want,
                            outs[0].reshape(batch, -1)[b], 2e-5)
        assert int(steps[0].item()) == step + 1 and int(steps[1].item()) == step + 1


@pytest.mark.parametrize("shape", [
    # heads, kv, hd, batch, contexts
    (32, 8, 128, 3, [1000, 4096, 37]),
    (128, 128, 64, 32, [100] * 32),      # ~27 pairs a block: more than a block's list holds
])
def test_fused_exchange_with_a_world_of_one(gpu, shape):
    """The one-kernel sharded step with a single rank: the kernel pushes its
    triples into its own gather buffer, raises its own pair flags, waits for
    them and merges. Nothing waits on another launch. Must equal the plain
    decode of the same caches; two steps, to use both gather buffers."""
    import torch

    from ttsxabe_b200 import DecodeScratch, Exchange

    heads, kv, hd, batch, tks = shape
    rows = batch * heads
    rng = np.random.default_rng(17)
    scale = float(np.float32(hd) ** np.float32(-0.5))
    caps = [-(-t // 8) * 8 for t in tks]
    ks = [gpu.upload_u16(O.round_f16(normal_f16(rng, kv * c * hd))) for c in caps]
    vs = [gpu.upload_u16(O.round_f16(normal_f16(rng, kv * c * hd))) for c in caps]
    with torch.cuda.stream(gpu.stream):
        gather = torch.zeros(2 * rows * (hd + 2), dtype=torch.float32, device=gpu.device)
        flags = torch.zeros(64, dtype=torch.int32, device=gpu.device)
        pflags = torch.zeros(batch * kv, dtype=torch.int32, device=gpu.device)
        step = torch.zeros(1, dtype=torch.int32, device=gpu.device)
    xch = Exchange(1, 0, [gather.data_ptr()], [flags.data_ptr()], step.data_ptr(),
                   [pflags.data_ptr()])
    scratch, plain = DecodeScratch(), DecodeScratch()
    for s in range(2):
        dq = gpu.upload(normal_f16(rng, batch * heads * hd))
        got = gpu.download(gpu.decode_batched_fused(dq, ks, vs, tks, caps, heads, kv, hd, scale,
                                                    False, scratch, xch))
        want = gpu.download(gpu.decode_batched(dq, ks, vs, tks, caps, heads, kv, hd, scale,
                                               False, plain))
        gpu.synchronize()
        assert_close_to(f"fused step {s}", want, got, 1e-5)
        assert int(step.item()) == s + 1
        assert int(pflags.min().item()) == s + 1


@pytest.mark.parametrize("shape", [
    # the reference's three (tests/kernels.rs:2072-2130), then a capacity whose
    # value rows are only 8-byte aligned (the register-fed kernel) and a long
    # context cut over many blocks
    (8, 2, 128, 40, 64), (8, 2, 128, 1000, 1024), (4, 4, 64, 300, 512),
    (20, 20, 64, 1500, 1500), (32, 8, 128, 40000, 40960),
    # few short pairs: clusters of eight blocks (and of four at head_dim 64), whose leading
    # block writes the twin
    (32, 8, 128, 3000, 3008), (20, 20, 64, 1500, 1504),
])
def test_the_decode_twin_is_the_quantiser_over_its_output(gpu, shape):
    """attn_decode_f16_q: the context is bit for bit what attn_decode_f16
    gives, and the int8 twin is quantize_q8 over that context, held at exact
    equality as the reference holds it (the group maximum associates)."""
    from ttsxabe_b200 import DecodeScratch

    heads, kv, hd, tk, cap = shape
    q = O.seq(heads * hd, 61)
    dk = gpu.upload_f16(O.seq(kv * cap * hd, 62))
    dv = gpu.upload_f16(O.seq(kv * cap * hd, 63))
    dq = gpu.upload(q)
    scale = float(np.float32(hd) ** np.float32(-0.5))
    scratch = DecodeScratch()
    plain = gpu.download(gpu.attn_decode_f16(dq, dk, dv, heads, kv, hd, tk, cap, scale, True,
                                             scratch))
    out, (codes, scales) = gpu.attn_decode_f16_q(dq, dk, dv, heads, kv, hd, tk, cap, scale, True,
                                                 scratch)
    out = gpu.download(out)
    assert np.array_equal(plain, out), "the context differs with the twin asked for"
    want_c, want_s = O.quantize_q8(out)
    assert np.array_equal(codes.cpu().numpy(), want_c)
    assert np.array_equal(scales.cpu().numpy(), want_s)


def test_the_twin_row_variant_fills_one_row_and_refuses_short_buffers(gpu):
    from ttsxabe_b200 import DecodeScratch, SliceOverrun

    heads, kv, hd, tk, cap, rows = 8, 2, 128, 300, 512, 3
    n = heads * hd
    q = O.seq(rows * n, 64)
    dk = gpu.upload_f16(O.seq(kv * cap * hd, 65))
    dv = gpu.upload_f16(O.seq(kv * cap * hd, 66))
    dq = gpu.upload(q)
    scale = float(np.float32(hd) ** np.float32(-0.5))
    scratch = DecodeScratch()
    out = gpu.zeros(rows * n)
    twin = gpu.q8_zeros(rows, n)
    gpu.attn_decode_f16_q_row(dq, n, dk, dv, heads, kv, hd, tk, cap, scale, False, scratch, out,
                              twin, 1)
    gpu.synchronize()
    got = gpu.download(out).reshape(rows, n)
    codes = twin[0].cpu().numpy().reshape(rows, n)
    scales = twin[1].cpu().numpy().reshape(rows, n // 32)
    assert not got[0].any() and not got[2].any() and got[1].any()
    assert not codes[0].any() and not codes[2].any() and not scales[0].any() and not scales[2].any()
    want_c, want_s = O.quantize_q8(got[1])
    assert np.array_equal(codes[1], want_c) and np.array_equal(scales[1], want_s)
    short = gpu.q8_zeros(1, n)
    with pytest.raises(SliceOverrun):
        gpu.attn_decode_f16_q_row(dq, n, dk, dv, heads, kv, hd, tk, cap, scale, False, scratch, out,
                                  short, 1)


def test_one_scratch_through_aligned_and_unaligned_launches(gpu):
    """A scratch keeps the tensor maps of the caches it has seen. A cache with
    16-byte aligned value rows that is first decoded beside one whose rows are
    only 8-byte aligned (no value map is made for that launch) must still get
    its value map when it is decoded alone afterwards; and the other way
    round."""
    from ttsxabe_b200 import DecodeScratch

    heads, kv, hd = 20, 20, 64
    rng = np.random.default_rng(5)
    caps, tks = [1504, 1500], [1400, 1500]
    q = normal_f16(rng, 2 * heads * hd)
    kb = [O.round_f16(normal_f16(rng, kv * c * hd)) for c in caps]
    vb = [O.round_f16(normal_f16(rng, kv * c * hd)) for c in caps]
    ks, vs = [gpu.upload_u16(x) for x in kb], [gpu.upload_u16(x) for x in vb]
    want = [O.decode_f64(q.reshape(2, -1)[i], kb[i], vb[i], heads, kv, hd, 0, tks[i], caps[i], 0.125,
                         True) for i in range(2)]
    scratch = DecodeScratch()
    dq = gpu.upload(q)
    both = gpu.download(gpu.decode_batched(dq, ks, vs, tks, caps, heads, kv, hd, 0.125, True,
                                           scratch)).reshape(2, -1)
    for i in range(2):
        assert_close_to(f"together, sequence {i}", want[i], both[i], 2e-5)
    for i in (0, 1, 0):
        one = gpu.download(gpu.decode_batched(gpu.upload(q.reshape(2, -1)[i]), [ks[i]], [vs[i]],
                                              [tks[i]], [caps[i]], heads, kv, hd, 0.125, True, scratch))
        assert_close_to(f"alone, sequence {i}", want[i], one, 2e-5)


@pytest.mark.parametrize("shape", [
    # heads, kv, hd, batch, keys, capacity: 64 or 72 pairs of equal length
    (32, 8, 128, 8, 3000, 3072), (64, 64, 64, 1, 2500, 2560), (36, 9, 128, 8, 2049, 2056),
    # a few short pairs: eight blocks a pair (8 pairs of 24 units), four (16 of 13, 32 of 20,
    # 10 of 12 at head_dim 64), a pair count that leaves eight too few units a block
    (32, 8, 128, 1, 3000, 3072), (32, 8, 128, 2, 1600, 1600), (32, 8, 128, 4, 2500, 2560),
    (20, 10, 64, 1, 1500, 1504), (32, 8, 128, 1, 2049, 2056),
])
def test_pairs_cut_over_clusters(gpu, shape):
    """When the (sequence, KV head) pairs of a launch are all the same length
    and two blocks a pair nearly fill the device - or the pairs are few and
    short, and four or eight blocks a pair fit - each pair goes to one
    thread-block cluster whose blocks merge through distributed shared
    memory. Same answers as ever: the f64 oracle at the reference's bar, the
    same bits on a second call, and poison in the unused capacity ignored."""
    from ttsxabe_b200 import DecodeScratch

    heads, kv, hd, batch, tk, cap = shape
    rng = np.random.default_rng(heads + tk)
    scale = float(np.float32(hd) ** np.float32(-0.5))
    q = normal_f16(rng, batch * heads * hd)
    kbits = [poison_f16_bits(O.round_f16(normal_f16(rng, kv * cap * hd)), kv, tk, hd, cap, False)
             for _ in range(batch)]
    vbits = [poison_f16_bits(O.round_f16(normal_f16(rng, kv * cap * hd)), kv, tk, hd, cap, True)
             for _ in range(batch)]
    ks, vs = [gpu.upload_u16(x) for x in kbits], [gpu.upload_u16(x) for x in vbits]
    scratch = DecodeScratch()
    dq = gpu.upload(q)
    a = gpu.download(gpu.decode_batched(dq, ks, vs, [tk] * batch, [cap] * batch, heads, kv, hd,
                                        scale, False, scratch)).reshape(batch, -1)
    b = gpu.download(gpu.decode_batched(dq, ks, vs, [tk] * batch, [cap] * batch, heads, kv, hd,
                                        scale, False, scratch)).reshape(batch, -1)
    assert np.array_equal(a, b) and np.isfinite(a).all()
    for s in range(batch):
        want = O.decode_f64(q.reshape(batch, -1)[s], kbits[s], vbits[s], heads, kv, hd, 0, tk, cap,
                            scale, False)
        assert_close_to(f"pairs by cluster {shape} sequence {s}", want, a[s], 2e-5)
    # the un-normalised triples of the same launch (what a sharded step exchanges)
    tri = gpu.download(gpu.decode_batched(dq, ks, vs, [tk] * batch, [cap] * batch, heads, kv, hd,
                                          scale, False, scratch, partial=True))
    tri = tri.reshape(batch, heads, hd + 2)
    got = tri[:, :, :hd] / tri[:, :, hd + 1:hd + 2]
    assert np.abs(got.reshape(batch, -1) - a).max() <= 1e-6 * np.abs(a).max()
