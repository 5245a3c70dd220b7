"""Fused prefill / encoder attention through the C ABI against the oracle.

Shapes, salts, the peaked softmax (q x 100) and the tolerance are those of the
reference's `fused_attention_sized` (crates/llmtie-cuda/tests/kernels.rs:
2249-2439); the BASELINE configs add the N(0,1) cases at the 2e-3 / 1e-3 bar.
"""
import numpy as np
import pytest

from oracle import oracle as O
from tests.helpers import (assert_parity, assert_prefill_tolerance, lay_caches, normal_f16,
                           prefill_spread)

pytestmark = pytest.mark.gpu

# (heads, kv_heads, hd, causal, tq, past, cap, f16 cache)
SIZED = [
    (4, 2, 128, True, 70, 33, 160, False),
    (4, 4, 64, False, 70, 33, 160, False),
    (4, 2, 64, False, 70, 33, 160, False),
    (4, 4, 128, True, 70, 33, 160, False),
    (4, 4, 64, True, 70, 33, 160, False),
    (4, 2, 64, True, 70, 33, 160, False),
    # f32 caches of odd capacity: the general kernel (even ones are rounded to f16 once and
    # take the tensor-memory kernel)
    (4, 2, 128, True, 70, 33, 161, False),
    (4, 4, 64, False, 70, 33, 161, False),
    (8, 2, 128, True, 150, 0, 256, True),
    (8, 1, 128, True, 90, 17, 128, True),
    (4, 4, 128, True, 200, 40, 256, True),
    (4, 2, 128, True, 130, 5, 138, True),
    # prompts shorter than a tile of the tensor-memory kernel (its boxes are wider than the caches)
    (8, 2, 128, True, 8, 0, 64, True),
    (8, 2, 128, True, 1, 0, 8, True),
    (8, 2, 128, True, 30, 33, 64, True),
    (8, 2, 128, False, 70, 0, 72, True),
    # one new row on a long past; one row into a second row block
    (8, 2, 128, True, 1, 200, 256, True),
    (8, 2, 128, True, 129, 0, 136, True),
    (8, 2, 128, True, 1, 1000, 1008, True),
    (4, 4, 64, False, 300, 0, 300, False),
    # crates/llmtie-cosy's callers, both off f32 caches: the speech LM's prefill
    # (14 / 2 heads, a group of 7; src/llm.rs:448-475) and the flow model's
    # non-causal 16-head attention (src/flow.rs:545-572)
    (14, 2, 64, True, 300, 20, 320, False),
    (14, 2, 64, True, 130, 0, 256, False),
    (16, 16, 64, False, 257, 0, 258, False),
]


@pytest.mark.parametrize("case", SIZED)
def test_fused_attention_sized(gpu, case):
    heads, kv, hd, causal, tq, past, cap, half = case
    tk = past + tq
    scale = float(np.float32(hd) ** np.float32(-0.5))
    q = O.seq(tq * heads * hd, 71) * np.float32(100.0)
    kc, vc = lay_caches(O.seq(kv * tk * hd, 72), O.seq(kv * tk * hd, 73), kv, tk, hd, cap)
    dq = gpu.upload(q)
    if half:
        out = gpu.flash_attn_f16(dq, gpu.upload_f16(kc), gpu.upload_f16(vc), tq, past, heads, kv,
                                 hd, cap, scale, causal)
    else:
        out = gpu.flash_attn(dq, gpu.upload(kc), gpu.upload(vc), tq, past, heads, kv, hd, cap,
                             scale, causal)
    got = gpu.download(out)
    want, spread = prefill_spread(q, kc, vc, tq, past, heads, kv, hd, cap, scale, causal)
    # the numpy restatement and the C oracle are the same function
    c_want = O.prefill(q, kc, vc, tq, past, heads, kv, hd, cap, scale, causal)
    assert np.abs(c_want - want).max() < 1e-5
    assert_prefill_tolerance(str(case), want, spread, got)


def test_prefill_refusals(gpu):
    from ttsxabe_b200 import (CacheOverrun, OddCacheCapacity, SliceOverrun,
                              UnsupportedAttention)

    dq = gpu.upload(O.seq(16 * 8 * 128, 1))
    dk = gpu.upload_f16(O.seq(2 * 256 * 128, 2))
    with pytest.raises(UnsupportedAttention):
        gpu.flash_attn_f16(dq, dk, dk, 16, 0, 8, 2, 64, 256, 1.0, True)   # f16 cache: 128 only
    with pytest.raises(UnsupportedAttention):
        gpu.flash_attn_f16(dq, dk, dk, 16, 0, 8, 3, 128, 256, 1.0, True)
    with pytest.raises(OddCacheCapacity):
        gpu.flash_attn_f16(dq, dk, dk, 16, 0, 8, 2, 128, 255, 1.0, True)
    with pytest.raises(CacheOverrun):
        gpu.flash_attn_f16(dq, dk, dk, 16, 250, 8, 2, 128, 256, 1.0, True)
    with pytest.raises(SliceOverrun):
        gpu.flash_attn_f16(dq, dk, dk, 17, 0, 8, 2, 128, 256, 1.0, True)
    assert gpu.supports_flash(128, 32, 8) and gpu.supports_flash(64, 20, 20)
    assert not gpu.supports_flash(96, 8, 2) and not gpu.supports_flash(128, 10, 4)


def test_config1_single_layer_prefill(gpu):
    """BASELINE config 1: batch 1, seq 128, 32 Q / 8 KV heads, hd 128, Q/K/V
    fp16 N(0,1), NeoX RoPE theta 10000 on Q and K, scale 1/sqrt(128), fp32
    output [128, 32, 128]."""
    heads, kv, hd, n = 32, 8, 128, 128
    rng = np.random.default_rng(1)
    q = normal_f16(rng, n * heads * hd)
    k = normal_f16(rng, n * kv * hd)
    v = normal_f16(rng, n * kv * hd)
    scale = float(np.float32(hd) ** np.float32(-0.5))
    cap = 256
    # oracle: f32 RoPE on the f16-rounded values, rotated K rounded into the cache
    qr = O.rope(q, n, heads, hd, 10000.0, 0)
    kr = O.rope(k, n, kv, hd, 10000.0, 0)
    kc = np.zeros(kv * cap * hd, np.uint16)
    vc = np.zeros(kv * cap * hd, np.uint16)
    O.cache_append_f16(kr, kc, n, kv, hd, cap, 0, False)
    O.cache_append_f16(v, vc, n, kv, hd, cap, 0, True)
    want = O.prefill(qr, kc, vc, n, 0, heads, kv, hd, cap, scale, True)

    # the reference's chain: rope q, rope k, append k, append v^T, flash_attn_f16
    dq, dk, dv = gpu.upload(q), gpu.upload(k), gpu.upload(v)
    gpu.rope(dq, 0, n, heads, hd, 10000.0, 0)
    gpu.rope(dk, 0, n, kv, hd, 10000.0, 0)
    dkc, dvc = gpu.zeros_f16(kv * cap * hd), gpu.zeros_f16(kv * cap * hd)
    gpu.cache_append_f16(dk, 0, dkc, n, kv, hd, cap, 0, False)
    gpu.cache_append_f16(dv, 0, dvc, n, kv, hd, cap, 0, True)
    out = gpu.flash_attn_f16(dq, dkc, dvc, n, 0, heads, kv, hd, cap, scale, True)
    got = gpu.download(out)
    assert got.shape == (n * heads * hd,)
    assert_parity("config 1", want, got)
    assert np.array_equal(gpu.download_u16(dvc), vc)

    # the fused varlen entry gives the same answer and the same cache
    dq2 = gpu.upload(q)
    kc2, vc2 = gpu.zeros_f16(kv * cap * hd), gpu.zeros_f16(kv * cap * hd)
    out2 = gpu.prefill_varlen(dq2, gpu.upload(k), gpu.upload(v), [0, n], [kc2], [vc2], [0],
                              [cap], None, heads, kv, hd, 10000.0, scale)
    assert_parity("config 1 (varlen entry)", want, gpu.download(out2))
    assert np.array_equal(gpu.download_u16(kc2), gpu.download_u16(dkc))
    assert np.array_equal(gpu.download_u16(vc2), vc)
    # q is rotated on its way into the kernel, with the chain's bits: the
    # caller's q is left as it was, and the answers are the chain's exactly
    assert np.array_equal(gpu.download(dq2), q)
    assert np.array_equal(gpu.download(out2), got)


def test_config2_ragged_batched_prefill(gpu):
    """BASELINE config 2: 8 ragged sequences, lengths seeded uniform in
    [256, 512], packed with cu_seqlens, 32 Q / 8 KV heads, hd 128, RoPE theta
    10000, the new K/V written into the fp16 KV cache."""
    heads, kv, hd, batch = 32, 8, 128, 8
    rng = np.random.default_rng(2)
    lens = rng.integers(256, 513, size=batch)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    total = int(cu[-1])
    scale = float(np.float32(hd) ** np.float32(-0.5))
    q = normal_f16(rng, total * heads * hd)
    k = normal_f16(rng, total * kv * hd)
    v = normal_f16(rng, total * kv * hd)
    cap = 512
    dq = gpu.upload(q)
    kcs = [gpu.zeros_f16(kv * cap * hd) for _ in range(batch)]
    vcs = [gpu.zeros_f16(kv * cap * hd) for _ in range(batch)]
    out = gpu.prefill_varlen(dq, gpu.upload(k), gpu.upload(v), cu, kcs, vcs, [0] * batch,
                             [cap] * batch, None, heads, kv, hd, 10000.0, scale)
    got = gpu.download(out).reshape(total, heads * hd)
    for b in range(batch):
        n, r0 = int(lens[b]), int(cu[b])
        qb = q.reshape(total, -1)[r0:r0 + n].reshape(-1)
        kb = k.reshape(total, -1)[r0:r0 + n].reshape(-1)
        vb = v.reshape(total, -1)[r0:r0 + n].reshape(-1)
        qr = O.rope(qb, n, heads, hd, 10000.0, 0)
        kr = O.rope(kb, n, kv, hd, 10000.0, 0)
        kc = np.zeros(kv * cap * hd, np.uint16)
        vc = np.zeros(kv * cap * hd, np.uint16)
        O.cache_append_f16(kr, kc, n, kv, hd, cap, 0, False)
        O.cache_append_f16(vb, vc, n, kv, hd, cap, 0, True)
        want = O.prefill(qr, kc, vc, n, 0, heads, kv, hd, cap, scale, True, fast=True)
        assert_parity(f"config 2 sequence {b} ({n} tokens)", want, got[r0:r0 + n].reshape(-1))
        assert np.array_equal(gpu.download_u16(vcs[b]), vc)
        # rotated keys: the device's sincosf and the host's differ in the last bit
        dk = O.widen_f16(gpu.download_u16(kcs[b]))
        assert np.abs(dk - O.widen_f16(kc)).max() <= 4e-3
    # one sequence against the f64 oracle as well
    n = int(lens[0])
    qr = O.rope(q.reshape(total, -1)[:n].reshape(-1), n, heads, hd, 10000.0, 0)
    want64 = O.prefill(qr, gpu.download_u16(kcs[0]), gpu.download_u16(vcs[0]), n, 0, heads, kv,
                       hd, cap, scale, True)
    assert_parity("config 2 sequence 0 (f64 oracle)", want64, got[:n].reshape(-1))


def test_ragged_prefill_of_short_prompts(gpu):
    """Prompts of a few tokens, some onto a kept prefix: every sequence is
    shorter than one 128-key tile, so every tensor map is narrower than its
    box. Same chain, same bar as config 2; the caller's q is not written."""
    heads, kv, hd = 32, 8, 128
    lens = [1, 5, 40, 100, 127, 64]
    pasts = [0, 0, 17, 0, 0, 60]
    batch = len(lens)
    rng = np.random.default_rng(77)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    total = int(cu[-1])
    scale = float(np.float32(hd) ** np.float32(-0.5))
    q = normal_f16(rng, total * heads * hd)
    k = normal_f16(rng, total * kv * hd)
    v = normal_f16(rng, total * kv * hd)
    cap = 128
    olds = []
    kcs, vcs = [], []
    for b in range(batch):
        # what the kept prefix holds (already rotated keys, transposed values)
        kc = np.zeros(kv * cap * hd, np.uint16)
        vc = np.zeros(kv * cap * hd, np.uint16)
        if pasts[b]:
            O.cache_append_f16(normal_f16(rng, pasts[b] * kv * hd), kc, pasts[b], kv, hd, cap, 0, False)
            O.cache_append_f16(normal_f16(rng, pasts[b] * kv * hd), vc, pasts[b], kv, hd, cap, 0, True)
        olds.append((kc, vc))
        kcs.append(gpu.upload_u16(kc))
        vcs.append(gpu.upload_u16(vc))
    dq = gpu.upload(q)
    out = gpu.prefill_varlen(dq, gpu.upload(k), gpu.upload(v), cu, kcs, vcs, pasts, [cap] * batch,
                             None, heads, kv, hd, 10000.0, scale)
    got = gpu.download(out).reshape(total, heads * hd)
    assert np.array_equal(gpu.download(dq), q)
    for b in range(batch):
        n, r0, past = lens[b], int(cu[b]), pasts[b]
        qb = q.reshape(total, -1)[r0:r0 + n].reshape(-1)
        kb = k.reshape(total, -1)[r0:r0 + n].reshape(-1)
        vb = v.reshape(total, -1)[r0:r0 + n].reshape(-1)
        qr = O.rope(qb, n, heads, hd, 10000.0, past)
        kr = O.rope(kb, n, kv, hd, 10000.0, past)
        kc, vc = olds[b][0].copy(), olds[b][1].copy()
        O.cache_append_f16(kr, kc, n, kv, hd, cap, past, False)
        O.cache_append_f16(vb, vc, n, kv, hd, cap, past, True)
        assert np.array_equal(gpu.download_u16(vcs[b]), vc)
        # attention over the cache as the device left it (its sincosf and the
        # host's differ in the last bit of a rotated key)
        want = O.prefill(qr, gpu.download_u16(kcs[b]), vc, n, past, heads, kv, hd, cap, scale, True)
        assert_parity(f"short prompt {b} ({n} tokens on {past})", want, got[r0:r0 + n].reshape(-1))
        assert np.abs(O.widen_f16(gpu.download_u16(kcs[b])) - O.widen_f16(kc)).max() <= 4e-3


def test_ragged_prefill_with_empty_sequences(gpu):
    """A batch in which some sequences bring no new token (cu_seqlens repeats
    an offset): they take no rows of q or out, their caches are not touched,
    and the others come out as when prefilled alone. A batch of nothing but
    empty sequences is a no-op."""
    heads, kv, hd, cap = 32, 8, 128, 256
    lens = [0, 37, 0, 130, 0]
    pasts = [5, 0, 0, 9, 0]
    batch = len(lens)
    rng = np.random.default_rng(123)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    total = int(cu[-1])
    scale = float(np.float32(hd) ** np.float32(-0.5))
    q = normal_f16(rng, total * heads * hd)
    k = normal_f16(rng, total * kv * hd)
    v = normal_f16(rng, total * kv * hd)
    olds = [(O.round_f16(normal_f16(rng, kv * cap * hd)), O.round_f16(normal_f16(rng, kv * cap * hd)))
            for _ in range(batch)]
    kcs = [gpu.upload_u16(a) for a, _ in olds]
    vcs = [gpu.upload_u16(b) for _, b in olds]
    dq, dk, dv = gpu.upload(q), gpu.upload(k), gpu.upload(v)
    got = gpu.download(gpu.prefill_varlen(dq, dk, dv, cu, kcs, vcs, pasts, [cap] * batch, None,
                                          heads, kv, hd, 10000.0, scale)).reshape(total, -1)
    for b in range(batch):
        n, r0 = lens[b], int(cu[b])
        if n == 0:
            assert np.array_equal(gpu.download_u16(kcs[b]), olds[b][0])
            assert np.array_equal(gpu.download_u16(vcs[b]), olds[b][1])
            continue
        kc1, vc1 = gpu.upload_u16(olds[b][0]), gpu.upload_u16(olds[b][1])
        rows = lambda x, w: gpu.upload(x.reshape(total, w)[r0:r0 + n].reshape(-1))
        alone = gpu.download(gpu.prefill_varlen(rows(q, heads * hd), rows(k, kv * hd), rows(v, kv * hd),
                                                [0, n], [kc1], [vc1], [pasts[b]], [cap], None, heads,
                                                kv, hd, 10000.0, scale))
        assert np.array_equal(got[r0:r0 + n].reshape(-1), alone), f"sequence {b}"
        assert np.array_equal(gpu.download_u16(kcs[b]), gpu.download_u16(kc1))
        assert np.array_equal(gpu.download_u16(vcs[b]), gpu.download_u16(vc1))
    # nothing but empty sequences
    none = gpu.prefill_varlen(gpu.zeros(heads * hd), gpu.zeros(kv * hd), gpu.zeros(kv * hd), [0, 0, 0],
                              kcs[:2], vcs[:2], [5, 0], [cap, cap], None, heads, kv, hd, 10000.0, scale)
    gpu.synchronize()
    assert np.array_equal(gpu.download_u16(kcs[0]), olds[0][0])


def test_ragged_prefill_of_more_sequences_than_one_launch_maps(gpu):
    """Eleven sequences: the tensor-core kernel carries eight tensor maps a
    launch, so the batch goes in groups; the second group holds a 40-token
    sequence, too short for a 128-key box, and takes the general kernel."""
    heads, kv, hd = 8, 2, 128
    rng = np.random.default_rng(12)
    lens = [int(x) for x in rng.integers(130, 300, size=11)]
    lens[9] = 40
    batch = len(lens)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    total = int(cu[-1])
    scale = float(np.float32(hd) ** np.float32(-0.5))
    q = normal_f16(rng, total * heads * hd)
    k = normal_f16(rng, total * kv * hd)
    v = normal_f16(rng, total * kv * hd)
    cap = 304
    kcs = [gpu.zeros_f16(kv * cap * hd) for _ in range(batch)]
    vcs = [gpu.zeros_f16(kv * cap * hd) for _ in range(batch)]
    dq = gpu.upload(q)
    out = gpu.prefill_varlen(dq, gpu.upload(k), gpu.upload(v), cu, kcs, vcs,
                             [0] * batch, [cap] * batch, None, heads, kv, hd, 10000.0, scale)
    got = gpu.download(out).reshape(total, heads * hd)
    assert np.array_equal(gpu.download(dq), q)      # rotated in a copy, not in place
    for b in range(batch):
        n, r0 = lens[b], int(cu[b])
        qr = O.rope(q.reshape(total, -1)[r0:r0 + n].reshape(-1), n, heads, hd, 10000.0, 0)
        want = O.prefill(qr, gpu.download_u16(kcs[b]), gpu.download_u16(vcs[b]), n, 0, heads, kv,
                         hd, cap, scale, True, fast=True)
        assert_parity(f"sequence {b} of 11 ({n} tokens)", want, got[r0:r0 + n].reshape(-1))


def test_whisper_encoder_rows(gpu):
    """BASELINE config 4, encoder: non-causal self-attention over 1500 frames,
    20 heads, hd 64, scale 1/8 on q, context f16 [t, d] from one [t, 3d]
    product (crates/llmtie-cuda/src/device.rs:5812-5865)."""
    heads, hd, t = 20, 64, 1500
    d = heads * hd
    rng = np.random.default_rng(4)
    qkv = normal_f16(rng, t * 3 * d).reshape(t, 3 * d)
    out = gpu.flash_attn_rows(gpu.upload(qkv), t, heads, hd, 0.125)
    got = O.widen_f16(gpu.download_u16(out))
    kc, vc = lay_caches(qkv[:, d:2 * d].reshape(t, heads, hd).transpose(1, 0, 2),
                        qkv[:, 2 * d:].reshape(t, heads, hd).transpose(1, 0, 2), heads, t, hd, t)
    want = O.prefill(np.ascontiguousarray(qkv[:, :d]), kc, vc, t, 0, heads, heads, hd, t, 0.125,
                     False, scale_q=True, fast=True)
    # the context is returned rounded to f16: half an ulp of f16 on top of the bar
    assert np.abs(want - got).max() <= 2e-3 + 2.0 ** -11 * np.abs(want).max()
    assert np.linalg.norm(want - got) / np.linalg.norm(want) <= 1e-3 + 2.0 ** -11


@pytest.mark.parametrize("t,heads", [(150, 4), (1500, 20)])
def test_the_encoder_attention_off_its_rows_is_the_split_path(gpu, t, heads):
    """crates/llmtie-cuda/tests/kernels.rs:4040-4079: flash_attn_rows over the
    packed [t][3d] product against the chain it replaces - q scaled,
    split_heads, split_heads_t, flash_attn over the f32 caches with scale 1,
    the context rounded to f16. The reference runs one kernel under both and
    asserts equal bits; here the rows path is the tensor-memory kernel and the
    chain the general one, whose sums associate differently, so the two are
    held to the bar the reference sets between its f16-cache and f32-cache
    readers (tests/kernels.rs:2561-2725: 2e-3), and most elements must still
    come out as the same f16."""
    hd = 64
    d = heads * hd
    scale = np.float32(hd) ** np.float32(-0.5)
    qkv = (O.seq(t * 3 * d, 611) * np.float32(3.0)).reshape(t, 3 * d)
    q = np.ascontiguousarray(qkv[:, :d]) * scale
    k = gpu.split_heads(gpu.upload(np.ascontiguousarray(qkv[:, d:2 * d])), t, heads, hd)
    v = gpu.split_heads_t(gpu.upload(np.ascontiguousarray(qkv[:, 2 * d:])), t, heads, hd)
    ctx = gpu.download(gpu.flash_attn(gpu.upload(q), k, v, t, 0, heads, heads, hd, t, 1.0, False))
    want = O.round_f16(ctx)
    got = gpu.download_u16(gpu.flash_attn_rows(gpu.upload(qkv), t, heads, hd, float(scale)))
    a, b = O.widen_f16(want), O.widen_f16(got)
    # (the bar is relative to the contexts' size, which here reaches into the tens)
    assert np.abs(a - b).max() <= 2e-3 * max(1.0, float(np.abs(a).max())), np.abs(a - b).max()
    assert np.linalg.norm(a - b) / np.linalg.norm(a) <= 1e-3
    differ = float((want != got).mean())
    assert differ <= 0.10, f"{differ:.4f} of the elements round to another f16"


@pytest.mark.parametrize("batch,t", [(3, 200), (8, 1500), (10, 130)])
def test_batched_encoder_rows_equal_one_call_per_utterance(gpu, batch, t):
    """BASELINE config 4 at batch 8 in two launches: bit for bit what one
    flash_attn_rows call per utterance returns (the reference's way,
    crates/llmtie-asr/src/model.rs:792-822); also a batch longer than one
    attention launch carries, and a caller-owned staging buffer."""
    import torch

    heads, hd = 20, 64
    d = heads * hd
    rng = np.random.default_rng(40 + batch)
    qkv = normal_f16(rng, batch * t * 3 * d)
    dq = gpu.upload(qkv)
    nbytes = batch * gpu._lib.llmtie_flash_rows_work_bytes(t, heads, hd)
    work = gpu._empty(nbytes // 2, torch.float16)
    got = gpu.download_u16(gpu.flash_attn_rows_batched(dq, batch, t, heads, hd, 0.125, work=work))
    got2 = gpu.download_u16(gpu.flash_attn_rows_batched(dq, batch, t, heads, hd, 0.125))
    assert np.array_equal(got, got2)
    for b in range(batch):
        one = gpu.upload(qkv[b * t * 3 * d:(b + 1) * t * 3 * d])
        want = gpu.download_u16(gpu.flash_attn_rows(one, t, heads, hd, 0.125))
        assert np.array_equal(got[b * t * d:(b + 1) * t * d], want), f"utterance {b}"


@pytest.mark.parametrize("n", [1, 2, 5, 8, 16, 32])
def test_whisper_cross_attention(gpu, n):
    """BASELINE config 4, decoder cross-attention: 1 to 32 query tokens over
    the 1500-frame encoder K/V, 20 heads, hd 64, scale 1/8 on q."""
    from ttsxabe_b200 import DecodeScratch

    heads, hd, tk = 20, 64, 1500
    rng = np.random.default_rng(40 + n)
    q = normal_f16(rng, n * heads * hd)
    kc = O.round_f16(normal_f16(rng, heads * tk * hd))
    vc = O.round_f16(normal_f16(rng, heads * hd * tk))
    scratch = DecodeScratch()
    out = gpu.cross_attn(gpu.upload(q), gpu.upload_u16(kc), gpu.upload_u16(vc), n, heads, hd, tk,
                         tk, 0.125, scratch)
    got = gpu.download(out)
    want = O.prefill(q, kc, vc, n, 0, heads, heads, hd, tk, 0.125, False, scale_q=True, tk=tk)
    assert_parity(f"cross attention n={n}", want, got)
    if n == 1:
        # one row is the reference's attn_decode_f16 call with scale_q
        dec = gpu.download(gpu.attn_decode_f16(gpu.upload(q), gpu.upload_u16(kc),
                                               gpu.upload_u16(vc), heads, heads, hd, tk, tk,
                                               0.125, True, scratch))
        assert np.array_equal(dec, got)
