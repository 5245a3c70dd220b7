"""The stacked attention projection in front of the Whisper decoder's
self-attention (crates/llmtie-cuda/src/device.rs:4393-4479): the reference's
own case (`the_stacked_projection_places_what_three_placed_products_do`,
crates/llmtie-cuda/tests/kernels.rs:3211-3330) and the model's shape, against
the f64 oracle, with the rest of both caches untouched; then the decode
attention that reads what it placed."""
import numpy as np
import pytest

from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("k,d,hd,cap,pos", [(96, 64, 16, 5, 2), (1280, 1280, 64, 448, 17),
                                            (70, 24, 8, 9, 8)])
def test_stacked_projection_places_its_columns(gpu, k, d, hd, cap, pos):
    a = O.seq(k, 60)
    w = np.concatenate([O.seq(d * k, 61), O.seq(d * k, 62), O.seq(d * k, 63)]) / np.float32(8.0)
    bq, bv = O.seq(d, 64), O.seq(d, 65)
    kc0, vc0 = O.seq(d * cap, 66), O.seq(d * cap, 67)
    w16 = O.round_f16(w)
    q, kc, vc = gpu.upload(O.seq(d, 68)), gpu.upload(kc0), gpu.upload(vc0)
    gpu.gemv_qkv_f16(gpu.upload(a), gpu.upload_u16(w16), (gpu.upload(bq), None, gpu.upload(bv)), k,
                     d, hd, cap, pos, q, kc, vc)
    wq, wk, wv = O.seq(d, 68).copy(), kc0.copy(), vc0.copy()
    O.gemv_qkv_f16(a, w16, (bq, None, bv), k, d, hd, cap, pos, wq, wk, wv)
    gq, gk, gv = gpu.download(q), gpu.download(kc), gpu.download(vc)
    full = max(np.abs(wq).max(), 1e-6)
    for name, want, got in (("q", wq, gq), ("keys", wk, gk), ("values", wv, gv)):
        assert np.abs(want - got).max() <= 2e-6 * full * np.sqrt(k), name
    # only position `pos` of either cache was written
    mk = np.ones((d // hd, cap, hd), bool)
    mk[:, pos, :] = False
    mv = np.ones((d, cap), bool)
    mv[:, pos] = False
    assert np.array_equal(gk.reshape(d // hd, cap, hd)[mk], kc0.reshape(d // hd, cap, hd)[mk])
    assert np.array_equal(gv.reshape(d, cap)[mv], vc0.reshape(d, cap)[mv])
    # and twice gives the same bits
    q2, kc2, vc2 = gpu.upload(O.seq(d, 68)), gpu.upload(kc0), gpu.upload(vc0)
    gpu.gemv_qkv_f16(gpu.upload(a), gpu.upload_u16(w16), (gpu.upload(bq), None, gpu.upload(bv)), k,
                     d, hd, cap, pos, q2, kc2, vc2)
    assert np.array_equal(gpu.download(q2), gq) and np.array_equal(gpu.download(kc2), gk)


def test_projection_refusals(gpu):
    from ttsxabe_b200 import CacheOverrun, RaggedBlock, SliceOverrun

    k, d, hd, cap = 96, 64, 16, 5
    a, w = gpu.upload(O.seq(k, 1)), gpu.upload_u16(O.round_f16(O.seq(3 * d * k, 2)))
    q, kc, vc = gpu.zeros(d), gpu.zeros(d * cap), gpu.zeros(d * cap)
    none = (None, None, None)
    with pytest.raises(RaggedBlock):
        gpu.gemv_qkv_f16(a, w, none, 95, d, hd, cap, 0, q, kc, vc)
    with pytest.raises(RaggedBlock):
        gpu.gemv_qkv_f16(a, w, none, k, d, 24, cap, 0, q, kc, vc)
    with pytest.raises(CacheOverrun):
        gpu.gemv_qkv_f16(a, w, none, k, d, hd, cap, cap, q, kc, vc)
    with pytest.raises(SliceOverrun):
        gpu.gemv_qkv_f16(a, w, none, k, d + hd, hd, cap, 0, q, kc, vc)


def test_decoder_self_attention_step(gpu):
    """A Whisper decoder layer's self-attention step as crates/llmtie-asr/src/
    model.rs:1029-1086 runs it: the stacked projection places q, k and v, then
    `attn_decode` off the f32 caches with the scale on the query."""
    from ttsxabe_b200 import DecodeScratch

    heads, hd, cap, past = 20, 64, 448, 40
    d = heads * hd
    rng = np.random.default_rng(3)
    kc0 = np.zeros((heads, cap, hd), np.float32)
    vc0 = np.zeros((heads, hd, cap), np.float32)
    kc0[:, :past] = rng.standard_normal((heads, past, hd))
    vc0[:, :, :past] = rng.standard_normal((heads, hd, past))
    a = rng.standard_normal(d).astype(np.float32)
    w16 = O.round_f16((rng.standard_normal(3 * d * d) / np.sqrt(d)).astype(np.float32))
    bq, bv = O.seq(d, 4), O.seq(d, 5)
    q, kc, vc = gpu.zeros(d), gpu.upload(kc0.reshape(-1)), gpu.upload(vc0.reshape(-1))
    gpu.gemv_qkv_f16(gpu.upload(a), gpu.upload_u16(w16), (gpu.upload(bq), None, gpu.upload(bv)), d,
                     d, hd, cap, past, q, kc, vc)
    got = gpu.download(gpu.attn_decode(q, kc, vc, heads, heads, hd, past + 1, cap, 0.125, True,
                                       DecodeScratch()))
    wq, wk, wv = np.zeros(d, np.float32), kc0.reshape(-1).copy(), vc0.reshape(-1).copy()
    O.gemv_qkv_f16(a, w16, (bq, None, bv), d, d, hd, cap, past, wq, wk, wv)
    want = O.decode_f32(wq, wk, wv, heads, heads, hd, past + 1, cap, 0.125, True)
    assert np.abs(want - got).max() <= 2e-5 * np.abs(want).max()
