"""The Whisper cross-attention caches: built from the decoder layers'
projections of the encoder output (crates/llmtie-asr/src/model.rs:872-960) and
read by the decoder's cross-attention.

Shapes, salts and the offset-and-bias case are those of the reference's
`the_packed_head_splits_are_the_f32_ones_converted`
(crates/llmtie-cuda/tests/kernels.rs:500-575); the results are held to the
oracle bit for bit.
"""
import numpy as np
import pytest

from oracle import oracle as O
from tests.helpers import assert_parity, normal_f16

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("t,heads,hd", [(7, 3, 4), (1500, 20, 64), (1, 2, 8), (130, 5, 6)])
def test_packed_head_splits_are_the_oracle_bit_for_bit(gpu, t, heads, hd):
    from ttsxabe_b200 import SliceOverrun

    d = heads * hd
    x = O.seq(t * d, 61)
    dx = gpu.upload(x)
    for transposed in (False, True):
        got = gpu.download_u16(gpu.split_heads_f16_at(dx, 0, None, t, heads, hd,
                                                      transposed=transposed))
        assert np.array_equal(got, O.split_heads_f16(x, None, t, heads, hd, transposed=transposed))
    # the block that starts `off` into a larger buffer, with a bias row added first
    off = 3 * t * d
    big = O.seq(off + 2 * t * d, 62)
    bias = O.seq(2 * d, 63)
    dbig, dbias = gpu.upload(big), gpu.upload(bias)
    block = big[off:off + t * d]
    for transposed in (False, True):
        for cap in (t, (t + 8) // 8 * 8):
            got = gpu.download_u16(gpu.split_heads_f16_at(dbig, off, (dbias, d), t, heads, hd,
                                                          cap=cap, transposed=transposed))
            want = O.split_heads_f16(block, bias[d:], t, heads, hd, cap=cap, transposed=transposed)
            assert np.array_equal(got, want), (transposed, cap)
    with pytest.raises(SliceOverrun):
        gpu.split_heads_f16_at(dbig, off + t * d + 1, None, t, heads, hd)
    with pytest.raises(SliceOverrun):
        gpu.split_heads_f16_at(dbig, off, (dbias, d + 1), t, heads, hd)


def test_every_layers_caches_in_two_launches(gpu):
    """`cross_kv_build` over four layers is the per-layer splits one after
    another (keys without a bias, values with their layer's), at a capacity
    padded to a multiple of 8 and zero past the frames."""
    layers, t, heads, hd, cap = 4, 1500, 20, 64, 1504
    d = heads * hd
    k_all, v_all, bias = O.seq(layers * t * d, 71), O.seq(layers * t * d, 72), O.seq(layers * d, 73)
    dk, dv, db = gpu.upload(k_all), gpu.upload(v_all), gpu.upload(bias)
    n0 = gpu.launch_count()
    kc, vc = gpu.cross_kv_build(dk, dv, db, layers, t, heads, hd, cap)
    assert gpu.launch_count() - n0 == 2
    kc, vc = gpu.download_u16(kc).reshape(layers, -1), gpu.download_u16(vc).reshape(layers, -1)
    for l in range(layers):
        one_k = gpu.download_u16(gpu.split_heads_f16_at(dk, l * t * d, None, t, heads, hd, cap=cap))
        one_v = gpu.download_u16(gpu.split_heads_t_f16_at(dv, l * t * d, (db, l * d), t, heads, hd,
                                                          cap=cap))
        assert np.array_equal(kc[l], one_k) and np.array_equal(vc[l], one_v)
        assert np.array_equal(kc[l], O.split_heads_f16(k_all[l * t * d:(l + 1) * t * d], None, t,
                                                       heads, hd, cap=cap))
        assert np.array_equal(vc[l], O.split_heads_f16(v_all[l * t * d:(l + 1) * t * d],
                                                       bias[l * d:(l + 1) * d], t, heads, hd,
                                                       cap=cap, transposed=True))
    assert not vc.reshape(layers, heads * hd, cap)[:, :, t:].any()


@pytest.mark.parametrize("n", [1, 8, 32])
def test_cross_attention_over_built_caches(gpu, n):
    """BASELINE config 4 end to end on the decoder side: caches built from f32
    projections at a capacity of 1504, then 1 to 32 query rows over their 1500
    frames, against the oracle; the same answer as over caches of capacity
    1500 (the reference's) to the bar's tolerance."""
    from ttsxabe_b200 import DecodeScratch

    heads, hd, t = 20, 64, 1500
    d = heads * hd
    rng = np.random.default_rng(400 + n)
    kx, vx = normal_f16(rng, t * d), normal_f16(rng, t * d)
    q = normal_f16(rng, n * d)
    dq, dkx, dvx = gpu.upload(q), gpu.upload(kx), gpu.upload(vx)
    outs = []
    for cap in (1504, 1500):
        kc = gpu.split_heads_f16_at(dkx, 0, None, t, heads, hd, cap=cap)
        vc = gpu.split_heads_t_f16_at(dvx, 0, None, t, heads, hd, cap=cap)
        scratch = DecodeScratch()
        outs.append(gpu.download(gpu.cross_attn(dq, kc, vc, n, heads, hd, t, cap, 0.125, scratch)))
    want = O.prefill(q, O.split_heads_f16(kx, None, t, heads, hd),
                     O.split_heads_f16(vx, None, t, heads, hd, transposed=True), n, 0, heads, heads,
                     hd, t, 0.125, False, scale_q=True, tk=t)
    assert_parity(f"cross attention n={n}, capacity 1504", want, outs[0])
    assert_parity(f"cross attention n={n}, capacity 1500", want, outs[1])
    assert np.abs(outs[0] - outs[1]).max() <= 2e-5 * np.abs(want).max()
