"""The CosyVoice3 callers of the attention path: the flow model's DiT block
(crates/llmtie-cosy/src/flow.rs:545-572) - GPT-J style partial rope on q and
k before the heads are split, f32 head splits, non-causal `flash_attn` at 16
heads of 64 - and the shapes of the speech LM (src/llm.rs:448-475; its decode
and prefill cases sit with the other shapes in test_gpu_decode / _prefill)."""
import numpy as np
import pytest

from oracle import oracle as O
from tests.helpers import assert_parity, normal_f16

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("positions,dim,rot", [(257, 1024, 64), (9, 12, 4), (33, 70, 70)])
def test_rope_gptj_rotates_the_first_pairs_of_each_row(gpu, positions, dim, rot):
    from ttsxabe_b200 import OddHeadDim, SliceOverrun

    x = O.seq(positions * dim, 81)
    inv = (1.0 / (10000.0 ** (np.arange(rot // 2, dtype=np.float32) * 2 / rot))).astype(np.float32)
    dx, dinv = gpu.upload(x), gpu.upload(inv)
    gpu.rope_gptj(dx, dinv, positions, dim, rot)
    got = gpu.download(dx).reshape(positions, dim)
    want = O.rope_gptj(x, inv, positions, dim, rot).reshape(positions, dim)
    # everything past rot_dim passes through untouched
    assert np.array_equal(got[:, rot:], x.reshape(positions, dim)[:, rot:])
    # the fast sine and cosine against libm's: a few ulp of the angle
    assert np.abs(got - want).max() <= 2e-4 * np.abs(x).max() * (1 + positions / 256)
    with pytest.raises(OddHeadDim):
        gpu.rope_gptj(dx, dinv, positions, dim, 3)
    with pytest.raises(SliceOverrun):
        gpu.rope_gptj(dx, dinv, positions + 1, dim, rot)


def test_flow_attention_block(gpu):
    """One row of the DiT's attention as flow.rs runs it: q and k rotated
    where they lie, k and v split by head into f32 [heads][n][64] and
    [heads][64][n], q left unsplit, non-causal fused attention."""
    n, heads, hd = 257, 16, 64
    d = heads * hd
    rng = np.random.default_rng(9)
    q, k, v = (normal_f16(rng, n * d) for _ in range(3))
    inv = (1.0 / (10000.0 ** (np.arange(hd // 2, dtype=np.float32) * 2 / hd))).astype(np.float32)
    dq, dk, dv, dinv = gpu.upload(q), gpu.upload(k), gpu.upload(v), gpu.upload(inv)
    gpu.rope_gptj(dq, dinv, n, d, hd)
    gpu.rope_gptj(dk, dinv, n, d, hd)
    kh = gpu.split_heads(dk, n, heads, hd)
    vt = gpu.split_heads_t(dv, n, heads, hd)
    scale = float(np.float32(hd) ** np.float32(-0.5))
    got = gpu.download(gpu.flash_attn(dq, kh, vt, n, 0, heads, heads, hd, n, scale, False))
    # the head splits are plain re-layouts
    kr = gpu.download(dk).reshape(n, heads, hd)
    assert np.array_equal(gpu.download(kh).reshape(heads, n, hd), kr.transpose(1, 0, 2))
    assert np.array_equal(gpu.download(vt).reshape(heads, hd, n),
                          v.reshape(n, heads, hd).transpose(1, 2, 0))
    # oracle on the rotated rows the device produced (the rope has its own test)
    want = O.prefill(gpu.download(dq), gpu.download(kh), gpu.download(vt), n, 0, heads, heads, hd,
                     n, scale, False, tk=n)
    assert_parity("flow attention", want, got)
