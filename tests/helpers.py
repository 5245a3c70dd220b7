"""Shared pieces of the parity tests: the error measures and the input makers."""
from __future__ import annotations

import numpy as np

from oracle import oracle as O


def max_abs(want, got) -> float:
    return float(np.max(np.abs(np.asarray(want, np.float64) - np.asarray(got, np.float64))))


def rel_l2(want, got) -> float:
    w = np.asarray(want, np.float64)
    g = np.asarray(got, np.float64)
    return float(np.linalg.norm(w - g) / max(np.linalg.norm(w), 1e-30))


def cosine(want, got) -> float:
    w = np.asarray(want, np.float64).ravel()
    g = np.asarray(got, np.float64).ravel()
    return float(w @ g / max(np.linalg.norm(w) * np.linalg.norm(g), 1e-30))


def assert_close_to(name, want, got, tol) -> None:
    """The reference's measure: worst error as a fraction of the largest
    expected magnitude (crates/llmtie-cuda/tests/kernels.rs:53-70)."""
    want = np.asarray(want, np.float32)
    got = np.asarray(got, np.float32)
    assert want.shape == got.shape, f"{name}: length"
    assert np.isfinite(got).all(), f"{name}: non-finite output"
    scale = max(float(np.abs(want).max()), 1e-6)
    d = np.abs(want.astype(np.float64) - got.astype(np.float64))
    at = int(d.argmax())
    assert d[at] / scale < tol, (
        f"{name}: {d[at] / scale:e} of full scale at [{at}], cpu {want[at]} vs gpu {got[at]}")


# BASELINE.json's bar: max-abs 2e-3 and relative-L2 1e-3 against the CPU
# attention on identical fp16-rounded inputs.
MAX_ABS_TOL = 2e-3
REL_L2_TOL = 1e-3


def assert_parity(name, want, got) -> None:
    got = np.asarray(got, np.float32)
    assert np.isfinite(got).all(), f"{name}: non-finite output"
    ma, rl, cs = max_abs(want, got), rel_l2(want, got), cosine(want, got)
    assert ma <= MAX_ABS_TOL and rl <= REL_L2_TOL, (
        f"{name}: max-abs {ma:.3e} (<= {MAX_ABS_TOL}), rel-L2 {rl:.3e} (<= {REL_L2_TOL}), "
        f"cosine {cs:.8f}")


def lay_caches(kvals, vvals, kv_heads, tk, hd, cap, fill=0.0):
    """[kv][tk][hd] values into K [kv][cap][hd] and V [kv][hd][cap]; the unused
    capacity holds `fill` (zero as a real cache's is, or a poison)."""
    kc = np.full((kv_heads, cap, hd), fill, dtype=np.float32)
    vc = np.full((kv_heads, hd, cap), fill, dtype=np.float32)
    kc[:, :tk, :] = np.asarray(kvals, np.float32).reshape(kv_heads, tk, hd)
    vc[:, :, :tk] = np.asarray(vvals, np.float32).reshape(kv_heads, tk, hd).transpose(0, 2, 1)
    return kc.reshape(-1), vc.reshape(-1)


def normal_f16(rng, n) -> np.ndarray:
    """i.i.d. N(0,1) rounded to f16 and widened: identical bits for both sides."""
    return O.through_f16(rng.standard_normal(n).astype(np.float32))


def poison_f16_bits(h, kv_heads, tk, hd, cap, transposed):
    """NaN bits into every cache slot past the live length."""
    a = np.asarray(h, np.uint16).copy()
    if transposed:
        a.reshape(kv_heads, hd, cap)[:, :, tk:] = 0x7E00
    else:
        a.reshape(kv_heads, cap, hd)[:, tk:, :] = 0x7E00
    return a


def prefill_spread(q, kc, vc, tq, past, heads, kv_heads, hd, cap, scale, causal):
    """The spread the reference's prefill tolerance uses: for each output,
    sum_p (e_p / l) * |v_p - want| over the keys the row sees
    (crates/llmtie-cuda/tests/kernels.rs:2337-2352). Returns (want, spread)."""
    tk = past + tq
    group = heads // kv_heads
    h16 = lambda x: np.asarray(x, np.float32).astype(np.float16).astype(np.float64)
    q = np.asarray(q, np.float32).reshape(tq, heads, hd)
    K = h16(np.asarray(kc).reshape(kv_heads, cap, hd))[:, :tk, :]
    V = h16(np.asarray(vc).reshape(kv_heads, hd, cap))[:, :, :tk]
    want = np.zeros((tq, heads, hd))
    spread = np.zeros((tq, heads, hd))
    for h in range(heads):
        kh = h // group
        s = (h16(q[:, h, :]) @ K[kh].T) * np.float64(np.float32(scale))
        if causal:
            r = np.arange(tq)[:, None]
            c = np.arange(tk)[None, :]
            s = np.where(c <= past + r, s, -np.inf)
        e = np.exp(s - s.max(axis=1, keepdims=True))
        l = e.sum(axis=1, keepdims=True)
        w = (h16(e.astype(np.float32)) @ V[kh].T) / l
        want[:, h, :] = w
        p = e / l
        for r0 in range(0, tq, 32):
            blk = slice(r0, min(tq, r0 + 32))
            dev = np.abs(V[kh].T[None, :, :] - w[blk][:, None, :])   # [rows][tk][hd]
            spread[blk, h, :] = np.einsum("rp,rpd->rd", p[blk], dev)
    return want.reshape(-1), spread.reshape(-1)


def assert_prefill_tolerance(name, want, spread, got) -> float:
    """err <= 2e-4 + 1e-2 |want| + 1e-2 spread everywhere, and the worst error
    under half its tolerance (kernels.rs:2354-2373)."""
    got = np.asarray(got, np.float64)
    assert np.isfinite(got).all(), f"{name}: non-finite output"
    tol = 2e-4 + 1e-2 * np.abs(want) + 1e-2 * spread
    ratio = np.abs(want - got) / tol
    worst = float(ratio.max())
    at = int(ratio.argmax())
    assert worst <= 1.0, f"{name}: [{at}] {got[at]} wanted {want[at]} ({worst:.3f} of tolerance)"
    assert worst < 0.5, f"{name}: worst error is {worst:.3f} of its tolerance"
    return worst
