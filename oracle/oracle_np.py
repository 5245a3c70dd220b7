"""An independent numpy restatement of the same reference routines, used only
to cross-check the C oracle (TEST INFRASTRUCTURE - parity unpinned).

Written from the reference's scalar code, not from oracle.c: vectorised where
numpy allows, so an indexing slip in one of the two shows as a disagreement.
"""
from __future__ import annotations

import numpy as np


def seq(n: int, salt: int) -> np.ndarray:
    """crates/llmtie-cuda/tests/kernels.rs:35-45."""
    mask = (1 << 64) - 1
    s = ((salt * 0x9E3779B97F4A7C15) & mask) | 1
    out = np.empty(n, dtype=np.float32)
    for i in range(n):
        s ^= (s << 13) & mask
        s ^= s >> 7
        s ^= (s << 17) & mask
        out[i] = np.float32(np.float32(s >> 40) / np.float32(8388608.0)) * np.float32(4.0) \
            - np.float32(2.0)
    return out


def h16(x: np.ndarray) -> np.ndarray:
    """Through f16 and back, round to nearest even, as f64."""
    return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float64)


def rope(x, t, heads, hd, theta, first, freq_div=None) -> np.ndarray:
    """crates/llmtie-dsp/src/rope.rs:83-126, all in f32."""
    x = np.asarray(x, dtype=np.float32).reshape(t, heads, hd).copy()
    half = hd // 2
    i = np.arange(half, dtype=np.float32)
    # f32 results of f32 operands, taken through f64 so that they are the
    # correctly rounded values a good libm returns (numpy's own f32 SIMD
    # routines are a few ulp off, which at position 4095 is visible).
    expo = (np.float32(-2.0) * i / np.float32(hd)).astype(np.float32)
    inv = np.power(np.float64(np.float32(theta)), expo.astype(np.float64)).astype(np.float32)
    if freq_div is not None:
        inv = (inv / np.asarray(freq_div, dtype=np.float32)).astype(np.float32)
    pos = (first + np.arange(t)).astype(np.float32)
    ang = (pos[:, None] * inv[None, :]).astype(np.float32)
    sn = np.sin(ang.astype(np.float64)).astype(np.float32)
    cs = np.cos(ang.astype(np.float64)).astype(np.float32)
    a, b = x[:, :, :half].copy(), x[:, :, half:].copy()
    x[:, :, :half] = a * cs[:, None, :] - b * sn[:, None, :]
    x[:, :, half:] = b * cs[:, None, :] + a * sn[:, None, :]
    return x.reshape(-1)


def prefill(q, k, v, tq, past, heads, kv_heads, hd, cap, scale, causal, scale_q=False, tk=0):
    """crates/llmtie-cuda/tests/kernels.rs:2300-2364. k, v: f32 arrays in the
    cache layouts (already holding f16-representable values or not: they are
    put through f16 here, as the kernel's staging does)."""
    tk = tk or past + tq
    group = heads // kv_heads
    scale = np.float32(scale)
    q = np.asarray(q, dtype=np.float32).reshape(tq, heads, hd)
    K = h16(np.asarray(k).reshape(kv_heads, cap, hd))
    V = h16(np.asarray(v).reshape(kv_heads, hd, cap))
    out = np.zeros((tq, heads, hd), dtype=np.float32)
    for h in range(heads):
        kh = h // group
        qh = h16(q[:, h, :] * scale) if scale_q else h16(q[:, h, :])
        s = qh @ K[kh, :tk, :].T
        if not scale_q:
            s = s * np.float64(scale)
        if causal:
            r = np.arange(tq)[:, None]
            c = np.arange(tk)[None, :]
            s = np.where(c <= past + r, s, -np.inf)
        m = s.max(axis=1, keepdims=True)
        e = np.exp(s - m)
        l = e.sum(axis=1, keepdims=True)
        acc = h16(e.astype(np.float32)) @ V[kh, :, :tk].T
        out[:, h, :] = (acc / l).astype(np.float32)
    return out.reshape(-1)


def decode(q, k, v, heads, kv_heads, hd, tk, cap, scale, scale_q):
    """crates/llmtie-cuda/tests/kernels.rs:2733-2774 at f64: q f32, k and v
    f32 arrays in the cache layouts holding what the device copy holds."""
    group = heads // kv_heads
    scale = np.float32(scale)
    q = np.asarray(q, dtype=np.float32).reshape(heads, hd)
    K = np.asarray(k, dtype=np.float64).reshape(kv_heads, cap, hd)
    V = np.asarray(v, dtype=np.float64).reshape(kv_heads, hd, cap)
    out = np.zeros((heads, hd), dtype=np.float32)
    for qh in range(heads):
        h = qh // group
        qr = (q[qh] * scale).astype(np.float64) if scale_q else q[qh].astype(np.float64)
        s = K[h, :tk, :] @ qr
        if not scale_q:
            s = s * np.float64(scale)
        e = np.exp(s - s.max())
        out[qh] = ((V[h, :, :tk] @ e) / e.sum()).astype(np.float32)
    return out.reshape(-1)


def quantize_q8(x):
    """kernels.rs:693-719 in numpy: (codes, scales) per group of 32, all f32."""
    x = np.asarray(x, dtype=np.float32).reshape(-1, 32)
    d = (np.abs(x).max(axis=1) * np.float32(1.0 / 127.0)).astype(np.float32)
    inv = np.where(d > 0, np.float32(1.0) / np.where(d > 0, d, np.float32(1.0)), np.float32(0.0))
    inv = inv.astype(np.float32)
    codes = np.rint((x * inv[:, None]).astype(np.float32)).astype(np.int8)
    return codes.reshape(-1), d
