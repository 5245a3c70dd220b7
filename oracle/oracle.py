"""ctypes face of liboracle.so, the C restatement of the reference's scalar
attention routines (TEST INFRASTRUCTURE - parity unpinned, see oracle.h).

Only tests, the smoke check and the benchmark's CPU arms may import this.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liboracle.so")

sz, f32, i32 = C.c_size_t, C.c_float, C.c_int
vp = C.c_void_p


def build(force: bool = False) -> str:
    src = [os.path.join(HERE, f) for f in ("oracle.c", "oracle.h", "Makefile")]
    stale = force or not os.path.exists(LIB) or any(
        os.path.getmtime(s) > os.path.getmtime(LIB) for s in src)
    if stale:
        subprocess.run(["make", "-s", "-B", "-C", HERE, "liboracle.so"], check=True)
    return LIB


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(LIB)
        L.orc_f32_to_f16.restype = C.c_uint16
        L.orc_f32_to_f16.argtypes = [f32]
        L.orc_f16_to_f32.restype = f32
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_round_f16.argtypes = [vp, vp, sz]
        L.orc_widen_f16.argtypes = [vp, vp, sz]
        L.orc_seq.argtypes = [vp, sz, C.c_uint64]
        L.orc_rope.argtypes = [vp, sz, sz, sz, f32, sz, vp]
        L.orc_cache_append_f16.argtypes = [vp, vp, sz, sz, sz, sz, sz, i32]
        L.orc_cache_append_f32.argtypes = [vp, vp, sz, sz, sz, sz, sz, i32]
        L.orc_cache_grow.argtypes = [vp, vp, sz, sz, sz, sz, sz, i32, sz]
        L.orc_rope_cache_f16.argtypes = [vp, vp, vp, vp, sz, sz, sz, f32, sz, vp, vp, sz]
        L.orc_prefill.argtypes = [vp, sz, vp, vp, i32, sz, sz, sz, sz, sz, sz, sz, f32, i32,
                                  i32, vp, sz]
        L.orc_prefill_fast.restype = i32
        L.orc_prefill_fast.argtypes = [vp, sz, vp, vp, i32, sz, sz, sz, sz, sz, sz, sz, f32, i32,
                                       i32, vp, sz, i32]
        L.orc_decode_f32.argtypes = [vp, vp, vp, sz, sz, sz, sz, sz, f32, i32, vp]
        L.orc_decode_f64.argtypes = [vp, vp, vp, sz, sz, sz, sz, sz, sz, f32, i32, vp, vp, vp,
                                     vp]
        L.orc_lse_merge.argtypes = [vp, vp, vp, sz, sz, sz, vp]
        L.orc_quantize_q8.argtypes = [vp, sz, vp, vp]
        L.orc_decode_fast.restype = i32
        L.orc_decode_fast.argtypes = [vp, vp, vp, sz, sz, sz, sz, sz, f32, i32, vp, i32]
        L.orc_max_threads.restype = i32
        L.orc_gemv_qkv_f16.argtypes = [vp, vp, vp, vp, vp, sz, sz, sz, sz, sz, vp, vp, vp]
        L.orc_rope_gptj.argtypes = [vp, vp, sz, sz, sz]
        L.orc_split_heads_f16.argtypes = [vp, vp, vp, sz, sz, sz, sz, i32]
        _lib = L
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u16(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint16)


def _p(a) -> int:
    return a.ctypes.data


def seq(n: int, salt: int) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().orc_seq(_p(out), n, salt)
    return out


def round_f16(x) -> np.ndarray:
    x = _f32(x).reshape(-1)
    out = np.empty(x.size, dtype=np.uint16)
    lib().orc_round_f16(_p(x), _p(out), x.size)
    return out


def widen_f16(h) -> np.ndarray:
    h = _u16(h).reshape(-1)
    out = np.empty(h.size, dtype=np.float32)
    lib().orc_widen_f16(_p(h), _p(out), h.size)
    return out


def through_f16(x) -> np.ndarray:
    return widen_f16(round_f16(x))


def rope(x, t, heads, hd, theta, first, freq_div=None) -> np.ndarray:
    out = _f32(x).reshape(-1).copy()
    fd = None if freq_div is None else _f32(freq_div)
    lib().orc_rope(_p(out), t, heads, hd, theta, first, None if fd is None else _p(fd))
    return out


def cache_append_f16(src, dst, n, kv_heads, hd, cap, past, transposed) -> None:
    src = _f32(src).reshape(-1)
    assert dst.dtype == np.uint16 and dst.flags.c_contiguous
    lib().orc_cache_append_f16(_p(src), _p(dst), n, kv_heads, hd, cap, past, int(transposed))


def cache_append_f32(src, dst, n, kv_heads, hd, cap, past, transposed) -> None:
    src = _f32(src).reshape(-1)
    assert dst.dtype == np.float32 and dst.flags.c_contiguous
    lib().orc_cache_append_f32(_p(src), _p(dst), n, kv_heads, hd, cap, past, int(transposed))


def cache_grow(src, dst, kv_heads, hd, old_cap, new_cap, live, transposed) -> None:
    assert src.dtype == dst.dtype and dst.flags.c_contiguous and src.flags.c_contiguous
    lib().orc_cache_grow(_p(src), _p(dst), kv_heads, hd, old_cap, new_cap, live,
                         int(transposed), src.dtype.itemsize)


def rope_cache_f16(q, k, v, freq_div, heads, kv_heads, hd, theta, pos, kc, vc, cap) -> np.ndarray:
    """Returns the rotated q; writes kc and vc in place."""
    q = _f32(q).reshape(-1).copy()
    k = _f32(k).reshape(-1)
    v = _f32(v).reshape(-1)
    fd = None if freq_div is None else _f32(freq_div)
    lib().orc_rope_cache_f16(_p(q), _p(k), _p(v), None if fd is None else _p(fd), heads,
                             kv_heads, hd, theta, pos, _p(kc), _p(vc), cap)
    return q


def prefill(q, k, v, tq, past, heads, kv_heads, hd, cap, scale, causal, *, scale_q=False,
            tk=0, q_stride=None, fast=False, threads=0) -> np.ndarray:
    """k, v: uint16 (f16 bits) or float32 caches in the reference's layouts."""
    q = _f32(q).reshape(-1)
    kv_f16 = k.dtype == np.uint16
    k = _u16(k) if kv_f16 else _f32(k)
    v = _u16(v) if kv_f16 else _f32(v)
    qs = heads * hd if q_stride is None else q_stride
    out = np.empty(tq * heads * hd, dtype=np.float32)
    if fast:
        lib().orc_prefill_fast(_p(q), qs, _p(k), _p(v), int(kv_f16), tq, past, tk, heads,
                               kv_heads, hd, cap, scale, int(causal), int(scale_q), _p(out),
                               heads * hd, threads)
    else:
        lib().orc_prefill(_p(q), qs, _p(k), _p(v), int(kv_f16), tq, past, tk, heads, kv_heads,
                          hd, cap, scale, int(causal), int(scale_q), _p(out), heads * hd)
    return out


def decode_f32(q, k, v, heads, kv_heads, hd, tk, cap, scale, scale_q) -> np.ndarray:
    q, k, v = _f32(q).reshape(-1), _f32(k).reshape(-1), _f32(v).reshape(-1)
    out = np.empty(heads * hd, dtype=np.float32)
    lib().orc_decode_f32(_p(q), _p(k), _p(v), heads, kv_heads, hd, tk, cap, scale,
                         int(scale_q), _p(out))
    return out


def decode_f64(q, k, v, heads, kv_heads, hd, t0, t1, cap, scale, scale_q, triple=False):
    q, k, v = _f32(q).reshape(-1), _u16(k).reshape(-1), _u16(v).reshape(-1)
    out = np.empty(heads * hd, dtype=np.float32)
    if not triple:
        lib().orc_decode_f64(_p(q), _p(k), _p(v), heads, kv_heads, hd, t0, t1, cap, scale,
                             int(scale_q), _p(out), None, None, None)
        return out
    o = np.empty(heads * hd, dtype=np.float32)
    m = np.empty(heads, dtype=np.float32)
    l = np.empty(heads, dtype=np.float32)
    lib().orc_decode_f64(_p(q), _p(k), _p(v), heads, kv_heads, hd, t0, t1, cap, scale,
                         int(scale_q), _p(out), _p(o), _p(m), _p(l))
    return out, o, m, l


def lse_merge(o, m, l, parts, rows, hd) -> np.ndarray:
    o, m, l = _f32(o).reshape(-1), _f32(m).reshape(-1), _f32(l).reshape(-1)
    out = np.empty(rows * hd, dtype=np.float32)
    lib().orc_lse_merge(_p(o), _p(m), _p(l), parts, rows, hd, _p(out))
    return out


def quantize_q8(x):
    """(codes int8 [n], scales f32 [n/32]) of x, n a multiple of 32."""
    x = _f32(x).reshape(-1)
    codes = np.empty(x.size, dtype=np.int8)
    scales = np.empty(x.size // 32, dtype=np.float32)
    lib().orc_quantize_q8(_p(x), x.size, _p(codes), _p(scales))
    return codes, scales


def decode_fast(q, k, v, heads, kv_heads, hd, tk, cap, scale, scale_q, threads=0):
    q, k, v = _f32(q).reshape(-1), _u16(k).reshape(-1), _u16(v).reshape(-1)
    out = np.empty(heads * hd, dtype=np.float32)
    used = lib().orc_decode_fast(_p(q), _p(k), _p(v), heads, kv_heads, hd, tk, cap, scale,
                                 int(scale_q), _p(out), threads)
    return out, used


def split_heads_f16(x, bias, t, heads, hd, cap=None, transposed=False) -> np.ndarray:
    """f16 bits of the cache [heads][cap][hd] (or transposed [heads][hd][cap])
    holding x [t][heads*hd] + bias; zero past t."""
    cap = t if cap is None else cap
    x = _f32(x).reshape(-1)
    b = None if bias is None else _f32(bias).reshape(-1)
    out = np.zeros(heads * cap * hd, dtype=np.uint16)
    lib().orc_split_heads_f16(_p(x), None if b is None else _p(b), _p(out), t, heads, hd, cap,
                              int(transposed))
    return out


def gemv_qkv_f16(a, w, bias, k, d, hd, cap, pos, q, kc, vc) -> None:
    """Writes q [d], and position pos of kc [d/hd][cap][hd] and vc [d][cap], in place."""
    a, w = _f32(a).reshape(-1), _u16(w).reshape(-1)
    bs = [None if b is None else _f32(b).reshape(-1) for b in bias]
    for x in (q, kc, vc):
        assert x.dtype == np.float32 and x.flags.c_contiguous
    lib().orc_gemv_qkv_f16(_p(a), _p(w), *[None if b is None else _p(b) for b in bs], k, d, hd,
                           cap, pos, _p(q), _p(kc), _p(vc))


def rope_gptj(x, inv_freq, positions, dim, rot_dim) -> np.ndarray:
    out = _f32(x).reshape(-1).copy()
    f = _f32(inv_freq).reshape(-1)
    lib().orc_rope_gptj(_p(out), _p(f), positions, dim, rot_dim)
    return out


def max_threads() -> int:
    return int(lib().orc_max_threads())
