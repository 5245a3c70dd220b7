"""The allocation-free decode entry point against the ordinary one.

`llmtie_attn_decode_f16_noalloc` exists for callers that cannot allocate while
decoding - a per-token pipeline thread that must never wait on the driver, a
process whose own pool already owns the whole device. It keeps its split-KV
partials in a static array inside the library instead of a DecodeScratch. It
is held here to the ordinary entry point's output on two calls in a row
through the C ABI: the second call finds the array as the first left it, so a
counter or a partial that leaked from one call into the next would show.

Collected last on purpose, so that a run that stops at the first failure has
already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as O
from tests.helpers import assert_close_to

pytestmark = pytest.mark.gpu


def _call_noalloc(gpu, dq, dk, dv, heads, kv, hd, tk, cap, scale, scale_q, out):
    lib = gpu._lib
    return lib.llmtie_attn_decode_f16_noalloc(
        gpu._h, dq.data_ptr(), dq.numel(), 0, dk.data_ptr(), dk.numel(), dv.data_ptr(),
        dv.numel(), heads, kv, hd, tk, cap, C.c_float(scale), int(scale_q), out.data_ptr(),
        out.numel(), 0)


def test_two_calls_in_a_row_match_the_ordinary_entry(gpu):
    from ttsxabe_b200 import DecodeScratch

    # two different shapes back to back: a long grouped context that is cut
    # over many blocks, then a short ungrouped one that reuses the same array
    cases = [(32, 8, 128, 7777, 8192, False, 0.0883883), (20, 20, 64, 1001, 1024, True, 0.125)]
    scratch = DecodeScratch()
    for i, (heads, kv, hd, tk, cap, scale_q, scale) in enumerate(cases):
        q = O.seq(heads * hd, 900 + i)
        k0 = O.seq(kv * cap * hd, 910 + i)
        v0 = O.seq(kv * cap * hd, 920 + i)
        dq, dk, dv = gpu.upload(q), gpu.upload_f16(k0), gpu.upload_f16(v0)
        want_dev = gpu.attn_decode_f16(dq, dk, dv, heads, kv, hd, tk, cap, scale, scale_q, scratch)
        want = gpu.download(want_dev)
        out = gpu.zeros(heads * hd)
        for call in range(2):
            st = _call_noalloc(gpu, dq, dk, dv, heads, kv, hd, tk, cap, scale, scale_q, out)
            assert st == 0, gpu._lib.llmtie_last_error()
            got = gpu.download(out)
            assert_close_to(f"no-alloc decode case {i} call {call}", want, got, 2e-5)
        # and both against the CPU oracle
        ref = O.decode_f64(q, O.round_f16(k0), O.round_f16(v0), heads, kv, hd, 0, tk, cap, scale,
                           scale_q)
        assert_close_to(f"no-alloc decode case {i} vs oracle", ref, got, 2e-5)


def test_sizes_beyond_the_static_scratch_are_refused(gpu):
    from ttsxabe_b200 import Misaligned, UnsupportedAttention

    hd = 64
    dq = gpu.upload(O.seq(80 * hd, 1))
    dk = gpu.upload_f16(O.seq(80 * 16 * hd, 2))
    out = gpu.zeros(80 * hd)
    # more kv heads than the array has counters for
    with pytest.raises(UnsupportedAttention):
        gpu.attn_decode_f16_noalloc(dq, dk, dk, 80, 80, hd, 8, 16, 0.1, False, out=out)
    # a capacity whose value rows are not 16-byte aligned (the Whisper cross cache's 1500)
    dk2 = gpu.upload_f16(O.seq(2 * 1500 * hd, 3))
    with pytest.raises(Misaligned):
        gpu.attn_decode_f16_noalloc(dq, dk2, dk2, 2, 2, hd, 100, 1500, 0.1, False, out=out)
