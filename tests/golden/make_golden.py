"""Generates tests/golden/attention_golden.npz: small seeded cases of the
attention path with the CPU oracle's outputs.

The reference ships no golden vectors for this path and cannot be run where
this was written, so these vectors come from the oracle (a restatement of the
reference's scalar routines) and pin it against drift; the GPU tests compare
the CUDA path with the same vectors. Inputs are not stored: each case is
regenerated from its seed. Run `python -m tests.golden.make_golden` to rewrite.
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle import oracle as O  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "attention_golden.npz")

# kind, then the shape; inputs come from the reference's `seq` generator.
CASES = {
    "prefill_causal_gqa_h128": ("prefill", 8, 2, 128, True, 40, 9, 64, 71),
    "prefill_window_h64": ("prefill", 4, 4, 64, False, 40, 0, 48, 81),
    "prefill_ragged_cap_h128": ("prefill", 4, 2, 128, True, 33, 5, 38, 91),
    "decode_gqa_h128": ("decode", 32, 8, 128, 333, 512, False, 300),
    "decode_cross_h64": ("decode", 20, 20, 64, 1500, 1500, True, 354),
    "decode_one_key": ("decode", 8, 2, 128, 1, 256, False, 300),
    "rope_4095": ("rope", 5, 3, 128, 10000.0, 4095, 75),
}


def case_inputs(spec):
    kind = spec[0]
    if kind == "prefill":
        _, heads, kv, hd, causal, tq, past, cap, salt = spec
        tk = past + tq
        q = O.seq(tq * heads * hd, salt) * np.float32(4.0)
        kc = np.zeros((kv, cap, hd), np.float32)
        vc = np.zeros((kv, hd, cap), np.float32)
        kc[:, :tk, :] = O.seq(kv * tk * hd, salt + 1).reshape(kv, tk, hd)
        vc[:, :, :tk] = O.seq(kv * tk * hd, salt + 2).reshape(kv, tk, hd).transpose(0, 2, 1)
        return q, O.round_f16(kc), O.round_f16(vc)
    if kind == "decode":
        _, heads, kv, hd, tk, cap, scale_q, salt = spec
        return (O.seq(heads * hd, salt), O.round_f16(O.seq(kv * cap * hd, salt + 1)),
                O.round_f16(O.seq(kv * hd * cap, salt + 2)))
    _, t, heads, hd, theta, first, salt = spec
    return (O.seq(t * heads * hd, salt),)


def run_case(spec) -> np.ndarray:
    kind = spec[0]
    if kind == "prefill":
        _, heads, kv, hd, causal, tq, past, cap, _ = spec
        q, kc, vc = case_inputs(spec)
        scale = float(np.float32(hd) ** np.float32(-0.5))
        return O.prefill(q, kc, vc, tq, past, heads, kv, hd, cap, scale, causal)
    if kind == "decode":
        _, heads, kv, hd, tk, cap, scale_q, _ = spec
        q, kc, vc = case_inputs(spec)
        return O.decode_f64(q, kc, vc, heads, kv, hd, 0, tk, cap, 0.11, scale_q)
    _, t, heads, hd, theta, first, _ = spec
    (x,) = case_inputs(spec)
    return O.rope(x, t, heads, hd, theta, first)


if __name__ == "__main__":
    np.savez_compressed(OUT, **{name: run_case(spec) for name, spec in CASES.items()})
    print(OUT, os.path.getsize(OUT), "bytes")
