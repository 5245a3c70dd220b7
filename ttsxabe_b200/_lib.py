"""ctypes binding of libllmtie_b200.so (the C ABI in include/llmtie_b200.h).

There is no fallback: if the library is missing or does not load, importing
the symbols raises, and every operator in this package goes through them.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libllmtie_b200.so")

vp = C.c_void_p
sz = C.c_size_t
i32 = C.c_int32
f32 = C.c_float
pvp = C.POINTER(C.c_void_p)
pi32 = C.POINTER(C.c_int32)

# name -> (restype, argtypes); the order is that of include/llmtie_b200.h.
PROTOTYPES = {
    "llmtie_open": (i32, [i32, pvp]),
    "llmtie_open_on_stream": (i32, [i32, vp, pvp]),
    "llmtie_close": (None, [vp]),
    "llmtie_last_error": (C.c_char_p, []),
    "llmtie_stream": (vp, [vp]),
    "llmtie_ordinal": (i32, [vp]),
    "llmtie_synchronize": (i32, [vp]),
    "llmtie_set_wait_limit_cycles": (i32, [vp, C.c_int64]),
    "llmtie_alloc": (i32, [vp, sz, pvp]),
    "llmtie_zeros": (i32, [vp, sz, pvp]),
    "llmtie_free": (i32, [vp, vp]),
    "llmtie_upload": (i32, [vp, vp, vp, sz]),
    "llmtie_download": (i32, [vp, vp, vp, sz]),
    "llmtie_round_f16": (i32, [vp, vp, vp, sz]),
    "llmtie_kv_want_capacity": (sz, [sz, sz, sz, sz]),
    "llmtie_kv_shared_prefix": (sz, [C.POINTER(C.c_uint32), sz, C.POINTER(C.c_uint32), sz]),
    "llmtie_kv_alloc_f16": (i32, [vp, sz, sz, sz, pvp, pvp]),
    "llmtie_cache_grow_f16": (i32, [vp, vp, sz, vp, sz, sz, sz, sz, sz, sz, i32]),
    "llmtie_cache_grow": (i32, [vp, vp, sz, vp, sz, sz, sz, sz, sz, sz, i32]),
    "llmtie_cache_append_f16": (i32, [vp, vp, sz, sz, vp, sz, sz, sz, sz, sz, sz, i32]),
    "llmtie_cache_append": (i32, [vp, vp, sz, sz, vp, sz, sz, sz, sz, sz, sz, i32]),
    "llmtie_gemv_qkv_f16": (
        i32, [vp, vp, sz, vp, sz, vp, vp, vp, sz, sz, sz, sz, sz, sz, vp, sz, vp, sz, vp, sz]),
    "llmtie_split_heads_f16_at": (i32, [vp, vp, sz, sz, vp, sz, sz, vp, sz, sz, sz, sz, sz, i32]),
    "llmtie_cross_kv_build": (i32, [vp, vp, sz, vp, sz, vp, sz, vp, sz, vp, sz, sz, sz, sz, sz, sz]),
    "llmtie_split_heads": (i32, [vp, vp, sz, sz, vp, sz, sz, sz, sz, sz, i32]),
    "llmtie_rope_gptj": (i32, [vp, vp, sz, vp, sz, sz, sz, sz]),
    "llmtie_rope_scaled": (i32, [vp, vp, sz, sz, vp, sz, sz, sz, f32, sz]),
    "llmtie_rope_cache_f16": (
        i32,
        [vp, vp, sz, sz, vp, sz, sz, vp, sz, sz, vp, sz, sz, sz, f32, sz, vp, sz, vp, sz, sz],
    ),
    "llmtie_rope_cache_batched": (
        i32, [vp, vp, sz, vp, sz, vp, sz, vp, sz, sz, sz, sz, f32, pi32, pvp, pvp, pi32]),
    "llmtie_supports_flash": (i32, [sz, sz, sz]),
    "llmtie_flash_attn_f16": (
        i32, [vp, vp, sz, vp, sz, vp, sz, vp, sz, sz, sz, sz, sz, sz, sz, f32, i32]),
    "llmtie_flash_attn": (
        i32, [vp, vp, sz, vp, sz, vp, sz, vp, sz, sz, sz, sz, sz, sz, sz, f32, i32]),
    "llmtie_flash_attn_rows": (i32, [vp, vp, sz, vp, sz, sz, sz, sz, f32, vp, sz]),
    "llmtie_flash_attn_rows_batched": (i32, [vp, vp, sz, vp, sz, sz, sz, sz, sz, f32, vp, sz]),
    "llmtie_flash_rows_work_bytes": (sz, [sz, sz, sz]),
    "llmtie_decode_scratch_new": (i32, [vp, pvp]),
    "llmtie_decode_scratch_free": (None, [vp, vp]),
    "llmtie_attn_decode_f16": (
        i32, [vp, vp, sz, sz, vp, sz, vp, sz, sz, sz, sz, sz, sz, f32, i32, vp, vp, sz, sz]),
    "llmtie_attn_decode_f16_q": (
        i32, [vp, vp, sz, sz, vp, sz, vp, sz, sz, sz, sz, sz, sz, f32, i32, vp, vp, sz, sz,
              vp, sz, vp, sz]),
    "llmtie_attn_decode": (
        i32, [vp, vp, sz, sz, vp, sz, vp, sz, sz, sz, sz, sz, sz, f32, i32, vp, vp, sz, sz]),
    "llmtie_attn_decode_f16_noalloc": (
        i32, [vp, vp, sz, sz, vp, sz, vp, sz, sz, sz, sz, sz, sz, f32, i32, vp, sz, sz]),
    "llmtie_decode_batched": (
        i32, [vp, vp, sz, pvp, pvp, pi32, pi32, sz, sz, sz, sz, f32, i32, vp, vp, sz, i32]),
    "llmtie_lse_merge": (i32, [vp, vp, sz, sz, sz, sz, vp, sz]),
    "llmtie_decode_batched_push": (
        i32, [vp, vp, sz, pvp, pvp, pi32, pi32, sz, sz, sz, sz, f32, i32, vp, vp]),
    "llmtie_decode_cut": (i32, [pi32, sz, sz, sz, i32, pi32, sz, pi32]),
    "llmtie_decode_resident_clusters": (i32, [vp, sz, i32]),
    "llmtie_decode_plan": (i32, [pi32, sz, sz, sz, sz, i32, i32, i32, i32, pi32, sz, pi32, pi32]),
    "llmtie_decode_batched_fused": (
        i32, [vp, vp, sz, pvp, pvp, pi32, pi32, sz, sz, sz, sz, f32, i32, vp, vp, pvp, vp, sz]),
    "llmtie_lse_merge_wait": (i32, [vp, vp, sz, sz, vp, sz]),
    "llmtie_decode_batched_signal": (
        i32, [vp, vp, sz, pvp, pvp, pi32, pi32, sz, sz, sz, sz, f32, i32, vp, vp, pvp]),
    "llmtie_lse_merge_pairs": (i32, [vp, vp, vp, vp, sz, sz, sz, vp, sz]),
    "llmtie_cross_attn": (
        i32, [vp, vp, sz, vp, sz, vp, sz, sz, sz, sz, sz, sz, f32, vp, vp, sz]),
    "llmtie_prefill_varlen": (
        i32,
        [vp, vp, sz, vp, sz, vp, sz, pi32, sz, pvp, pvp, pi32, pi32, vp, sz, sz, sz, f32, f32,
         vp, sz],
    ),
    "llmtie_kprof_enable": (None, [vp, i32]),
    "llmtie_kprof_reset": (None, [vp]),
    "llmtie_kprof_report": (sz, [vp, C.c_char_p, sz]),
    "llmtie_kernel_resources": (i32, [C.c_char_p, pi32, pi32, pi32]),
    "llmtie_launch_count": (C.c_uint64, [vp]),
}

_lib = None


def load() -> C.CDLL:
    """Loads the library once and types every entry point. Raises if absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is not built; run `python -m ttsxabe_b200.build` "
            "(there is no fallback path)"
        )
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks it
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
