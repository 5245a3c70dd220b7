"""The C-ABI library loads, exports every symbol the header declares, and -
without a GPU - refuses to open rather than falling back to anything."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "llmtie_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(llmtie_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_entry_points():
    names = declared_symbols()
    for must in ("llmtie_open", "llmtie_flash_attn_f16", "llmtie_attn_decode_f16",
                 "llmtie_flash_attn_rows", "llmtie_rope_cache_f16", "llmtie_cache_grow_f16",
                 "llmtie_decode_batched", "llmtie_lse_merge", "llmtie_prefill_varlen"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from ttsxabe_b200 import _lib

    lib = _lib.load()
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
        assert name in _lib.PROTOTYPES, f"{name} has no ctypes prototype"
    for name in _lib.PROTOTYPES:
        assert name in declared_symbols(), f"{name} is bound but not declared in the header"


def test_every_entry_point_cites_the_reference():
    """Each declaration sits under a comment naming the reference interface it
    replaces (file:line), or says it has no counterpart."""
    text = open(HEADER).read()
    assert text.count("device.rs:") >= 15
    assert "crates/llmtie-chat/src/model.rs" in text and "kernels.rs:" in text


def test_open_without_a_device_is_refused():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    from ttsxabe_b200 import NoDevice, Gpu

    with pytest.raises(NoDevice):
        Gpu.open(0)


def test_null_handle_is_refused_not_dereferenced():
    from ttsxabe_b200 import _lib

    lib = _lib.load()
    assert lib.llmtie_synchronize(None) == 12
    assert b"null" in lib.llmtie_last_error()
    out = C.c_void_p()
    assert lib.llmtie_alloc(None, 16, C.byref(out)) == 12
    assert lib.llmtie_launch_count(None) == 0


def test_shape_predicate_and_policy_need_no_device():
    from ttsxabe_b200 import _lib, want_capacity

    lib = _lib.load()
    assert lib.llmtie_supports_flash(128, 32, 8) == 1
    assert lib.llmtie_supports_flash(64, 20, 20) == 1
    assert lib.llmtie_supports_flash(96, 8, 2) == 0
    assert lib.llmtie_supports_flash(128, 10, 4) == 0
    # crates/llmtie-chat/src/model.rs:714-721
    assert want_capacity(0, 0, 300, 131072) == 1024      # prompt + 256 reserve, pow2
    assert want_capacity(0, 0, 1, 131072) == 256         # floor of 256
    assert want_capacity(1024, 1000, 24, 131072) == 0    # fits
    assert want_capacity(1024, 1024, 1, 131072) == 2048  # one token: no reserve
    assert want_capacity(256, 200, 100, 400) == 400      # capped at max positions
    assert want_capacity(256, 200, 300, 400) == 500      # ... but never below what is asked
    assert lib.llmtie_flash_rows_work_bytes(1500, 20, 64) == 2 * 20 * 1536 * 64 * 2
