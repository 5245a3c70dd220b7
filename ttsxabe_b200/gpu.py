"""Host-side mirror of `llmtie_cuda::Gpu` for the attention path.

Same method names, argument order and refusals as the reference's device
handle (crates/llmtie-cuda/src/device.rs), over the C ABI in
include/llmtie_b200.h. Device buffers are torch CUDA tensors standing in for
`CudaSlice<f32>` / `CudaSlice<u16>`: torch owns the memory, the library is
given raw pointers and element counts. f16 buffers are `torch.float16`
tensors (the reference carries the same bits as u16).

All work runs on the handle's own non-blocking stream; torch allocations made
through this class are made under that stream, so stream-ordered reuse holds.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np
import torch

from . import _lib


# ---- errors: one class per CudaError variant (crates/llmtie-cuda/src/error.rs) ----

class CudaError(RuntimeError):
    code = -1


class NoDevice(CudaError):
    code = 1


class DriverError(CudaError):
    code = 2


class SliceOverrun(CudaError):
    code = 3


class CacheOverrun(CudaError):
    code = 4


class OddCacheCapacity(CudaError):
    code = 5


class OddHeadDim(CudaError):
    code = 6


class UnsupportedAttention(CudaError):
    code = 7


class RaggedBlock(CudaError):
    code = 8


class Misaligned(CudaError):
    code = 9


class MissingKernel(CudaError):
    code = 10


class DeviceTimeout(CudaError):
    code = 11


class InvalidArgument(CudaError):
    code = 12


_ERRORS = {
    c.code: c
    for c in (NoDevice, DriverError, SliceOverrun, CacheOverrun, OddCacheCapacity, OddHeadDim,
              UnsupportedAttention, RaggedBlock, Misaligned, MissingKernel, DeviceTimeout,
              InvalidArgument)
}


def _check(status: int) -> None:
    if status != 0:
        msg = _lib.load().llmtie_last_error().decode("utf-8", "replace")
        raise _ERRORS.get(status, CudaError)(msg)


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


class DecodeScratch:
    """`DecodeScratch` (device.rs:166-233): the split-KV workspace a caller
    keeps per cache. Empty until the first call allocates."""

    def __init__(self) -> None:
        self._gpu: Optional["Gpu"] = None
        self._h = C.c_void_p()

    def _bind(self, gpu: "Gpu") -> C.c_void_p:
        if self._gpu is None:
            _check(gpu._lib.llmtie_decode_scratch_new(gpu._h, C.byref(self._h)))
            self._gpu = gpu
        elif self._gpu is not gpu:
            raise InvalidArgument("a DecodeScratch belongs to the Gpu that first used it")
        return self._h

    def close(self) -> None:
        if self._gpu is not None and self._h and self._gpu._h:
            self._gpu._lib.llmtie_decode_scratch_free(self._gpu._h, self._h)
        self._h = C.c_void_p()
        self._gpu = None

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass


class _ExchangeStruct(C.Structure):
    _fields_ = [("world", C.c_int32), ("rank", C.c_int32),
                ("gather", C.POINTER(C.c_void_p)), ("flags", C.POINTER(C.c_void_p)),
                ("step", C.c_void_p)]


class Exchange:
    """The peer-memory descriptor `llmtie_decode_batched_push` and
    `llmtie_lse_merge_wait` take: every rank's gather buffer and flag array as
    mapped into this process, and this rank's step counter."""

    def __init__(self, world: int, rank: int, gather_ptrs, flag_ptrs, step_ptr: int,
                 pair_flag_ptrs=None) -> None:
        self.world, self.rank = world, rank
        self._gather = (C.c_void_p * world)(*gather_ptrs)
        self._flags = (C.c_void_p * world)(*flag_ptrs)
        self.struct = _ExchangeStruct(world, rank, self._gather, self._flags, step_ptr)
        # every rank's [pairs][world] words, for the fused entry only
        self.pair_flags = (None if pair_flag_ptrs is None
                           else (C.c_void_p * world)(*pair_flag_ptrs))

    def ref(self):
        return C.byref(self.struct)


def decode_cut(tk, kv_heads: int, head_dim: int, sm_count: int = 148) -> list[int]:
    """How a batched decode over contexts `tk` is cut over the grid: the first
    128-key unit of every block, then the total (host only, no device)."""
    lib = _lib.load()
    table = (C.c_int32 * 161)()
    grid = C.c_int32(0)
    _check(lib.llmtie_decode_cut((C.c_int32 * len(tk))(*tk), len(tk), kv_heads, head_dim, sm_count,
                                 table, len(table), C.byref(grid)))
    return list(table[:grid.value + 1])


def decode_plan(tk, kv_heads: int, rows: int, head_dim: int, sm_count: int = 148,
                resident=None):
    """The whole choice a decode launch makes (host only): returns
    (blocks_a_pair, cut) - 0: cut by work, 1: a block a pair, 2 / 4 / 8: a
    cluster of that many blocks a pair - for a device that holds `resident`
    clusters of 2, 4 and 8 blocks at once (by default a B200's answers:
    74 / 33 / 15 at head_dim 128, 148 / 71 / 33 at 64, where two blocks fit an SM)."""
    if resident is None:
        resident = (74, 33, 15) if head_dim == 128 else (148, 71, 33)
    lib = _lib.load()
    table = (C.c_int32 * 161)()
    grid, mode = C.c_int32(0), C.c_int32(0)
    _check(lib.llmtie_decode_plan((C.c_int32 * len(tk))(*tk), len(tk), kv_heads, rows, head_dim,
                                  sm_count, resident[0], resident[1], resident[2], table,
                                  len(table), C.byref(grid), C.byref(mode)))
    return mode.value, list(table[:grid.value + 1])


class Gpu:
    """One device handle with its own stream (device.rs:737-842)."""

    def __init__(self, ordinal: int = 0) -> None:
        self._lib = _lib.load()
        self._h = C.c_void_p()
        _check(self._lib.llmtie_open(ordinal, C.byref(self._h)))
        self.ordinal = ordinal
        self.device = torch.device("cuda", ordinal)
        self.stream = torch.cuda.ExternalStream(self._lib.llmtie_stream(self._h),
                                                device=self.device)

    @classmethod
    def open(cls, ordinal: int = 0) -> "Gpu":
        return cls(ordinal)

    def close(self) -> None:
        if self._h:
            self._lib.llmtie_close(self._h)
            self._h = C.c_void_p()

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass

    # ---- memory -------------------------------------------------------------

    def _empty(self, n: int, dtype: torch.dtype) -> torch.Tensor:
        with torch.cuda.stream(self.stream):
            return torch.empty(int(n), dtype=dtype, device=self.device)

    def uninit(self, n: int) -> torch.Tensor:
        return self._empty(n, torch.float32)

    def zeros(self, n: int) -> torch.Tensor:
        with torch.cuda.stream(self.stream):
            return torch.zeros(int(n), dtype=torch.float32, device=self.device)

    def zeros_f16(self, n: int) -> torch.Tensor:
        with torch.cuda.stream(self.stream):
            return torch.zeros(int(n), dtype=torch.float16, device=self.device)

    def upload(self, x) -> torch.Tensor:
        a = np.ascontiguousarray(np.asarray(x, dtype=np.float32)).reshape(-1)
        t = self._empty(a.size, torch.float32)
        if a.size:
            _check(self._lib.llmtie_upload(self._h, t.data_ptr(), a.ctypes.data, a.nbytes))
            self.synchronize()   # `a` may be a temporary
        return t

    def upload_u16(self, x) -> torch.Tensor:
        a = np.ascontiguousarray(np.asarray(x, dtype=np.uint16)).reshape(-1)
        t = self._empty(a.size, torch.float16)
        if a.size:
            _check(self._lib.llmtie_upload(self._h, t.data_ptr(), a.ctypes.data, a.nbytes))
            self.synchronize()
        return t

    def upload_f16(self, x) -> torch.Tensor:
        """f32 values rounded to f16 on the device (device.rs:1422-1431)."""
        src = self.upload(x)
        dst = self._empty(src.numel(), torch.float16)
        _check(self._lib.llmtie_round_f16(self._h, src.data_ptr(), dst.data_ptr(), src.numel()))
        return dst

    def download(self, t: torch.Tensor) -> np.ndarray:
        out = np.empty(t.numel(), dtype=np.float32)
        assert t.dtype == torch.float32
        if out.size:
            _check(self._lib.llmtie_download(self._h, out.ctypes.data, t.data_ptr(), out.nbytes))
        return out

    def download_u16(self, t: torch.Tensor) -> np.ndarray:
        out = np.empty(t.numel(), dtype=np.uint16)
        assert t.element_size() == 2
        if out.size:
            _check(self._lib.llmtie_download(self._h, out.ctypes.data, t.data_ptr(), out.nbytes))
        return out

    def synchronize(self) -> None:
        _check(self._lib.llmtie_synchronize(self._h))

    def set_wait_limit_cycles(self, cycles: int) -> None:
        """How long a device-side wait may spin before it gives up and the
        next synchronize / download raises `DeviceTimeout`; 0 restores the
        default of about a second."""
        _check(self._lib.llmtie_set_wait_limit_cycles(self._h, int(cycles)))

    # ---- RoPE ----------------------------------------------------------------

    def rope(self, x, off, t, heads, head_dim, theta, first) -> None:
        self.rope_scaled(x, off, None, t, heads, head_dim, theta, first)

    def rope_scaled(self, x, off, freq_div, t, heads, head_dim, theta, first) -> None:
        _check(self._lib.llmtie_rope_scaled(self._h, x.data_ptr(), x.numel(), off,
                                            _ptr(freq_div), t, heads, head_dim, theta, first))

    def rope_gptj(self, x, inv_freq, positions, dim, rot_dim) -> None:
        """`rope_gptj` (device.rs:4853-4873): partial, interleaved, in place."""
        _check(self._lib.llmtie_rope_gptj(self._h, x.data_ptr(), x.numel(), inv_freq.data_ptr(),
                                          inv_freq.numel(), positions, dim, rot_dim))

    def split_heads(self, x, t, heads, head_dim, x_off=0, cap=None, transposed=False):
        """`split_heads` / `split_heads_t`: f32 [t][heads*hd] -> [heads][cap][hd]
        (or transposed [heads][hd][cap]), cap = t unless given."""
        cap = t if cap is None else cap
        out = self.zeros(heads * cap * head_dim)
        _check(self._lib.llmtie_split_heads(self._h, x.data_ptr(), x.numel(), x_off,
                                            out.data_ptr(), out.numel(), t, heads, head_dim, cap,
                                            int(bool(transposed))))
        return out

    def split_heads_t(self, x, t, heads, head_dim, x_off=0, cap=None):
        return self.split_heads(x, t, heads, head_dim, x_off, cap, transposed=True)

    def rope_cache_f16(self, proj: Sequence[torch.Tensor], q, k, v, freq_div, heads, kv_heads,
                       head_dim, theta, pos, kc, vc, cap) -> None:
        """q, k, v are (buffer index, element offset) into `proj`."""
        def span(which):
            bi, off = which
            if bi >= len(proj):
                return None, 0, off
            return proj[bi].data_ptr(), proj[bi].numel(), off
        qp, ql, qo = span(q)
        kp, kl, ko = span(k)
        vp_, vl, vo = span(v)
        _check(self._lib.llmtie_rope_cache_f16(
            self._h, qp, ql, qo, kp, kl, ko, vp_, vl, vo, _ptr(freq_div), heads, kv_heads,
            head_dim, theta, pos, kc.data_ptr(), kc.numel(), vc.data_ptr(), vc.numel(), cap))

    def rope_cache_batched(self, q, k, v, freq_div, heads, kv_heads, head_dim, theta, pos, kcs,
                           vcs, cap) -> None:
        """`rope_cache_f16` for a batch of sequences in one launch."""
        _check(self._lib.llmtie_rope_cache_batched(
            self._h, q.data_ptr(), q.numel(), k.data_ptr(), k.numel(), v.data_ptr(), v.numel(),
            _ptr(freq_div), len(kcs), heads, kv_heads, head_dim, theta, self._i32_table(pos),
            self._ptr_table(kcs), self._ptr_table(vcs), self._i32_table(cap)))

    # ---- KV cache ---------------------------------------------------------------

    def cache_append_f16(self, src, src_off, dst, n, kv_heads, head_dim, cap, past,
                         transposed) -> None:
        _check(self._lib.llmtie_cache_append_f16(
            self._h, src.data_ptr(), src.numel(), src_off, dst.data_ptr(), dst.numel(), n,
            kv_heads, head_dim, cap, past, int(bool(transposed))))

    def cache_append(self, src, src_off, dst, n, kv_heads, head_dim, cap, past,
                     transposed) -> None:
        _check(self._lib.llmtie_cache_append(
            self._h, src.data_ptr(), src.numel(), src_off, dst.data_ptr(), dst.numel(), n,
            kv_heads, head_dim, cap, past, int(bool(transposed))))

    def cache_grow_f16(self, src, dst, kv_heads, head_dim, old_cap, new_cap, live,
                       transposed) -> None:
        _check(self._lib.llmtie_cache_grow_f16(
            self._h, src.data_ptr(), src.numel(), dst.data_ptr(), dst.numel(), kv_heads,
            head_dim, old_cap, new_cap, live, int(bool(transposed))))

    def cache_grow(self, src, dst, kv_heads, head_dim, old_cap, new_cap, live,
                   transposed) -> None:
        _check(self._lib.llmtie_cache_grow(
            self._h, src.data_ptr(), src.numel(), dst.data_ptr(), dst.numel(), kv_heads,
            head_dim, old_cap, new_cap, live, int(bool(transposed))))

    # ---- the projection in front of decode attention ---------------------------------

    def gemv_qkv_f16(self, a, w, bias, k, d, head_dim, cap, pos, q, kc, vc) -> None:
        """`gemv_qkv_f16` (device.rs:4393-4479): `bias` is three f32 [d] tensors
        or Nones, for q, k and v."""
        bq, bk, bv = bias
        blen = min([b.numel() for b in bias if b is not None], default=0)
        _check(self._lib.llmtie_gemv_qkv_f16(
            self._h, a.data_ptr(), a.numel(), w.data_ptr(), w.numel(), _ptr(bq), _ptr(bk), _ptr(bv),
            blen, k, d, head_dim, cap, pos, q.data_ptr(), q.numel(), kc.data_ptr(), kc.numel(),
            vc.data_ptr(), vc.numel()))

    # ---- Whisper cross-attention cache ----------------------------------------------

    def split_heads_f16_at(self, x, x_off, bias, t, heads, head_dim, cap=None,
                           transposed=False) -> torch.Tensor:
        """`split_heads_f16_at` / `split_heads_t_f16_at` (device.rs:5636-5665):
        `bias` is None or (buffer, offset). Returns a zeroed f16 cache of
        capacity `cap` (t when not given) with the block in it."""
        cap = t if cap is None else cap
        out = self.zeros_f16(heads * cap * head_dim)
        b, boff = (None, 0) if bias is None else bias
        _check(self._lib.llmtie_split_heads_f16_at(
            self._h, x.data_ptr(), x.numel(), x_off, _ptr(b), 0 if b is None else b.numel(), boff,
            out.data_ptr(), out.numel(), t, heads, head_dim, cap, int(bool(transposed))))
        return out

    def split_heads_t_f16_at(self, x, x_off, bias, t, heads, head_dim, cap=None) -> torch.Tensor:
        return self.split_heads_f16_at(x, x_off, bias, t, heads, head_dim, cap, transposed=True)

    def cross_kv_build(self, k_all, v_all, v_bias, layers, t, heads, head_dim, cap):
        """Every decoder layer's cross-attention caches in two launches (see
        include/llmtie_b200.h). Returns (k, v): f16 [layers][heads][cap][hd]
        and [layers][heads][hd][cap]."""
        n = layers * heads * cap * head_dim
        k, v = self.zeros_f16(n), self.zeros_f16(n)
        _check(self._lib.llmtie_cross_kv_build(
            self._h, k_all.data_ptr(), k_all.numel(), v_all.data_ptr(), v_all.numel(),
            _ptr(v_bias), 0 if v_bias is None else v_bias.numel(), k.data_ptr(), k.numel(),
            v.data_ptr(), v.numel(), layers, t, heads, head_dim, cap))
        return k, v

    # ---- prefill / encoder --------------------------------------------------------

    def supports_flash(self, head_dim, heads, kv_heads) -> bool:
        return bool(self._lib.llmtie_supports_flash(head_dim, heads, kv_heads))

    def flash_attn(self, q, k, v, tq, past, heads, kv_heads, head_dim, cap, scale,
                   causal) -> torch.Tensor:
        out = self.uninit(tq * heads * head_dim)
        _check(self._lib.llmtie_flash_attn(
            self._h, q.data_ptr(), q.numel(), k.data_ptr(), k.numel(), v.data_ptr(), v.numel(),
            out.data_ptr(), out.numel(), tq, past, heads, kv_heads, head_dim, cap, scale,
            int(bool(causal))))
        return out

    def flash_attn_f16(self, q, k, v, tq, past, heads, kv_heads, head_dim, cap, scale,
                       causal) -> torch.Tensor:
        out = self.uninit(tq * heads * head_dim)
        _check(self._lib.llmtie_flash_attn_f16(
            self._h, q.data_ptr(), q.numel(), k.data_ptr(), k.numel(), v.data_ptr(), v.numel(),
            out.data_ptr(), out.numel(), tq, past, heads, kv_heads, head_dim, cap, scale,
            int(bool(causal))))
        return out

    def flash_attn_rows(self, qkv, t, heads, head_dim, scale) -> torch.Tensor:
        out = self._empty(t * heads * head_dim, torch.float16)
        _check(self._lib.llmtie_flash_attn_rows(
            self._h, qkv.data_ptr(), qkv.numel(), out.data_ptr(), out.numel(), t, heads,
            head_dim, scale, None, 0))
        return out

    def flash_attn_rows_batched(self, qkv, batch, t, heads, head_dim, scale, work=None,
                                out=None) -> torch.Tensor:
        """`flash_attn_rows` for `batch` utterances of one length in two launches:
        qkv f32 [batch][t][3d] -> f16 [batch][t][d]."""
        if out is None:
            out = self._empty(batch * t * heads * head_dim, torch.float16)
        _check(self._lib.llmtie_flash_attn_rows_batched(
            self._h, qkv.data_ptr(), qkv.numel(), out.data_ptr(), out.numel(), batch, t, heads,
            head_dim, scale, _ptr(work), 0 if work is None else work.numel() * work.element_size()))
        return out

    # ---- decode ----------------------------------------------------------------------

    def attn_decode_f16(self, q, k, v, heads, kv_heads, head_dim, tk, cap, scale, scale_q,
                        scratch: DecodeScratch) -> torch.Tensor:
        out = self.uninit(heads * head_dim)
        self.attn_decode_f16_row(q, 0, k, v, heads, kv_heads, head_dim, tk, cap, scale, scale_q,
                                 scratch, out, 0)
        return out

    def attn_decode_f16_row(self, q, q_off, k, v, heads, kv_heads, head_dim, tk, cap, scale,
                            scale_q, scratch: DecodeScratch, out, row) -> None:
        """`attn_decode_f16_q_row` without the int8 twin (device.rs:6001-6038)."""
        _check(self._lib.llmtie_attn_decode_f16(
            self._h, q.data_ptr(), q.numel(), q_off, k.data_ptr(), k.numel(), v.data_ptr(),
            v.numel(), heads, kv_heads, head_dim, tk, cap, scale, int(bool(scale_q)),
            scratch._bind(self), out.data_ptr(), out.numel(), row * heads * head_dim))

    def q8_zeros(self, rows: int, width: int):
        """An empty int8 twin for `rows` rows of `width` (device.rs `q8_zeros`):
        codes int8 [rows*width] and scales f32 [rows*width/32]."""
        with torch.cuda.stream(self.stream):
            return (torch.zeros(rows * width, dtype=torch.int8, device=self.device),
                    torch.zeros(rows * width // 32, dtype=torch.float32, device=self.device))

    def attn_decode_f16_q(self, q, k, v, heads, kv_heads, head_dim, tk, cap, scale, scale_q,
                          scratch: DecodeScratch):
        """`attn_decode_f16_q` (device.rs:5973-5991): the context and its int8
        twin (codes, scales)."""
        out = self.uninit(heads * head_dim)
        twin = self.q8_zeros(1, heads * head_dim)
        self.attn_decode_f16_q_row(q, 0, k, v, heads, kv_heads, head_dim, tk, cap, scale, scale_q,
                                   scratch, out, twin, 0)
        return out, twin

    def attn_decode_f16_q_row(self, q, q_off, k, v, heads, kv_heads, head_dim, tk, cap, scale,
                              scale_q, scratch: DecodeScratch, out, twin, row) -> None:
        """`attn_decode_f16_q_row` (device.rs:6001-6038): row `row` of `out` and of
        the twin, which are shared by the batch and filled a row at a time."""
        codes, scales = twin
        _check(self._lib.llmtie_attn_decode_f16_q(
            self._h, q.data_ptr(), q.numel(), q_off, k.data_ptr(), k.numel(), v.data_ptr(),
            v.numel(), heads, kv_heads, head_dim, tk, cap, scale, int(bool(scale_q)),
            scratch._bind(self), out.data_ptr(), out.numel(), row * heads * head_dim,
            codes.data_ptr(), codes.numel(), scales.data_ptr(), scales.numel()))

    def attn_decode_f16_noalloc(self, q, k, v, heads, kv_heads, head_dim, tk, cap, scale,
                                scale_q, out=None) -> torch.Tensor:
        """`attn_decode_f16` for callers that cannot allocate: no DecodeScratch,
        the partials live in a static array inside the library. The output
        buffer is still the caller's; pass `out` to keep this call free of any
        allocation. Calls must not overlap on the GPU (they share the array)."""
        if out is None:
            out = self.uninit(heads * head_dim)
        _check(self._lib.llmtie_attn_decode_f16_noalloc(
            self._h, q.data_ptr(), q.numel(), 0, k.data_ptr(), k.numel(), v.data_ptr(),
            v.numel(), heads, kv_heads, head_dim, tk, cap, scale, int(bool(scale_q)),
            out.data_ptr(), out.numel(), 0))
        return out

    def attn_decode(self, q, k, v, heads, kv_heads, head_dim, tk, cap, scale, scale_q,
                    scratch: DecodeScratch) -> torch.Tensor:
        out = self.uninit(heads * head_dim)
        _check(self._lib.llmtie_attn_decode(
            self._h, q.data_ptr(), q.numel(), 0, k.data_ptr(), k.numel(), v.data_ptr(),
            v.numel(), heads, kv_heads, head_dim, tk, cap, scale, int(bool(scale_q)),
            scratch._bind(self), out.data_ptr(), out.numel(), 0))
        return out

    # ---- batched / sharded supersets -------------------------------------------------------

    # The batched entries take HOST tables. A caller that makes the same call
    # every step can build them once (`ptr_table`, `i32_table`) and pass the
    # tables where the lists would go.
    @staticmethod
    def _ptr_table(tensors) -> C.Array:
        if isinstance(tensors, C.Array):
            return tensors
        return (C.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])

    @staticmethod
    def _i32_table(xs) -> C.Array:
        if isinstance(xs, C.Array):
            return xs
        return (C.c_int32 * len(xs))(*[int(x) for x in xs])

    ptr_table = _ptr_table
    i32_table = _i32_table

    def decode_batched(self, q, ks, vs, tk, cap, heads, kv_heads, head_dim, scale, scale_q,
                       scratch: DecodeScratch, out=None, partial=False) -> torch.Tensor:
        batch = len(ks)
        width = heads * (head_dim + 2) if partial else heads * head_dim
        if out is None:
            out = self.uninit(batch * width)
        _check(self._lib.llmtie_decode_batched(
            self._h, q.data_ptr(), q.numel(), self._ptr_table(ks), self._ptr_table(vs),
            self._i32_table(tk), self._i32_table(cap), batch, heads, kv_heads, head_dim, scale,
            int(bool(scale_q)), scratch._bind(self), out.data_ptr(), out.numel(),
            int(bool(partial))))
        return out

    def decode_batched_push(self, q, ks, vs, tk, cap, heads, kv_heads, head_dim, scale, scale_q,
                            scratch: DecodeScratch, xch: Exchange) -> None:
        """Decodes this rank's slices and pushes the triples into every rank's
        gather buffer over peer memory (see include/llmtie_b200.h)."""
        _check(self._lib.llmtie_decode_batched_push(
            self._h, q.data_ptr(), q.numel(), self._ptr_table(ks), self._ptr_table(vs),
            self._i32_table(tk), self._i32_table(cap), len(ks), heads, kv_heads, head_dim, scale,
            int(bool(scale_q)), scratch._bind(self), xch.ref()))

    def decode_batched_fused(self, q, ks, vs, tk, cap, heads, kv_heads, head_dim, scale, scale_q,
                             scratch: DecodeScratch, xch: Exchange, out=None) -> torch.Tensor:
        """The sharded step in one kernel: decode, push, wait and merge
        (see include/llmtie_b200.h). Returns the merged [batch*heads*hd]."""
        if xch.pair_flags is None:
            raise ValueError("the fused exchange needs per-pair flags")
        if out is None:
            out = self.uninit(len(ks) * heads * head_dim)
        _check(self._lib.llmtie_decode_batched_fused(
            self._h, q.data_ptr(), q.numel(), self._ptr_table(ks), self._ptr_table(vs),
            self._i32_table(tk), self._i32_table(cap), len(ks), heads, kv_heads, head_dim, scale,
            int(bool(scale_q)), scratch._bind(self), xch.ref(), xch.pair_flags, out.data_ptr(),
            out.numel()))
        return out

    def decode_batched_signal(self, q, ks, vs, tk, cap, heads, kv_heads, head_dim, scale, scale_q,
                              scratch: DecodeScratch, xch: Exchange) -> None:
        """Decode, push, and a flag per (sequence, KV head) pair (see
        include/llmtie_b200.h); `lse_merge_pairs` follows it."""
        if xch.pair_flags is None:
            raise ValueError("this exchange needs per-pair flags")
        _check(self._lib.llmtie_decode_batched_signal(
            self._h, q.data_ptr(), q.numel(), self._ptr_table(ks), self._ptr_table(vs),
            self._i32_table(tk), self._i32_table(cap), len(ks), heads, kv_heads, head_dim, scale,
            int(bool(scale_q)), scratch._bind(self), xch.ref(), xch.pair_flags))

    def lse_merge_pairs(self, xch: Exchange, merge_step, rows, rows_per_pair, head_dim,
                        out=None) -> torch.Tensor:
        if out is None:
            out = self.uninit(rows * head_dim)
        _check(self._lib.llmtie_lse_merge_pairs(
            self._h, xch.ref(), xch.pair_flags[xch.rank], merge_step.data_ptr(), rows,
            rows_per_pair, head_dim, out.data_ptr(), out.numel()))
        return out

    def lse_merge_wait(self, xch: Exchange, rows, head_dim, out=None) -> torch.Tensor:
        if out is None:
            out = self.uninit(rows * head_dim)
        _check(self._lib.llmtie_lse_merge_wait(self._h, xch.ref(), rows, head_dim,
                                               out.data_ptr(), out.numel()))
        return out

    def lse_merge(self, parts_buf, parts, rows, head_dim, out=None) -> torch.Tensor:
        if out is None:
            out = self.uninit(rows * head_dim)
        _check(self._lib.llmtie_lse_merge(self._h, parts_buf.data_ptr(), parts_buf.numel(),
                                          parts, rows, head_dim, out.data_ptr(), out.numel()))
        return out

    def cross_attn(self, q, k, v, n, heads, head_dim, tk, cap, scale,
                   scratch: DecodeScratch) -> torch.Tensor:
        out = self.uninit(n * heads * head_dim)
        _check(self._lib.llmtie_cross_attn(
            self._h, q.data_ptr(), q.numel(), k.data_ptr(), k.numel(), v.data_ptr(), v.numel(),
            n, heads, head_dim, tk, cap, scale, scratch._bind(self), out.data_ptr(),
            out.numel()))
        return out

    def prefill_varlen(self, q, k, v, cu_seqlens, kcs, vcs, past, cap, freq_div, heads,
                       kv_heads, head_dim, theta, scale, out=None) -> torch.Tensor:
        batch = len(kcs)
        total = int(cu_seqlens[batch])
        if out is None:
            out = self.uninit(total * heads * head_dim)
        _check(self._lib.llmtie_prefill_varlen(
            self._h, q.data_ptr(), q.numel(), k.data_ptr(), k.numel(), v.data_ptr(), v.numel(),
            self._i32_table(cu_seqlens), batch, self._ptr_table(kcs), self._ptr_table(vcs),
            self._i32_table(past), self._i32_table(cap), _ptr(freq_div), heads, kv_heads,
            head_dim, theta, scale, out.data_ptr(), out.numel()))
        return out

    # ---- profiling ------------------------------------------------------------------------

    def kprof_enable(self, on: bool = True) -> None:
        self._lib.llmtie_kprof_enable(self._h, int(on))

    def kprof_reset(self) -> None:
        self._lib.llmtie_kprof_reset(self._h)

    def kprof_report(self) -> dict:
        need = self._lib.llmtie_kprof_report(self._h, None, 0)
        buf = C.create_string_buffer(int(need) + 1)
        self._lib.llmtie_kprof_report(self._h, buf, len(buf))
        rep = {}
        for line in buf.value.decode().splitlines():
            name, count, ms = line.rsplit(" ", 2)
            rep[name] = (int(count), float(ms))
        return rep

    def kernel_resources(self, name: str):
        regs, local, smem = C.c_int32(), C.c_int32(), C.c_int32()
        st = self._lib.llmtie_kernel_resources(name.encode(), C.byref(regs), C.byref(local),
                                               C.byref(smem))
        if st != 0:
            return None
        return regs.value, local.value, smem.value

    def launch_count(self) -> int:
        return int(self._lib.llmtie_launch_count(self._h))
