"""The f16 KV cache of one layer and its growth policy.

`KvCache` is what `Cache`/`LayerCache` are in the model crates
(crates/llmtie-chat/src/model.rs:200-262, :714-747;
crates/llmtie-translate/src/model.rs:662-694): keys `[kv_heads][cap][hd]`,
values transposed `[kv_heads][hd][cap]`, both zeroed at allocation, capacity
a power of two of at least 256 that doubles by re-striding, `truncate` only
lowering the live length.
"""
from __future__ import annotations

from . import _lib
from .gpu import Gpu


def want_capacity(cap: int, past: int, n: int, max_positions: int) -> int:
    """Capacity to allocate so a cache of `cap` holds past + n positions; 0 if
    it already does (chat/model.rs:714-721)."""
    return int(_lib.load().llmtie_kv_want_capacity(cap, past, n, max_positions))


class KvCache:
    def __init__(self, gpu: Gpu, kv_heads: int, head_dim: int, max_positions: int) -> None:
        self.gpu = gpu
        self.kv_heads = kv_heads
        self.head_dim = head_dim
        self.max_positions = max_positions
        self.cap = 0
        self.len = 0
        self.k = None
        self.v = None

    def reserve(self, n: int) -> None:
        """Makes room for n more positions, growing by re-stride when needed."""
        want = want_capacity(self.cap, self.len, n, self.max_positions)
        if want == 0:
            return
        g = self.gpu
        kv_dim = self.kv_heads * self.head_dim
        k = g.zeros_f16(want * kv_dim)
        v = g.zeros_f16(want * kv_dim)
        if self.len > 0:
            g.cache_grow_f16(self.k, k, self.kv_heads, self.head_dim, self.cap, want, self.len,
                             False)
            g.cache_grow_f16(self.v, v, self.kv_heads, self.head_dim, self.cap, want, self.len,
                             True)
        self.k, self.v, self.cap = k, v, want

    def append(self, k_src, v_src, src_off_k: int, src_off_v: int, n: int) -> None:
        """Appends n positions of projected (already rotated) k and v."""
        self.reserve(n)
        g = self.gpu
        g.cache_append_f16(k_src, src_off_k, self.k, n, self.kv_heads, self.head_dim, self.cap,
                           self.len, False)
        g.cache_append_f16(v_src, src_off_v, self.v, n, self.kv_heads, self.head_dim, self.cap,
                           self.len, True)
        self.len += n

    def truncate(self, length: int) -> None:
        """Forgets every position from `length` on. Nothing is zeroed: attention
        reads only the live positions, and the next prefill writes its own keys
        and values from `length` before any attention reads them."""
        self.len = min(self.len, length)

    def clear(self) -> None:
        self.len = 0


def shared_prefix(held, ids) -> int:
    """Leading tokens of `ids` that a cache holding `held` can keep (never all
    of `ids`: the last token is always run)."""
    import ctypes as C

    h = (C.c_uint32 * len(held))(*held)
    i = (C.c_uint32 * len(ids))(*ids)
    return int(_lib.load().llmtie_kv_shared_prefix(h, len(held), i, len(ids)))


class Prefix:
    """`Prefix` (crates/llmtie-chat/src/generate.rs:258-283): the caches of one
    conversation kept from one completion to the next, with exactly the tokens
    they hold. A turn's prompt shares its opening with the last one, so only
    the tokens from the first that differs are prefilled."""

    def __init__(self, caches) -> None:
        self.caches = list(caches)          # one KvCache a layer
        self.held: list[int] = []

    def __len__(self) -> int:
        return len(self.held)

    def shared_with(self, ids) -> int:
        n = 0
        for a, b in zip(self.held, ids):
            if a != b:
                break
            n += 1
        return n

    def keep(self, ids) -> int:
        """Cuts the caches back to what they share with the prompt `ids`
        (generate.rs:139-141) and returns that length: the prompt is prefilled
        from there, with `past` = the returned value."""
        reused = shared_prefix(self.held, ids)
        for c in self.caches:
            c.truncate(reused)
        del self.held[reused:]
        return reused

    def extend(self, ids) -> None:
        """Records tokens the caches now hold (after a prefill or a decoded step)."""
        self.held.extend(int(x) for x in ids)

    def reset(self) -> None:
        """What complete_after does when a completion failed half way."""
        for c in self.caches:
            c.clear()
        self.held.clear()
