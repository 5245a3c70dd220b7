"""One long context spread over several GPUs.

The reference has no multi-GPU scheme; it scales a sequence inside one GPU by
splitting the keys over blocks and merging partial (o, m, l) triples
(crates/llmtie-cuda/src/kernels.rs:5779-5903, :6166-6175). This lifts the
same algebra one level: every rank holds a contiguous slice of each
sequence's KV positions in its own cache, decodes its slice into
un-normalised triples, one all-gather moves the triples (a few hundred KB),
and every rank merges them locally. Prefill shards by KV head instead and
needs no exchange at all.

One process per GPU; `torch.distributed` carries the all-gather (NCCL on
GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch
import torch.distributed as dist


def shard_bounds(tk: int, world: int, rank: int, align: int = 8) -> tuple[int, int]:
    """Positions [t0, t1) of a tk-long sequence that `rank` holds: contiguous,
    even to within `align`, and aligned so that every slice's value rows keep
    16-byte alignment in its own cache."""
    per = -(-tk // world)
    per = -(-per // align) * align
    t0 = min(tk, rank * per)
    t1 = min(tk, t0 + per)
    return t0, t1


def kv_head_shard(kv_heads: int, world: int, rank: int) -> tuple[int, int]:
    """KV heads [h0, h1) `rank` takes when a prefill is split by KV head
    (its query heads are h0*group .. h1*group). Needs world <= kv_heads."""
    if world > kv_heads:
        raise ValueError(f"{world} ranks cannot split {kv_heads} KV heads")
    per, extra = divmod(kv_heads, world)
    h0 = rank * per + min(rank, extra)
    return h0, h0 + per + (1 if rank < extra else 0)


class ShardedDecode:
    """Decode attention over KV slices held by the ranks of `group`.

    `partial_fn(q, partial) -> tensor` computes this rank's result for its
    slice: normalised [batch, heads*hd] when the world is one rank, else the
    triples [batch, heads, hd+2]. `merge_fn(gathered, parts, rows) -> tensor`
    merges [parts][rows][hd+2]. Both default to the GPU entry points; the CPU
    tests inject host implementations to exercise the exchange itself.
    """

    def __init__(self, heads: int, head_dim: int, group: Optional[dist.ProcessGroup] = None,
                 partial_fn: Optional[Callable] = None, merge_fn: Optional[Callable] = None,
                 stream: Optional[torch.cuda.Stream] = None) -> None:
        self.heads = heads
        self.head_dim = head_dim
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.partial_fn = partial_fn
        self.merge_fn = merge_fn
        self.stream = stream
        self._gathered = None
        self._fused = None
        self.exchange = "none" if self.world == 1 else "all-gather"

    @classmethod
    def on_gpu(cls, gpu, ks: Sequence[torch.Tensor], vs: Sequence[torch.Tensor],
               tk: Sequence[int], cap: Sequence[int], heads: int, kv_heads: int, head_dim: int,
               scale: float, scale_q: bool = False, group=None, p2p=False
               ) -> "ShardedDecode":
        """Binds the GPU entry points over this rank's caches. With `p2p` the
        exchange is fused into the kernels, no collective call in the step.
        "push" (or True): the decode kernel stores its triples into every
        rank's gather buffer over NVLink peer memory and a second, waiting
        kernel merges - the fastest measured (117 us a step on 8 GPUs against
        120 us for "fused" and 141 us for the all-gather). "fused": the whole
        step is one kernel; the block that finished a pair waits for the other
        ranks' triples of it and merges."""
        from .gpu import DecodeScratch

        scratch = DecodeScratch()
        batch = len(ks)
        outs = {}
        # the same tables every step: built once (the tensors stay referenced here)
        keep = (list(ks), list(vs))
        ks, vs = gpu.ptr_table(ks), gpu.ptr_table(vs)
        tk, cap = gpu.i32_table(tk), gpu.i32_table(cap)
        if p2p and dist.is_initialized() and dist.get_world_size(group) > 1:
            # Every rank must take the same path: if symmetric memory cannot be
            # set up on any one of them, all fall back to the all-gather.
            fused, why = None, ""
            try:
                fused = cls._on_gpu_p2p(gpu, ks, vs, tk, cap, heads, kv_heads, head_dim, scale,
                                        scale_q, group, scratch,
                                        one_kernel=("pairs" if p2p == "pairs" else p2p == "fused"))
            except (ImportError, RuntimeError, AttributeError) as e:
                why = str(e)
            ok = torch.tensor([1 if fused is not None else 0], dtype=torch.int32,
                              device=gpu.device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
            if int(ok.item()) == 1:
                fused._caches = keep
                return fused
            if dist.get_rank(group) == 0:
                import warnings
                warnings.warn("peer-memory exchange unavailable (%s); using the all-gather"
                              % (why or "another rank failed"))

        def partial_fn(q, partial):
            width = heads * (head_dim + 2) if partial else heads * head_dim
            if partial not in outs:
                outs[partial] = gpu.uninit(batch * width)
            return gpu.decode_batched(q, ks, vs, tk, cap, heads, kv_heads, head_dim, scale,
                                      scale_q, scratch, out=outs[partial], partial=partial)

        merged = {}

        def merge_fn(gathered, parts, rows):
            if "out" not in merged:
                merged["out"] = gpu.uninit(rows * head_dim)
            return gpu.lse_merge(gathered, parts, rows, head_dim, out=merged["out"])

        self = cls(heads, head_dim, group, partial_fn, merge_fn, gpu.stream)
        self._scratch = scratch
        self._caches = keep
        self.exchange = "none" if self.world == 1 else "all-gather"
        return self

    @classmethod
    def _on_gpu_p2p(cls, gpu, ks, vs, tk, cap, heads, kv_heads, head_dim, scale, scale_q, group,
                    scratch, one_kernel=True) -> "ShardedDecode":
        import torch.distributed._symmetric_memory as symm_mem

        from .gpu import Exchange

        world = dist.get_world_size(group)
        rank = dist.get_rank(group)
        batch = len(ks)
        rows = batch * heads
        pg = group if group is not None else dist.group.WORLD
        with torch.cuda.stream(gpu.stream):
            # [2 steps in flight][world][rows][hd + 2] triples, then the flags
            gather = symm_mem.empty(2 * world * rows * (head_dim + 2), dtype=torch.float32,
                                    device=gpu.device)
            flags = symm_mem.empty(64, dtype=torch.int32, device=gpu.device)
            pflags = symm_mem.empty(max(64, batch * kv_heads * world), dtype=torch.int32,
                                    device=gpu.device)
            gather.zero_()
            flags.zero_()
            pflags.zero_()
            step = torch.zeros(1, dtype=torch.int32, device=gpu.device)
            mstep = torch.zeros(2, dtype=torch.int32, device=gpu.device)
            out = torch.empty(rows * head_dim, dtype=torch.float32, device=gpu.device)
        gh = symm_mem.rendezvous(gather, pg)
        fh = symm_mem.rendezvous(flags, pg)
        ph = symm_mem.rendezvous(pflags, pg)
        torch.cuda.synchronize()
        dist.barrier(group)
        xch = Exchange(world, rank, [int(p) for p in gh.buffer_ptrs],
                       [int(p) for p in fh.buffer_ptrs], step.data_ptr(),
                       [int(p) for p in ph.buffer_ptrs])

        self = cls(heads, head_dim, group, None, None, gpu.stream)
        self._keep = (gather, flags, pflags, step, mstep, gh, fh, ph, xch, scratch, out)

        if one_kernel == "pairs":
            def fused(q):
                gpu.decode_batched_signal(q, ks, vs, tk, cap, heads, kv_heads, head_dim, scale,
                                          scale_q, scratch, xch)
                return gpu.lse_merge_pairs(xch, mstep, rows, heads // kv_heads, head_dim, out=out)
        elif one_kernel:
            def fused(q):
                return gpu.decode_batched_fused(q, ks, vs, tk, cap, heads, kv_heads, head_dim,
                                                scale, scale_q, scratch, xch, out=out)
        else:
            def fused(q):
                gpu.decode_batched_push(q, ks, vs, tk, cap, heads, kv_heads, head_dim, scale,
                                        scale_q, scratch, xch)
                return gpu.lse_merge_wait(xch, rows, head_dim, out=out)

        self._fused = fused
        # the attention kernel alone, for timing: triples into a local buffer
        local = {}

        def partial_fn(q, partial):
            width = heads * (head_dim + 2) if partial else heads * head_dim
            if partial not in local:
                local[partial] = gpu.uninit(batch * width)
            return gpu.decode_batched(q, ks, vs, tk, cap, heads, kv_heads, head_dim, scale,
                                      scale_q, scratch, out=local[partial], partial=partial)

        self.partial_fn = partial_fn
        self.exchange = ("peer-pairs" if one_kernel == "pairs"
                         else "peer-fused" if one_kernel else "peer-push")
        return self

    def decode(self, q: torch.Tensor) -> torch.Tensor:
        """q: [batch, heads*hd] (rotated), the same on every rank. Returns the
        attention output [batch*heads*hd] on every rank."""
        if getattr(self, "_fused", None) is not None:
            return self._fused(q)
        if self.world == 1:
            return self.partial_fn(q, False)
        part = self.partial_fn(q, True)
        if self._gathered is None or self._gathered.numel() != part.numel() * self.world:
            self._gathered = torch.empty(part.numel() * self.world, dtype=part.dtype,
                                         device=part.device)
        if self.stream is not None:
            with torch.cuda.stream(self.stream):
                dist.all_gather_into_tensor(self._gathered, part.reshape(-1), group=self.group)
        else:
            dist.all_gather_into_tensor(self._gathered, part.reshape(-1), group=self.group)
        rows = part.numel() // (self.head_dim + 2)
        return self.merge_fn(self._gathered, self.world, rows)

    def capture(self, q: torch.Tensor):
        """Records one decode step (attention, all-gather, merge) over the
        fixed buffer `q` into a CUDA graph on the handle's stream and returns
        (graph, out): `graph.replay()` re-runs the step with whatever `q` holds
        then, at one launch's host cost. The step is run once uncaptured first
        so that every buffer it needs exists before capture begins."""
        if self.stream is None:
            raise RuntimeError("capture needs the GPU binding (ShardedDecode.on_gpu)")
        self.decode(q)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=self.stream):
            out = self.decode(q)
        return graph, out
