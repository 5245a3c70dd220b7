#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload NAME]

The default workload is the long-context decode of the benchmark contract:
batch 8, context 131072 per sequence, 32 Q / 8 KV heads, head_dim 128, f16 KV
cache, the KV sequence split evenly over the N GPUs, an all-gather of the
partial (O, max, sum) triples and a log-sum-exp merge (strong scaling: the
total work is fixed as N grows). One step is one pass of decode attention
over the whole batch (one layer). Inputs are seeded synthetic tensors drawn
N(0,1) and rounded to f16; the KV cache is far larger than L2, so no flush is
needed between iterations.

`value` is whole-job KV bytes per second with everything resident in HBM;
`e2e` is the same metric through the C ABI with host buffers: the step's
q/k/v projections copied from pinned host memory, RoPE and the cache write,
attention, and the context read back. The CPU arm (`--impl reference`, and the
`cpu_baseline` object of the default arm) times the C restatement of the
reference's own scalar attention on the host cores.

The same line carries a `prefill` object: the causal 8192-position prefill of
the same contract, split by KV head over the N GPUs with no exchange, in
TFLOP/s against the tensor-pipe roofline, with its own end-to-end and CPU
figures; a few of its rows are checked against the CPU oracle before it is
timed. `sustained` repeats the decode step for at least two seconds, the
regime in which the part runs into its power cap.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HEADS, KV_HEADS, HD = 32, 8, 128
SCALE = float(np.float32(HD) ** np.float32(-0.5))
FALLBACK_HBM_GBS = 6650.0
FALLBACK_TFLOPS = 1590.0
FALLBACK_TFLOPS_SUSTAINED = 1400.0
# dram__bytes_read.sum + dram__bytes_write.sum of one prefill_tc_kernel<128>
# launch at 8192 positions, from the capture summarised in
# profiles/prefill_tc_kernel_seq8192.md (194.05 MB read + 98.96 MB written).
PREFILL_DRAM_BYTES_8K = 194.047e6 + 98.964e6

# DRAM traffic of the dominant kernel from the ncu captures summarised under
# profiles/. The decode entry is dram__bytes_read.sum + dram__bytes_write.sum
# per algorithmic byte, captured on a batch 8 x 16384-key launch (537.31 MB read
# + 4.40 MB written for 536.87 MB of KV) and scaled to the launch at hand, since
# traffic grows in proportion to the keys streamed; a full-size launch is too
# large to capture.
NCU_TRAFFIC = {
    "decode128k": (537.309e6 + 4.404e6) / 536.870912e6,
    # bytes per launch of the 8192-position prefill on one GPU (32 / 8 heads),
    # captured at that size; a rank holding fewer KV heads moves that share
    "prefill8k": PREFILL_DRAM_BYTES_8K,
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, FALLBACK_TFLOPS, "fallback"


def measured_sustained_tflops():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops_sustained"])
    except Exception:
        return FALLBACK_TFLOPS_SUSTAINED


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while a region is timed."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index = index
        self.rows = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "10"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            t0 = time.time()
            while not self.rows and time.time() - t0 < 5.0:
                time.sleep(0.02)   # nvidia-smi takes a moment to deliver its first row
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                pass

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                for name, cell in zip(names, r[5:9]):
                    if cell.lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                continue
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)),
                "reasons": sorted(reasons), "samples": len(sm)}


# ---- synthetic inputs ---------------------------------------------------------

def device_normal_f16(gpu, n: int, seed: int):
    """n i.i.d. N(0,1) values rounded to f16, generated on the device."""
    import torch

    with torch.cuda.stream(gpu.stream):
        gen = torch.Generator(device=gpu.device)
        gen.manual_seed(seed)
        out = torch.empty(n, dtype=torch.float16, device=gpu.device)
        step = 1 << 26
        for a in range(0, n, step):
            b = min(n, a + step)
            out[a:b] = torch.randn(b - a, generator=gen, device=gpu.device,
                                   dtype=torch.float32).to(torch.float16)
    return out


def dist_setup(n_gpus: int):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        # plain peer loads and stores only: no NVLink multicast objects
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    elif n_gpus > 1:
        raise SystemExit("bench.py --gpus N>1 must be launched with torch.distributed.run")
    return world, rank, local


def max_over_ranks(x: float, device) -> float:
    import torch
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size() == 1:
        return x
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier_sync(gpu):
    import torch
    import torch.distributed as dist

    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
    torch.cuda.synchronize()
    gpu.synchronize()


def time_steps(gpu, fn, steps: int, warmup: int) -> float:
    """Seconds for exactly `steps` calls of fn, CUDA events on the handle's
    stream, a barrier and a synchronize on both sides; max over ranks."""
    import torch

    for _ in range(warmup):
        fn()
    barrier_sync(gpu)
    with torch.cuda.stream(gpu.stream):
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
    barrier_sync(gpu)
    return max_over_ranks(e0.elapsed_time(e1) / 1e3, gpu.device)


# ---- workloads ------------------------------------------------------------------

def oracle_check_sharded_decode(gpu, q, out, ks, vs, tk, ctx, world, rank):
    """The merged output of the sharded step against the CPU oracle: every
    rank's slice of sequence 0, KV head 0 (keys [tk][hd], values [hd][tk]) is
    gathered, rank 0 lays them end to end (67 MB at 131072 keys) and runs the
    f64 oracle on that KV head's four query heads. Returns max-abs on rank 0,
    None elsewhere (and None when the slices are not all the same length)."""
    import torch
    import torch.distributed as dist

    from oracle import oracle as O

    group = HEADS // KV_HEADS
    if world > 1 and ctx % (8 * world) != 0:
        return None
    with torch.cuda.stream(gpu.stream):
        kslice = ks[0][:tk * HD].contiguous()                         # head 0: [tk][hd]
        vslice = vs[0][:HD * tk].contiguous()                         # head 0: [hd][tk]
        mine = torch.cat([kslice, vslice])
        if world > 1:
            allk = torch.empty(world * mine.numel(), dtype=mine.dtype, device=mine.device)
            dist.all_gather_into_tensor(allk, mine)
        else:
            allk = mine
        gpu.synchronize()
        host = allk.cpu().view(torch.int16).numpy().view(np.uint16).reshape(world, 2, tk * HD)
        got = out[:group * HD].cpu().numpy()
        hq = q[:group * HD].cpu().numpy()
    if rank != 0:
        return None
    kfull = np.ascontiguousarray(host[:, 0, :].reshape(world * tk, HD)).reshape(-1)
    vfull = np.ascontiguousarray(
        host[:, 1, :].reshape(world, HD, tk).transpose(1, 0, 2)).reshape(-1)
    want = O.decode_f64(hq, kfull, vfull, group, 1, HD, 0, world * tk, world * tk, SCALE, False)
    return float(np.abs(want - got).max())


def decode128k(args, world, rank, local):
    """Config 5, decode: batch 8 x 131072 context, KV split over the ranks."""
    import torch

    from ttsxabe_b200 import Gpu
    from ttsxabe_b200.sharded import ShardedDecode, shard_bounds

    batch, ctx = args.batch, args.context
    gpu = Gpu.open(local)
    t0, t1 = shard_bounds(ctx, world, rank)
    tk = t1 - t0
    cap = tk
    ks = [device_normal_f16(gpu, KV_HEADS * cap * HD, 1000 + 17 * b + rank) for b in range(batch)]
    vs = [device_normal_f16(gpu, KV_HEADS * cap * HD, 5000 + 17 * b + rank) for b in range(batch)]
    with torch.cuda.stream(gpu.stream):
        gen = torch.Generator(device=gpu.device)
        gen.manual_seed(7)   # the same query on every rank
        q = torch.randn(batch * HEADS * HD, generator=gen, device=gpu.device)
        q = q.to(torch.float16).to(torch.float32)
    sd = ShardedDecode.on_gpu(gpu, ks, vs, [tk] * batch, [cap] * batch, HEADS, KV_HEADS, HD,
                              SCALE, p2p=False if args.exchange == "nccl" else args.exchange)
    gpu.synchronize()

    # The sharded paths have no single-GPU test to stand on, so the step is
    # checked here: against the CPU oracle on one KV head of one sequence, and
    # the fused exchange against the all-gather path on the same inputs.
    exchange_err = None
    fused_exchange = sd.exchange.startswith("peer-")
    with torch.cuda.stream(gpu.stream):
        first = sd.decode(q).clone()
    oracle_err = oracle_check_sharded_decode(gpu, q, first, ks, vs, tk, ctx, world, rank)
    if oracle_err is not None and not (oracle_err < 2e-5 * 4.0):
        raise SystemExit("decode disagrees with the CPU oracle: max-abs %g" % oracle_err)
    if fused_exchange:
        ref = ShardedDecode.on_gpu(gpu, ks, vs, [tk] * batch, [cap] * batch, HEADS, KV_HEADS, HD,
                                   SCALE, p2p=False)
        with torch.cuda.stream(gpu.stream):   # the copies must queue behind the kernels
            a = first
            b = sd.decode(q).clone()      # a second step: the other gather buffer
            c = ref.decode(q).clone()
            gpu.synchronize()
            exchange_err = float(max((a - c).abs().max().item(), (b - c).abs().max().item()))
        if not (exchange_err < 1e-5):
            bad = ((a - c).abs().reshape(batch * HEADS, HD).max(dim=1).values > 1e-5)
            sys.stderr.write("rank %d: %d of %d rows differ, first %s\n" % (
                rank, int(bad.sum().item()), batch * HEADS,
                bad.nonzero().flatten()[:16].tolist()))
            raise SystemExit("fused exchange disagrees with the all-gather path: %g" % exchange_err)

    # Kernels of ours per step: the attention kernel, and the merge when sharded.
    launches0 = gpu.launch_count()
    sd.decode(q)
    per_step = gpu.launch_count() - launches0
    step = lambda: sd.decode(q)
    if world > 1 and not args.no_graph:
        # At 8 GPUs a step is ~100 us of device work behind three host calls;
        # replaying it as a CUDA graph keeps the host out of the timed region.
        graph, _ = sd.capture(q)
        def step():
            with torch.cuda.stream(gpu.stream):
                graph.replay()
    clocks = ClockSampler(local)
    clocks.__enter__()
    secs = time_steps(gpu, step, args.steps, args.warmup)
    launches = per_step * args.steps

    # the attention kernel alone (what the roofline is about)
    ksecs = time_steps(gpu, lambda: sd.partial_fn(q, world > 1), args.steps, 3)

    kv_bytes_total = batch * 2 * KV_HEADS * ctx * HD * 2      # the reference's count
    kv_bytes_rank = batch * 2 * KV_HEADS * tk * HD * 2

    # ---- end to end through the C ABI with host buffers ------------------------
    nq, nkv = HEADS * HD, KV_HEADS * HD
    # one pinned staging buffer [q | k | v], so the step's inputs are one copy
    hqkv = torch.randn(batch * (nq + 2 * nkv)).pin_memory()
    hqkv[:batch * nq] = hqkv[:batch * nq].to(torch.float16).to(torch.float32)
    hout = torch.empty(batch * nq).pin_memory()
    dqkv = gpu.uninit(batch * (nq + 2 * nkv))
    dq = dqkv[:batch * nq]
    dk = dqkv[batch * nq:batch * (nq + nkv)]
    dv = dqkv[batch * (nq + nkv):]
    lib, h = gpu._lib, gpu._h
    pos = tk - 1          # the step's new token lands in the last cache slot
    esz = 4

    pos_t, cap_t = gpu.i32_table([pos] * batch), gpu.i32_table([cap] * batch)
    ks_t, vs_t = gpu.ptr_table(ks), gpu.ptr_table(vs)

    def e2e_enqueue():
        lib.llmtie_upload(h, dqkv.data_ptr(), hqkv.data_ptr(), batch * (nq + 2 * nkv) * esz)
        gpu.rope_cache_batched(dq, dk, dv, None, HEADS, KV_HEADS, HD, 10000.0, pos_t, ks_t, vs_t,
                               cap_t)
        return sd.decode(dqkv)         # q is the first batch*nq floats

    def e2e_step():
        out = e2e_enqueue()
        lib.llmtie_download(h, hout.data_ptr(), out.data_ptr(), batch * nq * esz)

    e2e_graph = not args.no_graph
    if e2e_graph:
        # The same calls - the copy in from pinned host memory, RoPE and the
        # cache write, attention, exchange and merge, the copy out - recorded
        # once and replayed; the step ends with the handle's synchronize.
        e2e_step()
        torch.cuda.synchronize()
        g2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g2, stream=gpu.stream):
            out = e2e_enqueue()
            hout.copy_(out, non_blocking=True)

        def e2e_step():
            with torch.cuda.stream(gpu.stream):
                g2.replay()
            gpu.synchronize()

    for _ in range(max(1, args.warmup)):
        e2e_step()
    barrier_sync(gpu)
    w0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    barrier_sync(gpu)
    e2e_secs = max_over_ranks((time.perf_counter() - w0), gpu.device) / args.steps
    clocks.__exit__()
    clk = clocks.summary()

    # ---- the same step for at least two seconds: the power-capped regime --------
    sus_steps = max(200, int(2.2 / max(secs / args.steps, 1e-6)))
    with ClockSampler(local) as sus_clocks:
        sus_secs = time_steps(gpu, step, sus_steps, 3)

    hbm, _, which = measured_peaks()
    per_step = secs / args.steps
    achieved = kv_bytes_rank / (ksecs / args.steps) / 1e9
    line = {
        "metric": "decode KV GB/s",
        "value": kv_bytes_total / per_step / 1e9,
        "unit": "GB/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": per_step * 1e3,
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "f16 KV cache, f32 accumulate",
        "data": "synthetic",
        "config": {
            "workload": WORKLOAD % (batch, ctx),
            "global_batch": batch,
            "context": ctx,
            "parallelism": "kv-seq-shard x%d" % world,
            "l2": "inputs (%.0f MB per GPU) exceed L2, no flush" % (kv_bytes_rank / 1e6),
        },
        "tokens_per_s": batch / per_step,
        "clocks": clk,
        "e2e": {
            "value": kv_bytes_total / e2e_secs / 1e9,
            "unit": "GB/s",
            "ms_per_step": e2e_secs * 1e3,
            "h2d_bytes_per_step": batch * (nq + 2 * nkv) * esz,
            "d2h_bytes_per_step": batch * nq * esz,
            "cuda_graph": e2e_graph,
        },
        "gpu_launches": int(launches),
        "cuda_graph": bool(world > 1 and not args.no_graph),
        "exchange": {"none": "none", "all-gather": "nccl all-gather",
                     "peer-push": "peer-memory push fused into the decode kernel, merge in a "
                                  "second waiting kernel",
                     "peer-pairs": "peer-memory push with a flag per (sequence, KV head) pair, "
                                   "merged by a kernel launched as the decode kernel's "
                                   "programmatic dependent",
                     "peer-fused": "peer-memory push, wait and merge all fused into the decode "
                                   "kernel"}[sd.exchange],
        "exchange_max_abs_vs_allgather": exchange_err,
        "exchange_max_abs_vs_oracle": oracle_err,
        "sustained": {
            "steps": sus_steps,
            "seconds": sus_secs,
            "ms_per_step": sus_secs / sus_steps * 1e3,
            "value": kv_bytes_total / (sus_secs / sus_steps) / 1e9,
            "unit": "GB/s",
            "frac_of_hbm_peak_per_gpu": kv_bytes_rank / (sus_secs / sus_steps) / 1e9 / hbm,
            "clocks": sus_clocks.summary(),
        },
        "roofline": {
            "bound": "hbm",
            "achieved": achieved,
            "peak": hbm,
            "unit": "GB/s",
            "frac": achieved / hbm,
            "traffic": (None if NCU_TRAFFIC["decode128k"] is None
                        else NCU_TRAFFIC["decode128k"] * kv_bytes_rank),
            "peak_source": "of " + which,
            "kernel": "decode_stream_kernel<128>",
            "kernel_ms": ksecs / args.steps * 1e3,
            "algorithmic_bytes_per_launch": kv_bytes_rank,
            "frac_of_nominal_8tbs": achieved / 8000.0,
        },
    }
    # free the 4.3 GB of cache before the prefill leg
    del sd, ks, vs
    return gpu, line


WORKLOAD = ("config 5 decode: batch %d, context %d per sequence, 32 Q / 8 KV heads, "
            "head_dim 128, f16 KV ~N(0,1), KV sequence split evenly over the GPUs, "
            "all-gather of (O, max, sum), LSE merge")


def cpu_prefill_sample(q_rows, kc, vc, rows, past, heads, kv, cap):
    """Times the oracle's threaded prefill on the last `rows` query rows of the
    sequence, every head. Returns (TFLOP/s, threads, seconds, output)."""
    from oracle import oracle as O

    t0 = time.perf_counter()
    out = np.empty(rows * heads * HD, dtype=np.float32)
    used = O.lib().orc_prefill_fast(q_rows.ctypes.data, heads * HD, kc.ctypes.data,
                                    vc.ctypes.data, 1, rows, past, 0, heads, kv, HD, cap, SCALE, 1,
                                    0, out.ctypes.data, heads * HD, 0)
    dt = time.perf_counter() - t0
    pairs = sum(past + r + 1 for r in range(rows))
    return 4.0 * HD * heads * pairs / dt / 1e12, int(used), dt, out


def prefill_leg(args, gpu, world, rank, local):
    """Config 5, prefill: causal, 8192 positions, split by KV head, no
    exchange. Returns the `prefill` object of the bench line."""
    import torch

    from oracle import oracle as O
    from ttsxabe_b200.sharded import kv_head_shard

    tq = args.seq
    h0, h1 = kv_head_shard(KV_HEADS, world, rank)
    kv = h1 - h0
    heads = kv * (HEADS // KV_HEADS)
    cap = tq
    kc = device_normal_f16(gpu, kv * cap * HD, 11 + rank)
    vc = device_normal_f16(gpu, kv * cap * HD, 13 + rank)
    n = tq * heads * HD
    hq = torch.randn(n).to(torch.float16).to(torch.float32).pin_memory()
    hout = torch.empty(n).pin_memory()
    q = gpu.uninit(n)
    out = gpu.uninit(n)
    lib, h = gpu._lib, gpu._h
    with torch.cuda.stream(gpu.stream):
        q.copy_(hq, non_blocking=True)

    def step():
        lib.llmtie_flash_attn_f16(h, q.data_ptr(), q.numel(), kc.data_ptr(), kc.numel(),
                                  vc.data_ptr(), vc.numel(), out.data_ptr(), out.numel(), tq, 0,
                                  heads, kv, HD, cap, SCALE, 1)

    # ---- a few rows against the CPU oracle before anything is timed -------------
    step()
    gpu.synchronize()
    parity = None
    cpu = None
    if rank == 0:
        hk = kc.cpu().view(torch.int16).numpy().view(np.uint16)
        hv = vc.cpu().view(torch.int16).numpy().view(np.uint16)
        got = out.cpu().numpy().reshape(tq, heads * HD)
        hq2 = hq.numpy().reshape(tq, heads * HD)
        worst_abs, worst_rel = 0.0, 0.0
        for r0 in sorted({0, tq // 2 - 1, tq - 16}):
            want = O.prefill(np.ascontiguousarray(hq2[r0:r0 + 16]), hk, hv, 16, r0, heads, kv, HD,
                             cap, SCALE, True)
            g16 = got[r0:r0 + 16].reshape(-1)
            worst_abs = max(worst_abs, float(np.abs(want - g16).max()))
            worst_rel = max(worst_rel, float(np.linalg.norm(want - g16) / np.linalg.norm(want)))
        parity = {"rows_checked": "16 rows from each of 0, %d and %d, every head, f64 oracle"
                                  % (tq // 2 - 1, tq - 16),
                  "max_abs": worst_abs, "rel_l2": worst_rel}
        if not (worst_abs <= 2e-3 and worst_rel <= 1e-3):
            raise SystemExit("prefill disagrees with the CPU oracle: %s" % parity)
        if world == 1 and not args.no_cpu:
            rows = min(256, tq)
            tf_cpu, used, dt, cpu_out = cpu_prefill_sample(
                np.ascontiguousarray(hq2[tq - rows:]), hk, hv, rows, tq - rows, heads, kv, cap)
            cpu = {"value": tf_cpu, "unit": "TFLOP/s", "cores": used, "kind": "port",
                   "sample": "the last %d of the %d query rows, every head (%.2f s); the C "
                             "restatement of the reference's scalar attention, threaded over "
                             "heads and row blocks" % (rows, tq, dt)}

    launches0 = gpu.launch_count()
    with ClockSampler(local) as clocks:
        secs = time_steps(gpu, step, args.steps, args.warmup)
    launches = gpu.launch_count() - launches0 - args.warmup

    # ---- end to end: q from pinned host memory, the context back -----------------
    def e2e_step():
        lib.llmtie_upload(h, q.data_ptr(), hq.data_ptr(), n * 4)
        step()
        lib.llmtie_download(h, hout.data_ptr(), out.data_ptr(), n * 4)

    e2e_step()
    barrier_sync(gpu)
    e2e_n = max(3, min(args.steps, 10))
    w0 = time.perf_counter()
    for _ in range(e2e_n):
        e2e_step()
    barrier_sync(gpu)
    e2e_secs = max_over_ranks(time.perf_counter() - w0, gpu.device) / e2e_n

    flops_total = 4.0 * HD * HEADS * (tq * (tq + 1) / 2)
    flops_rank = 4.0 * HD * heads * (tq * (tq + 1) / 2)
    _, tf, which = measured_peaks()
    tf_sus = measured_sustained_tflops()
    per_step = secs / args.steps
    achieved = flops_rank / per_step / 1e12
    traffic = NCU_TRAFFIC["prefill8k"]
    if traffic is not None:
        traffic = traffic * heads / HEADS * (tq / 8192.0)
    res = {
        "metric": "attn prefill TFLOP/s",
        "value": flops_total / per_step / 1e12,
        "unit": "TFLOP/s",
        "ms_per_step": per_step * 1e3,
        "steps": args.steps,
        "tokens_per_s": tq / per_step,
        "scaling": "strong, kv-head-shard x%d, no exchange" % world,
        "config": {"workload": "config 5 prefill: causal, seq %d, 32 Q / 8 KV heads, head_dim "
                               "128, f16 K/V ~N(0,1), sharded by KV head" % tq,
                   "seq_len": tq,
                   "l2": "flushed by the %d MB output written each step" % (n * 4 >> 20)},
        "dtype": "f16 operands, f32 accumulate",
        "clocks": clocks.summary(),
        "gpu_launches": int(launches),
        "parity_vs_oracle": parity,
        "e2e": {"value": flops_total / e2e_secs / 1e12, "unit": "TFLOP/s",
                "ms_per_step": e2e_secs * 1e3, "h2d_bytes_per_step": n * 4,
                "d2h_bytes_per_step": n * 4},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": tf, "unit": "TFLOP/s",
                     "frac": achieved / tf, "frac_of_sustained": achieved / tf_sus,
                     "traffic": traffic, "peak_source": "of " + which,
                     "kernel": "prefill_tc_kernel<128>", "kernel_ms": per_step * 1e3,
                     "algorithmic_flops_per_launch": flops_rank,
                     "frac_of_nominal_2250": achieved / 2250.0},
    }
    if cpu is not None:
        res["cpu_baseline"] = cpu
    return res


def prefill8k(args, world, rank, local):
    """The prefill leg on its own, as a bench line."""
    from ttsxabe_b200 import Gpu

    gpu = Gpu.open(local)
    res = prefill_leg(args, gpu, world, rank, local)
    line = dict(res)
    line.update({"n_gpus": world, "warmup": args.warmup, "higher_is_better": True,
                 "scaling": "strong", "vs_baseline": None, "data": "synthetic"})
    line["config"] = dict(res["config"], parallelism="kv-head-shard x%d" % world)
    return gpu, line


def graph_time(gpu, fn, reps: int = 20, rounds: int = 5) -> float:
    """Device seconds per call of fn: `reps` calls recorded into one CUDA graph
    on the handle's stream and the graph replayed, so that host launch cost
    does not hide microsecond kernels. Median of `rounds` replays."""
    import torch

    fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=gpu.stream):
        for _ in range(reps):
            fn()
    times = []
    with torch.cuda.stream(gpu.stream):
        graph.replay()
        for _ in range(rounds):
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1) / 1e3 / reps)
    return float(np.median(times))


def other_configs(args, world, rank, local):
    """The remaining benchmark configs on one GPU, device time per call
    (graph-replayed): config 1 and 2 prefill, config 3 decode at batch 1 and
    16, config 4 Whisper encoder and cross-attention. Parity for each is in
    tests/; this only times them."""
    import torch

    from ttsxabe_b200 import DecodeScratch, Gpu

    gpu = Gpu.open(local)
    hbm, tf, which = measured_peaks()
    res = {}
    rng = np.random.default_rng(0)

    def randn(n):
        with torch.cuda.stream(gpu.stream):
            return torch.randn(n, device=gpu.device).to(torch.float16).to(torch.float32)

    # config 1 / 2: ragged causal prefill with RoPE and the cache write
    for name, lens in (("config1_prefill_128", [128]),
                       ("config2_prefill_8x[256,512]", list(rng.integers(256, 513, size=8)))):
        total = int(sum(lens))
        cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        cap = 512
        q, k, v = randn(total * HEADS * HD), randn(total * KV_HEADS * HD), randn(total * KV_HEADS * HD)
        kcs = [gpu.zeros_f16(KV_HEADS * cap * HD) for _ in lens]
        vcs = [gpu.zeros_f16(KV_HEADS * cap * HD) for _ in lens]
        out = gpu.uninit(total * HEADS * HD)
        fn = lambda: gpu.prefill_varlen(q, k, v, cu, kcs, vcs, [0] * len(lens), [cap] * len(lens),
                                        None, HEADS, KV_HEADS, HD, 10000.0, SCALE, out=out)
        t = graph_time(gpu, fn)
        flops = 4.0 * HD * HEADS * sum(L * (L + 1) / 2 for L in lens)
        res[name] = {"us": t * 1e6, "tflops": flops / t / 1e12, "tokens_per_s": total / t,
                     "frac_of_tensor_peak": flops / t / 1e12 / tf}

    # config 3: one query per sequence, context in [2048, 4096]
    for batch in (1, 16):
        tks = [int(x) for x in rng.integers(2048, 4097, size=batch)]
        cap = 4096
        ks = [device_normal_f16(gpu, KV_HEADS * cap * HD, 10 + b) for b in range(batch)]
        vs = [device_normal_f16(gpu, KV_HEADS * cap * HD, 50 + b) for b in range(batch)]
        q = randn(batch * HEADS * HD)
        out = gpu.uninit(batch * HEADS * HD)
        sc = DecodeScratch()
        fn = lambda: gpu.decode_batched(q, ks, vs, tks, [cap] * batch, HEADS, KV_HEADS, HD, SCALE,
                                        False, sc, out=out)
        t = graph_time(gpu, fn)
        byts = sum(2 * KV_HEADS * tk * HD * 2 for tk in tks)
        res["config3_decode_batch%d" % batch] = {
            "us": t * 1e6, "gbs": byts / t / 1e9, "tokens_per_s": batch / t,
            "frac_of_hbm_peak": byts / t / 1e9 / hbm}

    # config 4: Whisper large-v2 shapes
    wh, whd, wt = 20, 64, 1500
    d = wh * whd
    for batch in (1, 8):
        qkv = randn(batch * wt * 3 * d)
        work = gpu._empty(batch * gpu._lib.llmtie_flash_rows_work_bytes(wt, wh, whd) // 2,
                          torch.float16)
        out = gpu._empty(batch * wt * d, torch.float16)
        flops = batch * 4.0 * whd * wh * wt * wt

        def looped():   # the reference's way: one call per utterance
            for b in range(batch):
                gpu._lib.llmtie_flash_attn_rows(
                    gpu._h, qkv.data_ptr() + b * wt * 3 * d * 4, wt * 3 * d,
                    out.data_ptr() + b * wt * d * 2, wt * d, wt, wh, whd, 0.125, work.data_ptr(),
                    work.numel() * 2)

        def batched():  # the whole batch in two launches
            gpu.flash_attn_rows_batched(qkv, batch, wt, wh, whd, 0.125, work=work, out=out)

        t = graph_time(gpu, looped, reps=5)
        res["config4_encoder_batch%d" % batch] = {"us": t * 1e6, "tflops": flops / t / 1e12,
                                                  "frac_of_tensor_peak": flops / t / 1e12 / tf}
        if batch > 1:
            t = graph_time(gpu, batched, reps=5)
            res["config4_encoder_batch%d_one_call" % batch] = {
                "us": t * 1e6, "tflops": flops / t / 1e12,
                "frac_of_tensor_peak": flops / t / 1e12 / tf}
    # The cross-attention caches as the model builds them: all 32 decoder
    # layers' projections of the encoder output split into f16 caches in two
    # launches, at a capacity of 1504 (1500 frames padded to a multiple of 8,
    # which is what lets the decoder stream them through the ring kernel).
    layers, wcap = 32, 1504
    k_all, v_all, v_bias = randn(layers * wt * d), randn(layers * wt * d), randn(layers * d)
    kcs = gpu.zeros_f16(layers * wh * wcap * whd)
    vcs = gpu.zeros_f16(layers * wh * wcap * whd)
    build = lambda: gpu._lib.llmtie_cross_kv_build(
        gpu._h, k_all.data_ptr(), k_all.numel(), v_all.data_ptr(), v_all.numel(),
        v_bias.data_ptr(), v_bias.numel(), kcs.data_ptr(), kcs.numel(), vcs.data_ptr(),
        vcs.numel(), layers, wt, wh, whd, wcap)
    t = graph_time(gpu, build, reps=5)
    moved = 2 * layers * wt * d * (4 + 2)          # f32 in, f16 out, keys and values
    res["config4_cross_kv_build_32_layers"] = {"us": t * 1e6, "gbs": moved / t / 1e9,
                                               "frac_of_hbm_peak": moved / t / 1e9 / hbm}
    one = wh * wcap * whd
    sc = DecodeScratch()
    for wcap_i, kc, vc in ((wcap, kcs[:one], vcs[:one]),
                           (wt, device_normal_f16(gpu, wh * wt * whd, 3),
                            device_normal_f16(gpu, wh * wt * whd, 4))):
        for n in (1, 8, 32):
            q = randn(n * d)
            out = gpu.uninit(n * d)
            fn = lambda: gpu._lib.llmtie_cross_attn(gpu._h, q.data_ptr(), q.numel(), kc.data_ptr(),
                                                    kc.numel(), vc.data_ptr(), vc.numel(), n, wh,
                                                    whd, wt, wcap_i, 0.125, sc._bind(gpu),
                                                    out.data_ptr(), out.numel())
            t = graph_time(gpu, fn)
            byts = 2 * wh * wt * whd * 2
            res["config4_cross_n%d_cap%d" % (n, wcap_i)] = {"us": t * 1e6, "gbs": byts / t / 1e9,
                                                            "frac_of_hbm_peak": byts / t / 1e9 / hbm}
    # ---- the callers either side of the BASELINE configs ----------------------------
    # the Whisper decoder's self-attention off f32 caches (20 heads x 64, at most 448 keys)
    for tk in (224, 448):
        q, k, v = randn(wh * whd), randn(wh * 448 * whd), randn(wh * 448 * whd)
        fn = lambda: gpu.attn_decode(q, k, v, wh, wh, whd, tk, 448, 0.125, True, sc)
        res["whisper_self_decode_f32_tk%d" % tk] = {"us": graph_time(gpu, fn) * 1e6}
    # prefill off f32 caches: the flow model's 16 heads x 64 over 2000 frames, the speech
    # LM's 14 / 2 heads x 64 (crates/llmtie-cosy), and the chat geometry at 2048 positions
    for name, (h_, kv_, hd_, causal, tq, past) in (
            ("flow_16x64_2000_frames_f32", (16, 16, 64, False, 2000, 0)),
            ("speech_lm_14_2x64_300_on_20_f32", (14, 2, 64, True, 300, 20)),
            ("prefill_32_8x128_2048_f32", (HEADS, KV_HEADS, HD, True, 2048, 0))):
        cap = past + tq
        q, k, v = randn(tq * h_ * hd_), randn(kv_ * cap * hd_), randn(kv_ * cap * hd_)
        fn = lambda: gpu.flash_attn(q, k, v, tq, past, h_, kv_, hd_, cap, float(hd_) ** -0.5,
                                    causal)
        t = graph_time(gpu, fn, reps=5)
        keys = tq * (tq + 1) / 2 + tq * past if causal else tq * cap
        res[name] = {"us": t * 1e6, "tflops": 4.0 * hd_ * h_ * keys / t / 1e12}
    # prompts shorter than a key tile; a few short sequences decoding together
    for lens in ([16], [100], [100, 50, 30, 120]):
        total = int(sum(lens))
        cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        q, k, v = randn(total * HEADS * HD), randn(total * KV_HEADS * HD), randn(total * KV_HEADS * HD)
        kcs2 = [gpu.zeros_f16(KV_HEADS * 512 * HD) for _ in lens]
        vcs2 = [gpu.zeros_f16(KV_HEADS * 512 * HD) for _ in lens]
        out = gpu.uninit(total * HEADS * HD)
        fn = lambda: gpu.prefill_varlen(q, k, v, cu, kcs2, vcs2, [0] * len(lens), [512] * len(lens),
                                        None, HEADS, KV_HEADS, HD, 10000.0, SCALE, out=out)
        res["prefill_prompts_%s" % "_".join(str(x) for x in lens)] = {"us": graph_time(gpu, fn) * 1e6}
    for batch, lo, hi in ((1, 1024, 1025), (4, 512, 1025), (8, 512, 1025)):
        tks = [int(x) for x in rng.integers(lo, hi, size=batch)]
        cap = 1024
        ks = [device_normal_f16(gpu, KV_HEADS * cap * HD, 110 + b) for b in range(batch)]
        vs = [device_normal_f16(gpu, KV_HEADS * cap * HD, 150 + b) for b in range(batch)]
        q = randn(batch * HEADS * HD)
        out = gpu.uninit(batch * HEADS * HD)
        fn = lambda: gpu.decode_batched(q, ks, vs, tks, [cap] * batch, HEADS, KV_HEADS, HD, SCALE,
                                        False, sc, out=out)
        res["decode_batch%d_ctx%d_%d" % (batch, lo, hi - 1)] = {"us": graph_time(gpu, fn) * 1e6}
    # a layer's decode step as a model makes it: RoPE + cache write, then attention
    for batch, tk in ((1, 3000), (8, 1024)):
        cap = 4096
        ks = [device_normal_f16(gpu, KV_HEADS * cap * HD, 210 + b) for b in range(batch)]
        vs = [device_normal_f16(gpu, KV_HEADS * cap * HD, 250 + b) for b in range(batch)]
        q, k, v = randn(batch * HEADS * HD), randn(batch * KV_HEADS * HD), randn(batch * KV_HEADS * HD)
        out = gpu.uninit(batch * HEADS * HD)
        pos_t, cap_t = gpu.i32_table([tk - 1] * batch), gpu.i32_table([cap] * batch)
        tk_t, ks_t, vs_t = gpu.i32_table([tk] * batch), gpu.ptr_table(ks), gpu.ptr_table(vs)

        def step():
            gpu.rope_cache_batched(q, k, v, None, HEADS, KV_HEADS, HD, 10000.0, pos_t, ks_t, vs_t,
                                   cap_t)
            gpu.decode_batched(q, ks_t, vs_t, tk_t, cap_t, HEADS, KV_HEADS, HD, SCALE, False, sc,
                               out=out)
        res["decode_step_batch%d_ctx%d" % (batch, tk)] = {"us": graph_time(gpu, step) * 1e6}
    line = {"metric": "per-config device time", "unit": "us", "n_gpus": 1, "data": "synthetic",
            "timing": "CUDA-graph replay, median of 5", "peaks": {"hbm_gbs": hbm, "tflops": tf,
                                                                  "source": which},
            "configs": res}
    return gpu, line


# ---- CPU arms ---------------------------------------------------------------------

def host_normal_f16(n: int, seed: int) -> np.ndarray:
    """n i.i.d. N(0,1) values rounded to f16 (as bits), made on the host cores."""
    import torch

    gen = torch.Generator()
    gen.manual_seed(seed)
    out = np.empty(n, dtype=np.uint16)
    step = 1 << 26
    for a in range(0, n, step):
        b = min(n, a + step)
        out[a:b] = torch.randn(b - a, generator=gen).to(torch.float16).view(torch.int16) \
            .numpy().view(np.uint16)
    return out


def cpu_decode_sample(context: int, reps: int, threads: int = 0):
    """Times the oracle's threaded decode on one sequence of the workload
    (1 of 8; every sequence is the same amount of work). Returns GB/s."""
    from oracle import oracle as O

    n = KV_HEADS * context * HD
    k = host_normal_f16(n, 1)
    v = host_normal_f16(n, 2)
    q = np.random.default_rng(0).standard_normal(HEADS * HD).astype(np.float32)
    best = None
    used = 0
    for _ in range(reps):
        t0 = time.perf_counter()
        _, used = O.decode_fast(q, k, v, HEADS, KV_HEADS, HD, context, context, SCALE, False,
                                threads)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    bytes_one = 2 * KV_HEADS * context * HD * 2
    return bytes_one / best / 1e9, used, best


def reference_arm(args):
    """The reference's own CPU attention (its scalar decode restated in C,
    threaded over heads and key slabs) on the host cores, on the same
    workload as the GPU arm: every one of the batch's sequences each step,
    f16 K/V drawn N(0,1). A step is a few tenths of a second."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O

    ctx, batch = args.context, args.batch
    n = KV_HEADS * ctx * HD
    ks = [host_normal_f16(n, 1000 + 17 * b) for b in range(batch)]
    vs = [host_normal_f16(n, 5000 + 17 * b) for b in range(batch)]
    q = np.random.default_rng(7).standard_normal((batch, HEADS * HD)).astype(np.float32)
    q = q.astype(np.float16).astype(np.float32)
    used = 0
    times = []
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        for b in range(batch):
            _, used = O.decode_fast(q[b], ks[b], vs[b], HEADS, KV_HEADS, HD, ctx, ctx, SCALE,
                                    False, 0)
        if i >= args.warmup:
            times.append(time.perf_counter() - t0)
    per = float(np.mean(times))
    bytes_step = batch * 2 * KV_HEADS * ctx * HD * 2
    gbs = bytes_step / per / 1e9
    sample = ("the whole step: all %d sequences (%d keys x 8 KV heads each, %.0f MB of KV a "
              "step), %d host threads" % (batch, ctx, bytes_step / 1e6, used))
    print(json.dumps({
        "impl": "reference",
        "metric": "decode KV GB/s", "value": gbs, "unit": "GB/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": per * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16 KV cache, f32 accumulate", "data": "synthetic",
        "config": {"workload": WORKLOAD % (batch, ctx),
                   "global_batch": batch, "context": ctx,
                   "parallelism": "host threads x%d" % used},
        "tokens_per_s": batch / per,
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": used, "kind": "port",
                         "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    # A short default run on purpose: the roofline's denominator is a burst
    # figure, and a B200 streaming HBM flat out reports sw_power_cap and drops
    # its SM clock after some 40 ms (the kernel then runs ~10 % slower).
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode128k",
                    choices=["decode128k", "prefill8k", "configs"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=131072)
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline legs")
    ap.add_argument("--no-prefill", action="store_true",
                    help="leave the prefill object out of the decode line")
    ap.add_argument("--exchange", default="push", choices=["push", "pairs", "fused", "nccl"],
                    help="how the ranks exchange their triples: everything in the decode "
                         "kernel over peer memory (fused), the push in the kernel and the merge "
                         "in a second waiting kernel (push), or an NCCL all-gather (nccl)")
    ap.add_argument("--nccl", action="store_true", help="the same as --exchange nccl")
    ap.add_argument("--no-graph", action="store_true",
                    help="time the sharded step as separate host calls, not a CUDA graph")
    args = ap.parse_args()
    if args.nccl:
        args.exchange = "nccl"
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        reference_arm(args)
        return

    # Libraries (NCCL's version banner, for one) write to stdout; the contract
    # is ONE JSON line there, so everything else is sent to stderr.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    world, rank, local = dist_setup(args.gpus)
    fn = {"decode128k": decode128k, "prefill8k": prefill8k, "configs": other_configs}[
        args.workload]
    gpu, line = fn(args, world, rank, local)
    if args.workload == "decode128k" and not args.no_prefill:
        import torch

        torch.cuda.empty_cache()
        line["prefill"] = prefill_leg(args, gpu, world, rank, local)
    sys.stdout.flush()
    os.dup2(real_stdout, 1)
    os.close(real_stdout)
    if rank == 0:
        if world == 1 and not args.no_cpu and args.workload == "decode128k":
            gbs, used, secs = cpu_decode_sample(args.context, reps=40)
            line["cpu_baseline"] = {
                "value": gbs, "unit": "GB/s", "cores": used, "kind": "port",
                "sample": "1 of the %d sequences (f16 K/V ~N(0,1)), best of 40 passes (%.2f s "
                          "each), %d host threads; the C restatement of the reference's scalar "
                          "decode, threaded over heads and key slabs"
                          % (args.batch, secs, used)}
        print(json.dumps(line))
    import torch.distributed as dist

    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
