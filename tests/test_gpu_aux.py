"""What stands around the kernels: the bounded device waits and how a wait
that runs out reaches the host, the per-kernel profile and the kernel
resource query (crates/llmtie-cuda/src/device.rs:1458-1465, :1490-1565).

Nothing here faults or hangs a device: the one wait that runs out is a wait
for a flag that nothing raises, given a limit of about a millisecond, after
which the kernel returns normally.
"""
import numpy as np
import pytest

from oracle import oracle as O
from tests.helpers import assert_close_to, lay_caches

pytestmark = pytest.mark.gpu


def _exchange_of_one_device(gpu, world, rows, hd, step_value):
    """An exchange descriptor whose every "rank" is a plain buffer of this one
    device (no peer or symmetric memory): gather [2][world][rows][hd+2], flags
    [world] and the step counter, all zero but the step."""
    import torch

    from ttsxabe_b200.gpu import Exchange

    with torch.cuda.stream(gpu.stream):
        gather = torch.zeros(2 * world * rows * (hd + 2), dtype=torch.float32, device=gpu.device)
        flags = torch.zeros(64, dtype=torch.int32, device=gpu.device)
        step = torch.full((1,), step_value, dtype=torch.int32, device=gpu.device)
    xch = Exchange(world, 0, [gather.data_ptr()] * world, [flags.data_ptr()] * world,
                   step.data_ptr())
    return xch, gather, flags, step


def test_a_wait_that_runs_out_is_reported_and_the_handle_stays_usable(gpu):
    """The merge of a sharded step waits for every rank's flag. Here rank 1's
    flag is never raised and the limit is about a millisecond: the kernel
    returns, the next synchronize raises DeviceTimeout - once -, a download
    reports it just the same, and a decode on the same handle afterwards is
    correct."""
    import torch

    from ttsxabe_b200 import DecodeScratch, DeviceTimeout

    world, rows, hd = 2, 32, 128
    xch, gather, flags, step = _exchange_of_one_device(gpu, world, rows, hd, step_value=1)
    with torch.cuda.stream(gpu.stream):
        flags[0] = 1            # rank 0 has delivered, rank 1 never does
    gpu.synchronize()
    gpu.set_wait_limit_cycles(2_000_000)
    try:
        gpu.lse_merge_wait(xch, rows, hd)
        with pytest.raises(DeviceTimeout, match="site 61"):
            gpu.synchronize()
        gpu.synchronize()       # reported once
        out = gpu.lse_merge_wait(xch, rows, hd)
        with pytest.raises(DeviceTimeout):
            gpu.download(out)   # what it copied is what the kernel never wrote
        gpu.synchronize()
    finally:
        gpu.set_wait_limit_cycles(0)

    # both flags up: the same call merges (two equal triples merge to their value)
    rng = np.random.default_rng(5)
    tri = rng.standard_normal((rows, hd + 2)).astype(np.float32)
    tri[:, hd] = 0.25                      # m
    tri[:, hd + 1] = np.abs(tri[:, hd + 1]) + 1.0   # l
    both = np.concatenate([tri.reshape(-1), tri.reshape(-1)])
    with torch.cuda.stream(gpu.stream):
        gather[:both.size] = torch.from_numpy(both).to(gpu.device)
        flags[:2] = 1
    got = gpu.download(gpu.lse_merge_wait(xch, rows, hd)).reshape(rows, hd)
    want = tri[:, :hd] / tri[:, hd + 1:hd + 2]
    assert np.abs(got - want).max() <= 1e-6 * np.abs(want).max()

    # and the handle decodes as before
    heads, kv, tk, cap = 8, 2, 3000, 3072
    q = O.seq(heads * hd, 900)
    k0, v0 = O.seq(kv * cap * hd, 901), O.seq(kv * hd * cap, 902)
    scratch = DecodeScratch()
    dec = gpu.download(gpu.attn_decode_f16(gpu.upload(q), gpu.upload_f16(k0), gpu.upload_f16(v0),
                                           heads, kv, hd, tk, cap, 0.11, False, scratch))
    want = O.decode_f64(q, O.round_f16(k0), O.round_f16(v0), heads, kv, hd, 0, tk, cap, 0.11, False)
    assert_close_to("decode after a reported timeout", want, dec, 2e-5)


def test_kprof_charges_each_launch_to_its_kernel(gpu):
    """With the profile on, a known sequence of calls shows up under the
    kernels' names with their counts, the most expensive first; the
    tensor-memory prefill and the general one are told apart."""
    heads, kv, hd, tq = 8, 2, 128, 256
    scale = float(np.float32(hd) ** np.float32(-0.5))
    q = O.seq(tq * heads * hd, 1)
    dq = gpu.upload(q)
    # capacity 256: aligned rows, the tensor-memory kernel as the caches lie; 138: after a
    # copy of the live keys into aligned caches
    kc, vc = lay_caches(O.seq(kv * tq * hd, 2), O.seq(kv * tq * hd, 3), kv, tq, hd, 256)
    dk, dv = gpu.upload_f16(kc), gpu.upload_f16(vc)
    n2 = 130
    kc2, vc2 = lay_caches(O.seq(kv * n2 * hd, 4), O.seq(kv * n2 * hd, 5), kv, n2, hd, 138)
    dk2, dv2 = gpu.upload_f16(kc2), gpu.upload_f16(vc2)
    d32k, d32v = gpu.upload(kc), gpu.upload(vc)
    gpu.synchronize()
    gpu.kprof_reset()
    gpu.kprof_enable(True)
    try:
        gpu.rope(dq, 0, tq, heads, hd, 10000.0, 0)
        gpu.rope(dq, 0, tq, heads, hd, 10000.0, 0)
        gpu.flash_attn_f16(dq, dk, dv, tq, 0, heads, kv, hd, 256, scale, True)
        gpu.flash_attn_f16(dq, dk2, dv2, n2, 0, heads, kv, hd, 138, scale, True)
        # f32 caches: rounded to f16 once, then the tensor-memory kernel
        gpu.flash_attn(dq, d32k, d32v, tq, 0, heads, kv, hd, 256, scale, True)
        rep = gpu.kprof_report()
    finally:
        gpu.kprof_enable(False)
    assert rep["rope"][0] == 2
    assert rep["flash_attn_h_tc"][0] == 1
    assert rep["caches_to_f16"][0] == 2 and rep["flash_attn_tc"][0] == 2
    assert "flash_attn_h" not in rep and "flash_attn" not in rep
    assert all(ms > 0.0 for _, ms in rep.values())
    assert list(rep.values()) == sorted(rep.values(), key=lambda e: -e[1])
    gpu.kprof_reset()
    assert gpu.kprof_report() == {}
    # off again: nothing is charged
    gpu.rope(dq, 0, tq, heads, hd, 10000.0, 0)
    assert gpu.kprof_report() == {}


def test_the_general_prefill_kernel_behind_its_switch():
    """With LLMTIE_B200_NO_TC the tensor-memory kernel is never taken (the
    switch is read once a process, hence the child): the general kernel
    serves f16 and f32 caches, aligned or not, at the same bar, and kprof
    names it."""
    import os
    import subprocess
    import sys

    code = r"""
import numpy as np
from oracle import oracle as O
from tests.helpers import lay_caches, prefill_spread, assert_prefill_tolerance
from ttsxabe_b200 import Gpu
gpu = Gpu.open(0)
gpu.kprof_enable(True)
for heads, kv, hd, causal, tq, past, cap, half in [(8, 2, 128, True, 150, 0, 256, True),
                                                   (4, 2, 128, True, 130, 5, 138, True),
                                                   (4, 2, 64, True, 70, 33, 160, False),
                                                   (16, 16, 64, False, 257, 0, 258, False)]:
    tk = past + tq
    scale = float(np.float32(hd) ** np.float32(-0.5))
    q = O.seq(tq * heads * hd, 71) * np.float32(100.0)
    kc, vc = lay_caches(O.seq(kv * tk * hd, 72), O.seq(kv * tk * hd, 73), kv, tk, hd, cap)
    dq = gpu.upload(q)
    if half:
        out = gpu.flash_attn_f16(dq, gpu.upload_f16(kc), gpu.upload_f16(vc), tq, past, heads, kv, hd, cap, scale, causal)
    else:
        out = gpu.flash_attn(dq, gpu.upload(kc), gpu.upload(vc), tq, past, heads, kv, hd, cap, scale, causal)
    want, spread = prefill_spread(q, kc, vc, tq, past, heads, kv, hd, cap, scale, causal)
    assert_prefill_tolerance(str((heads, kv, hd, tq, cap)), want, spread, gpu.download(out))
rep = gpu.kprof_report()
assert not any(name.endswith("_tc") or name == "caches_to_f16" for name in rep), rep
assert rep["flash_attn_h"][0] == 2 and sum(rep[n][0] for n in rep if n in ("flash_attn", "flash_attn_64")) == 2, rep
print("general kernel ok")
"""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, LLMTIE_B200_NO_TC="1", PYTHONPATH=root)
    done = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True,
                          text=True, timeout=600)
    assert done.returncode == 0 and "general kernel ok" in done.stdout, done.stdout + done.stderr


def test_the_register_fed_decode_kernel_behind_its_switch():
    """With LLMTIE_B200_DECODE_NO_STREAM the ring kernel is never taken (read
    once a process, hence the child): the register-fed kernel - otherwise only
    reached by caches at addresses the ring cannot copy from - serves aligned
    capacities and those that are multiples of 4 only, at the same bar, twice
    through one scratch."""
    import os
    import subprocess
    import sys

    code = r"""
import numpy as np
from oracle import oracle as O
from tests.helpers import assert_close_to
from ttsxabe_b200 import Gpu, DecodeScratch
gpu = Gpu.open(0)
gpu.kprof_enable(True)
for i, (heads, kv, hd, tk, cap, scale_q) in enumerate([(8, 2, 128, 256, 256, False), (6, 6, 64, 1499, 1500, True),
                                                      (32, 8, 128, 7777, 8192, False), (14, 2, 64, 700, 1024, False),
                                                      (20, 20, 64, 1500, 1500, True)]):
    q = O.seq(heads * hd, 300 + i)
    k0, v0 = O.seq(kv * cap * hd, 400 + i), O.seq(kv * hd * cap, 500 + i)
    scratch = DecodeScratch()
    dq, dk, dv = gpu.upload(q), gpu.upload_f16(k0), gpu.upload_f16(v0)
    a = gpu.download(gpu.attn_decode_f16(dq, dk, dv, heads, kv, hd, tk, cap, 0.11, scale_q, scratch))
    b = gpu.download(gpu.attn_decode_f16(dq, dk, dv, heads, kv, hd, tk, cap, 0.11, scale_q, scratch))
    assert np.array_equal(a, b)
    want = O.decode_f64(q, O.round_f16(k0), O.round_f16(v0), heads, kv, hd, 0, tk, cap, 0.11, scale_q)
    assert_close_to(str((heads, kv, hd, tk, cap)), want, a, 2e-5)
rep = gpu.kprof_report()
assert not any(name.endswith("_run") for name in rep), rep
assert sum(c for name, (c, _) in rep.items() if name.startswith("attn_decode_h")) == 10, rep
print("register-fed kernel ok")
"""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, LLMTIE_B200_DECODE_NO_STREAM="1", PYTHONPATH=root)
    done = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True,
                          text=True, timeout=600)
    assert done.returncode == 0 and "register-fed kernel ok" in done.stdout, done.stdout + done.stderr


def test_kernel_resources_are_what_the_compiler_gave(gpu):
    """(registers a thread, local bytes a thread, static shared bytes a block)
    per kernel name; None for a name that is not in the library."""
    seen = {}
    for name in ("flash_attn_h_tc", "flash_attn_64_tc", "attn_decode_h128_run",
                 "attn_decode_h64_run", "attn_decode_h128", "attn_decode_f64", "lse_merge",
                 "lse_merge_wait"):
        res = gpu.kernel_resources(name)
        assert res is not None, name
        regs, local, smem = res
        assert 0 < regs <= 255 and local >= 0 and smem >= 0, (name, res)
        seen[name] = res
    # the key loop of the ring kernel must not spill
    assert seen["attn_decode_h128_run"][1] == 0
    assert gpu.kernel_resources("no_such_kernel") is None


def test_calls_with_nothing_to_do_launch_nothing(gpu):
    """Zero rows, zero new tokens, zero sequences, zero layers: every entry
    answers OK, launches nothing and writes nothing (the reference's methods
    return early on empty work, e.g. crates/llmtie-cuda/src/device.rs:5702-5745
    on `tq == 0`)."""
    from ttsxabe_b200 import DecodeScratch

    heads, kv, hd, cap = 8, 2, 128, 64
    buf = O.seq(4 * heads * hd, 9)
    x = gpu.upload(buf)
    kc, vc = gpu.zeros_f16(kv * cap * hd), gpu.zeros_f16(kv * cap * hd)
    k32, v32 = gpu.zeros(kv * cap * hd), gpu.zeros(kv * cap * hd)
    ck, cv = gpu.zeros_f16(heads * cap * hd), gpu.zeros_f16(heads * cap * hd)   # a cache a query head
    scratch = DecodeScratch()
    gpu.synchronize()
    before = gpu.launch_count()
    gpu.rope(x, 0, 0, heads, hd, 10000.0, 0)
    gpu.cache_append_f16(x, 0, kc, 0, kv, hd, cap, 3, False)
    gpu.cache_append(x, 0, k32, 0, kv, hd, cap, 3, True)
    gpu.flash_attn_f16(x, kc, vc, 0, 5, heads, kv, hd, cap, 0.1, True)
    gpu.flash_attn(x, k32, v32, 0, 5, heads, kv, hd, cap, 0.1, True)
    gpu.flash_attn_rows(gpu.upload(O.seq(3 * 20 * 64, 1)), 0, 20, 64, 0.125)
    gpu.cross_attn(x, ck, cv, 0, heads, hd, 10, cap, 0.1, scratch)
    gpu.split_heads(x, 0, heads, hd)
    gpu.prefill_varlen(x, x, x, [0, 0], [kc], [vc], [0], [cap], None, heads, kv, hd, 10000.0, 0.1)
    gpu.prefill_varlen(x, x, x, [0], [], [], [], [], None, heads, kv, hd, 10000.0, 0.1)
    gpu.lse_merge(x, 0, 4, hd)
    gpu.synchronize()
    assert gpu.launch_count() == before
    assert np.array_equal(gpu.download(x), buf)
    assert not gpu.download_u16(kc).any() and not gpu.download(k32).any()


def test_resident_clusters_as_the_driver_answers(gpu):
    """What the launch asks before it gives pairs a cluster each: more blocks
    a cluster, fewer clusters; the narrower kernel's ring is half the size, so
    twice as many fit. (The host-side plan in tests/test_decode_cut.py is
    checked against a B200's answers: 74 / 33 / 15 and 148 / 71 / 33.)"""
    for hd in (128, 64):
        n = [gpu._lib.llmtie_decode_resident_clusters(gpu._h, hd, c) for c in (2, 4, 8)]
        assert n[0] >= n[1] >= n[2] >= 1, (hd, n)
        assert n[0] * 2 <= 2 * 148 and n[2] * 8 <= 2 * 148
    assert gpu._lib.llmtie_decode_resident_clusters(gpu._h, 96, 2) == 0
