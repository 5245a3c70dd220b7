"""The multi-GPU decode path's host logic on CPU: two gloo ranks each take a
slice of the keys, compute their (o, m, l) triples with the oracle standing in
for the device, exchange them through ShardedDecode's all-gather, and merge;
the result equals single-rank attention over the whole cache."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_bounds_cover_the_sequence():
    from ttsxabe_b200.sharded import kv_head_shard, shard_bounds

    for tk in (1, 7, 8, 1000, 4096, 131072, 131073):
        for world in (1, 2, 4, 8):
            cuts = [shard_bounds(tk, world, r) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == tk
            for (a0, a1), (b0, b1) in zip(cuts[:-1], cuts[1:]):
                assert a1 == b0 and a0 <= a1
                assert a0 % 8 == 0 or a0 == a1 == tk   # empty tail slices sit at the end
    assert [kv_head_shard(8, 8, r) for r in range(8)] == [(r, r + 1) for r in range(8)]
    assert [kv_head_shard(8, 2, r) for r in range(2)] == [(0, 4), (4, 8)]
    assert [kv_head_shard(8, 3, r) for r in range(3)] == [(0, 3), (3, 6), (6, 8)]
    with pytest.raises(ValueError):
        kv_head_shard(8, 16, 0)


def _worker(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as O
    from ttsxabe_b200.sharded import ShardedDecode, shard_bounds

    heads, kv, hd, batch, tk = 8, 2, 64, 3, 1003
    cap = 1024
    scale = 0.125
    rng = np.random.default_rng(5)      # the same inputs on both ranks
    q = O.through_f16(rng.standard_normal(batch * heads * hd).astype(np.float32))
    ks = [O.round_f16(rng.standard_normal(kv * cap * hd).astype(np.float32)) for _ in range(batch)]
    vs = [O.round_f16(rng.standard_normal(kv * cap * hd).astype(np.float32)) for _ in range(batch)]
    t0, t1 = shard_bounds(tk, world, rank)

    def partial_fn(qt, partial):
        assert partial
        qn = qt.numpy().reshape(batch, heads * hd)
        out = np.empty((batch, heads, hd + 2), np.float32)
        for b in range(batch):
            _, o, m, l = O.decode_f64(qn[b], ks[b], vs[b], heads, kv, hd, t0, t1, cap, scale,
                                      False, triple=True)
            out[b, :, :hd] = o.reshape(heads, hd)
            out[b, :, hd] = m
            out[b, :, hd + 1] = l
        return torch.from_numpy(out.reshape(-1))

    def merge_fn(gathered, parts, rows):
        g = gathered.numpy().reshape(parts, rows, hd + 2)
        return torch.from_numpy(O.lse_merge(np.ascontiguousarray(g[:, :, :hd]),
                                            np.ascontiguousarray(g[:, :, hd]),
                                            np.ascontiguousarray(g[:, :, hd + 1]), parts, rows, hd))

    sd = ShardedDecode(heads, hd, None, partial_fn, merge_fn)
    assert sd.world == world and sd.rank == rank
    got = sd.decode(torch.from_numpy(q)).numpy().reshape(batch, -1)
    for b in range(batch):
        want = O.decode_f64(q.reshape(batch, -1)[b], ks[b], vs[b], heads, kv, hd, 0, tk, cap,
                            scale, False)
        err = float(np.abs(want - got[b]).max())
        assert err < 2e-6, (rank, b, err)
    np.save(os.path.join(tmp, f"out{rank}.npy"), got)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharded_decode_equals_one_rank(tmp_path):
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    a = np.load(tmp_path / "out0.npy")
    b = np.load(tmp_path / "out1.npy")
    assert np.array_equal(a, b), "both ranks must hold the same merged context"


def _leaver(rank, world, port, tmp):
    """Rank 1 takes part in the first step and then leaves between steps (its
    process ends with nothing of its own in flight); rank 0 goes into the next
    step's exchange alone and must get an error, not a hang."""
    import datetime

    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=4))
    from ttsxabe_b200.sharded import ShardedDecode

    heads, hd, batch = 2, 4, 1
    part = torch.arange(batch * heads * (hd + 2), dtype=torch.float32)
    sd = ShardedDecode(heads, hd, None, lambda q, partial: part.clone(),
                       lambda g, parts, rows: g.reshape(parts, rows, hd + 2)[0, :, :hd].reshape(-1))
    sd.decode(torch.zeros(batch * heads * hd))        # a step with both ranks: fine
    if rank == 1:
        return                                        # leaves between steps
    try:
        sd.decode(torch.zeros(batch * heads * hd))
        verdict = "returned"
    except Exception as e:                            # the collective's own timeout or a reset
        verdict = "raised " + type(e).__name__
    with open(os.path.join(tmp, "verdict.txt"), "w") as f:
        f.write(verdict)


def test_a_rank_that_leaves_between_steps_ends_the_next_exchange_with_an_error(tmp_path):
    """Failure on the host, no device involved: the surviving rank's next
    all-gather ends with an error within the process group's timeout (four
    seconds here) instead of waiting for ever."""
    world = 2
    port = 31500 + (os.getpid() % 2000)
    mp.spawn(_leaver, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    verdict = (tmp_path / "verdict.txt").read_text()
    assert verdict.startswith("raised"), verdict
