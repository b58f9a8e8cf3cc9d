"""Sharding over ranks (mamba_trainer_b200/sharding.py): the batch-then-heads plan, the per-shard count of
reversed heads, and - as two gloo ranks on CPU - the path bench.py takes at N > 1: each rank runs its shard
(here through the oracle, the GPU box runs the kernels), per-token outputs are gathered, per-head gradients
reduced, and both must equal the unsharded result."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mamba_trainer_b200 import sharding, synthetic
from mamba_trainer_b200.ssm import Discretization
from tests._util import oracle_run


def test_plan_covers_everything_once():
    for batch, heads, world in [(8, 12, 1), (8, 12, 2), (8, 12, 8), (2, 8, 8), (1, 4, 4), (5, 3, 2)]:
        seen = torch.zeros(batch, heads, dtype=torch.int32)
        for r in range(world):
            s = sharding.shard_plan(batch, heads, world, r)
            seen[s.batch, s.heads] += 1
        assert (seen == 1).all(), (batch, heads, world)
    with pytest.raises(ValueError):
        sharding.shard_plan(2, 3, 4, 0)      # 3 heads do not split over 2 ranks per sequence
    with pytest.raises(ValueError):
        sharding.shard_plan(2, 4, 2, 2)


def test_reversed_heads_follow_their_shard():
    """A bidirectional scan reverses the last `reverse_heads` heads (models/mamba3.rs:352-370).  When the
    heads of a sequence are split over ranks, each shard reverses exactly those of its heads that lie in
    that tail: summed over the shards of a sequence that is the whole tail, and the oracle on the shard
    with its own count reproduces the unsharded result."""
    for batch, heads, world, rev in [(2, 8, 8, 4), (1, 4, 4, 1), (8, 12, 2, 6), (2, 8, 8, 8), (2, 8, 8, 0)]:
        per_row = {}
        for r in range(world):
            s = sharding.shard_plan(batch, heads, world, r)
            n = sharding.shard_reverse_heads(heads, rev, s)
            assert 0 <= n <= s.n_heads
            # the shard's reversed heads are its last n, and they are global heads >= heads - rev
            assert all(h >= heads - rev for h in range(s.heads.stop - n, s.heads.stop))
            assert all(h < heads - rev for h in range(s.heads.start, s.heads.stop - n))
            for b in range(s.batch.start, s.batch.stop):
                per_row[b] = per_row.get(b, 0) + n
        assert all(v == rev for v in per_row.values()), (batch, heads, world, rev)
    # numerically: 2 sequences x 4 heads over 4 ranks (two heads per rank), the last 3 heads reversed
    from oracle.m3_oracle import mamba3_scan_bidirectional
    w = synthetic.Workload("bidir_shard", 2, 24, 4, 4, 8, 8, 2, torch.float32, Discretization.LearnedTrapezoid, True, "scaled")
    t = synthetic.make_inputs(w, seed=5)
    full, _ = mamba3_scan_bidirectional(t["x"], t["b"], t["c"], t["dt"], t["a_log"], t["lam"], t["theta"], t["d_skip"],
                                         None, w.chunk, False, reverse_heads=3)
    for r in range(4):
        s = sharding.shard_plan(2, 4, 4, r)
        ts = sharding.shard_inputs(t, s)
        part, _ = mamba3_scan_bidirectional(ts["x"], ts["b"], ts["c"], ts["dt"], ts["a_log"], ts["lam"], ts["theta"],
                                             ts["d_skip"], None, w.chunk, False,
                                             reverse_heads=sharding.shard_reverse_heads(4, 3, s))
        assert torch.equal(part, full[s.batch, :, s.heads]), r


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, batch, heads, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        w = synthetic.Workload("shard_case", batch, 24, heads, 4, 6, 8, 2, torch.float32,
                               Discretization.LearnedTrapezoid, True, "scaled")
        t = synthetic.make_inputs(w, seed=11)                    # identical on every rank
        shard = sharding.shard_plan(batch, heads, world, rank)
        local = sharding.shard_inputs(t, shard)
        y, _, g = oracle_run(local, w.chunk, False)
        full_y = sharding.gather_per_token(y, batch, heads)
        full_dx = sharding.gather_per_token(g["x"], batch, heads)
        da = sharding.reduce_per_head(g["a_log"], heads, shard)
        dd = sharding.reduce_per_head(g["d_skip"], heads, shard)
        if rank == 0:
            ey, _, eg = oracle_run(t, w.chunk, False)
            q.put((float((full_y - ey).abs().max()), float((full_dx - eg["x"]).abs().max()),
                   float((da - eg["a_log"]).abs().max()), float((dd - eg["d_skip"]).abs().max())))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("batch,heads", [(4, 2), (1, 4)])
def test_two_ranks_reproduce_the_unsharded_scan(batch, heads):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, batch, heads, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    errs = q.get(timeout=5)
    assert max(errs) < 1e-10, errs
