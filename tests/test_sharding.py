"""Sharding over ranks: host logic on CPU, world_size 2 over gloo.  Each rank runs the oracle on
its shard; gathered outputs and reduced per-head gradients must equal the unsharded result."""
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
