"""Multi-rank host logic on CPU (gloo, world_size 2): batch shards cover the batch exactly,
the sharded computation reproduces the un-sharded one with no exchange on the data path, and
the whole-job timing rule is max over ranks."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dcnv4_b200 import sharding


def test_shard_bounds_cover_exactly():
    for n in (0, 1, 5, 64, 257):
        for world in (1, 2, 3, 8):
            spans = [sharding.shard_bounds(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (a, b), (c, d) in zip(spans, spans[1:]):
                assert b == c and a <= b and c <= d
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_bounds(4, 2, 2)


def test_job_throughput_uses_slowest_rank():
    assert sharding.job_throughput([10, 10], [1.0, 2.0]) == 10.0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, N, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import cref, inputs as oin
        torch.set_num_threads(1)
        t = oin.dcnv4_inputs(N, 8, 8, 2, 16, seed=7)               # same seed on every rank
        args = (3, 3, 1, 1, 1, 1, 1, 1, 2, 16, 1.0, 0)
        full = cref.dcnv4_forward(t["value"], t["offset_mask"], *args)
        gv_full, gom_full = cref.dcnv4_backward(t["value"], t["offset_mask"], t["grad_out"], *args)
        lo, hi = sharding.shard_bounds(N, rank, world)
        mine = {k: sharding.shard(v, rank, world) for k, v in t.items()}
        part = cref.dcnv4_forward(mine["value"], mine["offset_mask"], *args)
        gv, gom = cref.dcnv4_backward(mine["value"], mine["offset_mask"], mine["grad_out"], *args)
        # the shard's results are the corresponding rows of the full results: no exchange needed
        ok = (torch.equal(part, full[lo:hi]) and torch.equal(gv, gv_full[lo:hi])
              and torch.equal(gom, gom_full[lo:hi]))
        # whole-job timing: max over ranks, as the benchmark does
        elapsed = torch.tensor([1.0 + rank], dtype=torch.float64)
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        flags = torch.tensor([int(ok)])
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        if rank == 0:
            out_q.put((int(flags.item()), float(elapsed.item()), hi - lo))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_two_ranks_shard_without_exchange():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, 5, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(150)
        assert p.exitcode == 0
    ok, slowest, n0 = q.get(timeout=10)
    assert ok == 1 and slowest == 2.0 and n0 == 3
