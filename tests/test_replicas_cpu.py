"""The N > 1 path on CPU: two `gloo` ranks run the replica measurement protocol (barrier, maximum of the
per-rank times, sum of the units) that bench.py uses under torch.distributed.run."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    from turbopi_b200.replicas import ReplicaGroup
    g = ReplicaGroup.from_env(backend="gloo")
    g.barrier()
    # rank r "processed" 100 * (r + 1) units in 10 * (r + 1) ms
    rate, ms = g.throughput(100.0 * (rank + 1), 10.0 * (rank + 1))
    mx = g.max_over_ranks(float(rank))
    g.barrier()
    q.put((rank, g.world, rate, ms, mx))
    g.close()


@pytest.mark.timeout(120)
def test_two_gloo_ranks_aggregate_like_the_bench():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=100) for _ in range(world))
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    for rank, w, rate, ms, mx in got:
        assert w == 2
        assert ms == 20.0                      # slowest rank
        assert rate == pytest.approx(300.0 / 0.020)   # all units over the slowest rank's time
        assert mx == 1.0


def test_single_process_needs_no_group():
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        os.environ.pop(k, None)
    from turbopi_b200.replicas import ReplicaGroup
    g = ReplicaGroup.from_env(backend="gloo")
    assert (g.rank, g.world) == (0, 1)
    rate, ms = g.throughput(50.0, 5.0)
    assert rate == pytest.approx(10000.0) and ms == 5.0
    g.barrier()
    g.close()
