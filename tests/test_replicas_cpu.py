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


def _serve_main(rank, world, port, q, leave_after):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    from turbopi_b200.replicas import ReplicaGroup, RequestDispatcher
    g = ReplicaGroup.from_env(backend="gloo")
    served = []

    def infer(req):                      # a stand-in replica: the "actions" are a function of the request
        served.append(req)
        return torch.full((2,), float(req) * 10.0)

    d = RequestDispatcher(g, infer, timeout_s=3.0)
    results, stats = d.serve(list(range(8)), leave_after=leave_after if rank == 1 else None)
    q.put((rank, None if results is None else [float(r[0]) for r in results], stats["done"], stats["requeued"], served))
    if leave_after is None:
        g.barrier()
    g.close() if leave_after is None else None


@pytest.mark.timeout(120)
@pytest.mark.parametrize("leave_after", [None, 1])
def test_dispatcher_splits_a_batch_and_requeues_what_a_lost_replica_left(leave_after):
    """8 requests on 2 replicas: contiguous chunks of 4, results in request order on rank 0.  With rank 1 leaving
    after its first request, rank 0 runs the three requests that never arrived."""
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_serve_main, args=(r, world, port, q, leave_after)) for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(world):
        rank, results, done, requeued, served = q.get(timeout=100)
        got[rank] = (results, done, requeued, served)
    for p in procs:
        p.join(timeout=30)
    results, done0, requeued, served0 = got[0]
    assert results == [float(i) * 10.0 for i in range(8)]
    assert got[1][0] is None
    if leave_after is None:
        assert requeued == [] and served0 == [0, 1, 2, 3] and got[1][3] == [4, 5, 6, 7]
    else:
        assert requeued == [5, 6, 7] and got[1][3] == [4] and served0 == [0, 1, 2, 3, 5, 6, 7]


def test_split_requests_is_contiguous_and_even():
    from turbopi_b200.replicas import split_requests
    assert split_requests(64, 8) == [(8 * r, 8 * r + 8) for r in range(8)]
    assert split_requests(8, 1) == [(0, 8)]
    assert split_requests(10, 4) == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert split_requests(2, 4) == [(0, 1), (1, 2), (2, 2), (2, 2)]


def test_dispatcher_keeps_several_requests_in_flight_per_replica():
    """`infer` given as a list of callables (pipelines of one replica): the chunk is served by one host thread per
    pipeline, every request exactly once, results in request order."""
    import threading
    import time
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        os.environ.pop(k, None)
    from turbopi_b200.replicas import ReplicaGroup, RequestDispatcher
    g = ReplicaGroup.from_env(backend="gloo")
    served = [[], [], []]
    running, peak = [0], [0]
    lock = threading.Lock()

    def lane(k):
        def infer(req):
            with lock:
                running[0] += 1
                peak[0] = max(peak[0], running[0])
            time.sleep(0.02)
            served[k].append(req)
            with lock:
                running[0] -= 1
            return torch.full((2,), float(req))
        return infer

    d = RequestDispatcher(g, [lane(0), lane(1), lane(2)], timeout_s=5.0)
    results, stats = d.serve(list(range(12)))
    assert [float(r[0]) for r in results] == [float(i) for i in range(12)]
    assert sorted(served[0] + served[1] + served[2]) == list(range(12))
    assert peak[0] >= 2 and all(len(s) >= 1 for s in served)          # the lanes did overlap
    assert stats["done"] == 12 and stats["requeued"] == [] and len(stats["latencies_ms"]) == 12
    g.close()


def test_a_failing_pipeline_fails_the_batch_loudly():
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        os.environ.pop(k, None)
    from turbopi_b200.replicas import ReplicaGroup, RequestDispatcher
    g = ReplicaGroup.from_env(backend="gloo")

    def good(req):
        import time
        time.sleep(0.05)                 # long enough for the other lane to draw a request
        return torch.zeros(1)

    def bad(req):
        raise RuntimeError("pipeline broke")

    for lanes in ([bad], [good, bad]):
        with pytest.raises(RuntimeError, match="pipeline broke"):
            RequestDispatcher(g, lanes, timeout_s=1.0).serve(list(range(6)))
    g.close()
