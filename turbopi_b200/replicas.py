"""Process plumbing for N > 1 GPUs: the measurement protocol and the request dispatcher.

The inference path does not shard: the reference serves one policy per process and its quantised
kernels have no exchange step, so N GPUs run N independent replicas (one process per GPU, launched
by torch.distributed.run).  The only communication is the measurement protocol: a barrier on both
sides of a timed region, the maximum of the per-rank device times, and the sum of the units the
ranks processed.  `nccl` on GPUs, `gloo` for the same logic on CPU.

Serving a batch of independent requests on G replicas (`RequestDispatcher`): the batch is cut into G
contiguous chunks, replica r runs chunk r one request after another through its own captured graph, and
the results meet on the host of rank 0 through a key-value store -- no collective, no peer memory, no
cross-GPU load anywhere on the data path.  Because nothing on that path is a collective, a replica that
leaves between two requests stalls nobody: the collector notices the missing results after a timeout and
runs those requests itself.
"""
import os
import pickle
import threading
import time
from datetime import timedelta

import torch


class ReplicaGroup:
    def __init__(self, rank, world, local_rank, device):
        self.rank, self.world, self.local_rank, self.device = rank, world, local_rank, device

    @classmethod
    def from_env(cls, backend=None):
        """Join the process group torch.distributed.run describes in the environment (RANK, WORLD_SIZE,
        LOCAL_RANK, MASTER_ADDR, MASTER_PORT).  A single process (WORLD_SIZE unset or 1) joins nothing."""
        rank = int(os.environ.get("RANK", "0"))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        local = int(os.environ.get("LOCAL_RANK", "0"))
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        device = torch.device("cuda", local) if backend == "nccl" else torch.device("cpu")
        if backend == "nccl":
            torch.cuda.set_device(device)
        if world > 1:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            if backend == "nccl":
                dist.init_process_group("nccl", device_id=device)
            else:
                dist.init_process_group(backend)
        return cls(rank, world, local, device)

    def barrier(self):
        """All ranks arrive, then this rank's GPU work is drained."""
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    def _reduce(self, value, op):
        if self.world == 1:
            return float(value)
        import torch.distributed as dist
        t = torch.tensor([value], dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=op)
        return float(t.item())

    def max_over_ranks(self, value):
        import torch.distributed as dist
        return self._reduce(value, dist.ReduceOp.MAX)

    def sum_over_ranks(self, value):
        import torch.distributed as dist
        return self._reduce(value, dist.ReduceOp.SUM)

    def throughput(self, units_this_rank, elapsed_ms_this_rank):
        """Whole-job rate: the units all ranks processed divided by the slowest rank's time (units / s)."""
        total = self.sum_over_ranks(units_this_rank)
        ms = self.max_over_ranks(elapsed_ms_this_rank)
        return total / (ms * 1e-3), ms

    def close(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


def split_requests(n_requests, world):
    """Contiguous chunk [start, stop) of each rank: n // world requests each, the remainder to the first ranks."""
    base, extra = divmod(n_requests, world)
    bounds, start = [], 0
    for r in range(world):
        stop = start + base + (1 if r < extra else 0)
        bounds.append((start, stop))
        start = stop
    return bounds


class RequestDispatcher:
    """Runs batches of independent requests on the replicas of a ReplicaGroup.

    `infer(request) -> result` is this rank's replica (any picklable result, e.g. a CPU tensor).  Every
    rank calls `serve(requests)` with the same list; rank 0 returns (results in request order, stats), the
    other ranks return (None, stats of their own chunk).  Results travel through a TCP key-value store on
    the host (rank 0 holds it); a request whose result does not arrive within `timeout_s` is run by rank 0
    itself, so a replica that has left does not lose work.
    """

    def __init__(self, group, infer, port=None, timeout_s=30.0):
        # `infer` may be a list of callables: that many requests of this rank's chunk are in flight at a time,
        # one host thread and (on a GPU) one CUDA stream per callable, each callable being a pipeline of its own
        # (its own buffers and scratch).  A Pi0.5 inference is a chain of ~600 short dependent launches that
        # leaves most SMs idle most of the time; two or three chains side by side fill them.
        self.lanes = list(infer) if isinstance(infer, (list, tuple)) else [infer]
        self.group, self.infer, self.timeout_s = group, self.lanes[0], float(timeout_s)
        self._streams = None
        if len(self.lanes) > 1 and group.device.type == "cuda":
            self._streams = [torch.cuda.Stream(device=group.device) for _ in self.lanes]
        self.batch_id = 0
        self.store = None
        if group.world > 1:
            import torch.distributed as dist
            host = os.environ.get("MASTER_ADDR", "127.0.0.1")
            port = int(port if port is not None else int(os.environ.get("MASTER_PORT", "29500")) + 17)
            self.store = dist.TCPStore(host, port, world_size=group.world, is_master=(group.rank == 0),
                                       timeout=timedelta(seconds=max(60.0, 4 * self.timeout_s)), wait_for_workers=True)

    def _run(self, request, lane=0):
        t0 = time.perf_counter()
        if self._streams is not None:
            with torch.cuda.stream(self._streams[lane]):
                result = self.lanes[lane](request)
                self._streams[lane].synchronize()
        else:
            result = self.lanes[lane](request)
            if self.group.device.type == "cuda":
                torch.cuda.current_stream(self.group.device).synchronize()
        return result, (time.perf_counter() - t0) * 1e3

    def serve(self, requests, leave_after=None):
        """`leave_after`: (tests) this rank stops after that many requests of its chunk, as a replica that
        went away between two requests would."""
        g = self.group
        self.batch_id += 1
        n = len(requests)
        lo, hi = split_requests(n, g.world)[g.rank]
        t_start = time.perf_counter()
        mine, lat = {}, []
        todo = iter(enumerate(range(lo, hi)))
        lock = threading.Lock()
        errors = []

        def work(lane):
            while True:
                with lock:
                    nxt = next(todo, None)
                if nxt is None or (leave_after is not None and nxt[0] >= leave_after):
                    return
                i = nxt[1]
                try:
                    result, ms = self._run(requests[i], lane)
                except BaseException as exc:           # a worker thread must not swallow its pipeline's error
                    with lock:
                        errors.append(exc)
                    return
                with lock:
                    lat.append(ms)
                    if g.rank == 0:
                        mine[i] = result
                    else:
                        self.store.set(f"b{self.batch_id}/r{i}", pickle.dumps((result, ms)))

        if len(self.lanes) == 1:
            work(0)
        else:
            threads = [threading.Thread(target=work, args=(lane,)) for lane in range(len(self.lanes))]
            for t in threads:
                t.start()
            for t in threads:
                t.join()
        if errors:
            raise errors[0]
        stats = {"rank": g.rank, "chunk": (lo, hi), "done": len(lat), "latencies_ms": lat, "requeued": []}
        if g.rank != 0:
            return None, stats
        results = [None] * n
        for i, r in mine.items():
            results[i] = r
        deadline = time.perf_counter() + self.timeout_s
        for i in range(n):
            if results[i] is not None:
                continue
            key = f"b{self.batch_id}/r{i}"
            try:
                self.store.wait([key], timedelta(seconds=max(0.05, deadline - time.perf_counter())))
                results[i], ms = pickle.loads(self.store.get(key))
                lat.append(ms)
            except Exception:                      # the owner of this request is gone: run it here
                results[i], ms = self._run(requests[i])
                lat.append(ms)
                stats["requeued"].append(i)
        wall = time.perf_counter() - t_start
        lat_sorted = sorted(lat)
        pick = lambda q: lat_sorted[min(len(lat_sorted) - 1, int(q * len(lat_sorted)))]
        stats.update(requests=n, wall_s=wall, requests_per_s=n / wall, p50_ms=pick(0.50), p99_ms=pick(0.99),
                     latencies_ms=lat)
        return results, stats
