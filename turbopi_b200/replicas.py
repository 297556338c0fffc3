"""Process plumbing for N > 1 GPUs.

The inference path does not shard: the reference serves one policy per process and its quantised
kernels have no exchange step, so N GPUs run N independent replicas (one process per GPU, launched
by torch.distributed.run).  The only communication is the measurement protocol: a barrier on both
sides of a timed region, the maximum of the per-rank device times, and the sum of the units the
ranks processed.  `nccl` on GPUs, `gloo` for the same logic on CPU.
"""
import os

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
