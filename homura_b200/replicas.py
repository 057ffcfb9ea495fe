"""Host-side plumbing for the replica layout: one process per GPU, weights replicated, the
global batch of independent sequences split into contiguous shards, no collective on the
token path.  torch.distributed is used only for the barriers around a timed region and for the
max-over-ranks of the device time (NCCL on GPUs, gloo on CPU)."""
from __future__ import annotations

import os
from typing import List, Tuple


def shard_sequences(n_sequences: int, rank: int, world: int) -> range:
    """Contiguous shard of sequence ids owned by `rank` (sizes differ by at most one)."""
    if world < 1 or not 0 <= rank < world or n_sequences < 0:
        raise ValueError("bad shard arguments")
    base, extra = divmod(n_sequences, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def aggregate_rate(units_per_rank: List[int], seconds_max_over_ranks: float) -> float:
    """Whole-job throughput: all units processed by all ranks over the slowest rank's time."""
    if seconds_max_over_ranks <= 0:
        raise ValueError("non-positive time")
    return sum(units_per_rank) / seconds_max_over_ranks


class Rendezvous:
    """rank / world / local_rank from the torchrun environment plus barrier() and max()."""

    def __init__(self, backend: str | None = None):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self._dist = None
        self._cuda = False
        if self.world > 1:
            import torch
            import torch.distributed as dist

            if backend is None:
                backend = "nccl" if torch.cuda.is_available() else "gloo"
            if backend == "nccl":
                torch.cuda.set_device(self.local)
                dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
                self._cuda = True
            else:
                dist.init_process_group(backend)
            self._dist = dist

    def barrier(self):
        if self._dist is None:
            return
        self._dist.barrier()
        if self._cuda:
            import torch

            torch.cuda.synchronize()

    def max(self, value: float) -> float:
        if self._dist is None:
            return float(value)
        import torch

        t = torch.tensor([float(value)], dtype=torch.float64, device="cuda" if self._cuda else "cpu")
        self._dist.all_reduce(t, op=self._dist.ReduceOp.MAX)
        return float(t.item())

    def gather_ints(self, value: int) -> List[int]:
        if self._dist is None:
            return [int(value)]
        import torch

        t = torch.zeros(self.world, dtype=torch.int64, device="cuda" if self._cuda else "cpu")
        t[self.rank] = int(value)
        self._dist.all_reduce(t, op=self._dist.ReduceOp.SUM)
        return [int(v) for v in t.tolist()]

    def close(self):
        if self._dist is not None:
            self._dist.destroy_process_group()
            self._dist = None
