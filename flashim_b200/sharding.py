"""Batch sharding of independent image pairs over the GPUs of one node.

The conv path has no cross-sample arithmetic (FlashIM itself only stacks the two match directions on the batch axis,
flashim/models/romav2/model.py:251-268), so N GPUs each take a contiguous slice of the pairs and never exchange data:
no collective is part of the data path. ``torch.distributed`` is used only to line the ranks up for timing (a barrier)
and to combine their clocks and counts (a MAX and a SUM of one scalar).
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import torch


def shard_pairs(total_pairs: int, rank: int, world: int) -> tuple[int, int]:
    """``(first_pair, pair_count)`` of ``rank``: contiguous, sizes differ by at most one, earlier ranks take the extra."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(total_pairs, world)
    count = base + (1 if rank < extra else 0)
    first = rank * base + min(rank, extra)
    return first, count


@dataclass
class Ranks:
    """This process among the ranks of a ``torchrun`` launch (one process per GPU)."""

    rank: int = 0
    world: int = 1
    local_rank: int = 0
    backend: str | None = None

    @classmethod
    def from_env(cls, backend: str = "nccl") -> "Ranks":
        world = int(os.environ.get("WORLD_SIZE", "1"))
        ranks = cls(int(os.environ.get("RANK", "0")), world, int(os.environ.get("LOCAL_RANK", "0")))
        if world > 1:
            import torch.distributed as dist

            if not dist.is_initialized():
                kwargs = {}
                if backend == "nccl":
                    torch.cuda.set_device(ranks.local_rank)
                    kwargs["device_id"] = torch.device("cuda", ranks.local_rank)
                dist.init_process_group(backend, **kwargs)
            ranks.backend = backend
        return ranks

    def _device(self):
        return torch.device("cuda", self.local_rank) if self.backend == "nccl" else torch.device("cpu")

    def barrier(self) -> None:
        if self.world > 1:
            import torch.distributed as dist

            dist.barrier()

    def _reduce(self, value: float, op) -> float:
        if self.world == 1:
            return float(value)
        import torch.distributed as dist

        t = torch.tensor([value], dtype=torch.float64, device=self._device())
        dist.all_reduce(t, op=op)
        return float(t.item())

    def max(self, value: float) -> float:
        import torch.distributed as dist

        return self._reduce(value, dist.ReduceOp.MAX)

    def sum(self, value: float) -> float:
        import torch.distributed as dist

        return self._reduce(value, dist.ReduceOp.SUM)

    def gather_strings(self, value: str) -> list[str]:
        """Every rank's string on every rank (used to compare per-shard output digests)."""
        if self.world == 1:
            return [value]
        import torch.distributed as dist

        out: list = [None] * self.world
        dist.all_gather_object(out, value)
        return out

    def close(self) -> None:
        if self.world > 1:
            import torch.distributed as dist

            if dist.is_initialized():
                dist.destroy_process_group()
