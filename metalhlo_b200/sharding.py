"""How the hot path's workloads are split over the GPUs of one node (one process per GPU).

Nothing here talks to a device: these are the index computations `bench.py` and multi-GPU hosts share, kept apart so
that they can be tested with CPU process groups. The partitioning follows the table of the path's configurations:
rows of the norm sweep, (batch x head) of attention, batches of batched GEMMs and of the GPT-2 forward pass are
independent and need no collective; the large GEMM splits B and C by columns and exchanges C.
"""
from __future__ import annotations

import dataclasses


@dataclasses.dataclass(frozen=True)
class Shard:
    start: int  # first unit this rank owns
    count: int  # number of units it owns

    @property
    def stop(self) -> int:
        return self.start + self.count


def contiguous_shard(total: int, world: int, rank: int) -> Shard:
    """Contiguous block of `total` units for `rank`; the first `total % world` ranks get one unit more."""
    if world < 1 or not 0 <= rank < world or total < 0:
        raise ValueError(f"bad shard request: total={total} world={world} rank={rank}")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return Shard(start, base + (1 if rank < extra else 0))


def column_shard(n: int, world: int, rank: int, multiple: int = 8) -> Shard:
    """Column block of a GEMM's B and C. Blocks are equal and a multiple of `multiple` columns (16-byte rows for
    16-bit elements, which the TMA descriptors and the vector stores of the epilogue need)."""
    if n % (world * multiple) != 0:
        raise ValueError(f"{n} columns do not split into {world} blocks that are multiples of {multiple}")
    return Shard(rank * (n // world), n // world)


def weak_rows(rows_per_gpu: int, world: int, rank: int) -> Shard:
    """Weak scaling of the norm sweep: every rank owns `rows_per_gpu` rows of a [world * rows_per_gpu, hidden] tensor."""
    return Shard(rank * rows_per_gpu, rows_per_gpu)


def max_over_ranks(value: float, dist=None, device=None) -> float:
    """The slowest rank's time: every multi-GPU number is reported as the maximum over ranks."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    import torch

    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def exchange_handles(own: bytes, dist) -> list[bytes]:
    """All ranks' 64-byte IPC handles in rank order (the set-up step of the GEMM whose epilogue stores into peers)."""
    handles: list = [None] * dist.get_world_size()
    dist.all_gather_object(handles, own)
    return handles
