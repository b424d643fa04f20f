"""Data-parallel sharding of the sampling workload over ranks (one process per GPU).

The graph is replicated on every rank; the independent units — minibatches or walkers — are dealt
to the ranks and no tensor ever crosses ranks on the data path.  The only collective is the
end-of-run reduction of statistics.  (The reference has no multi-GPU support at all:
src/distributed/context.h is an empty struct.)
"""
from typing import Tuple

import torch


def shard_batches(batches: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Round-robin: global batch b goes to rank b mod world.  `batches` is [num_batches, batch_size]."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    return batches[rank::world].contiguous()


def batch_owner(batch_index: int, world: int) -> int:
    return batch_index % world


def shard_batch_ids(num_batches: int, rank: int, world: int) -> torch.Tensor:
    """Global numbers of the minibatches shard_batches hands to `rank` (int64, on the CPU).  Passed to the batched
    sampler as `batch_ids`, they key every minibatch's random stream by its GLOBAL number, so the sample a
    minibatch receives does not depend on the number of ranks or on how a rank groups its minibatches into calls."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    return torch.arange(rank, int(num_batches), world, dtype=torch.int64)


def shard_walkers(num_walkers: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous ranges: returns (offset, count) of the walkers of `rank`.  The offset is passed to the
    walk kernel as `walker_offset`, which keys every walker's random stream by its GLOBAL index, so the
    union of the ranks' traces equals the single-GPU trace."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, rem = divmod(int(num_walkers), world)
    count = base + (1 if rank < rem else 0)
    offset = rank * base + min(rank, rem)
    return offset, count


def reduce_run_stats(seconds: float, units: int, device=None, group=None) -> Tuple[float, int]:
    """(max over ranks of the elapsed seconds, sum over ranks of the processed units).  Uses
    torch.distributed when it is initialised (NCCL on GPUs, gloo on CPUs), else returns the inputs."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return float(seconds), int(units)
    t = torch.tensor([seconds], dtype=torch.float64, device=device)
    u = torch.tensor([units], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    dist.all_reduce(u, op=dist.ReduceOp.SUM, group=group)
    return float(t.item()), int(round(u.item()))
