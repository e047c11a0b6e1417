"""Batch sharding for multi-GPU runs: one process per GPU, contiguous split of the batch axis.

Every cell (batch element, grid cell) of a Clebsch-Gordan product is independent
(Gpart::for_each_cell_multi, core/Gpart.hpp:325-360 of GElib), so the only multi-GPU mode is to give each
rank a contiguous slice of the batch; the products need no collective.  The two places where ranks talk
are off the data path: timing (max over ranks) and the gradient of an operand that is broadcast over the
batch (batch size 1), which is the sum over all cells and therefore over all ranks.
"""
import torch
import torch.distributed as dist


def shard_bounds(total, rank, world):
    """[begin, end) of rank's contiguous slice of `total` cells; slices differ by at most one cell."""
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_batch(t, rank, world):
    """The rank's slice of a tensor along the batch axis; a broadcast operand (batch 1) is replicated."""
    if t.size(0) == 1:
        return t
    b, e = shard_bounds(t.size(0), rank, world)
    return t[b:e]


def max_over_ranks(value, device=None):
    """max of a python float over all ranks (identity without an initialised process group)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def allreduce_broadcast_grad(grad):
    """Sums the gradient of a batch-broadcast operand over ranks (each rank holds the sum over its cells)."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        g = torch.view_as_real(grad) if grad.is_complex() else grad
        dist.all_reduce(g, op=dist.ReduceOp.SUM)
    return grad
