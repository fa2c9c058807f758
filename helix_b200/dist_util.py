"""The only cross-rank communication of the multi-GPU sweep: a barrier and a max over ranks.

Shapes are independent, so the data path has no collective; ranks only agree on the slowest
rank's time (NCCL on GPUs, gloo in the CPU tests).
"""
import torch


def max_over_ranks(value, dist=None, device="cpu"):
    """Largest `value` (a float) over all ranks of the default process group; identity without one."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def aggregate_throughput(units_per_rank, seconds, dist=None, device="cpu"):
    """Whole-job units per second: every rank's units over the slowest rank's time."""
    world = dist.get_world_size() if (dist is not None and dist.is_initialized()) else 1
    return units_per_rank * world / max_over_ranks(seconds, dist, device)


def barrier(dist=None):
    if dist is not None and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
