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


def sum_over_ranks(value, dist=None, device="cpu"):
    """Sum of `value` (a float) over all ranks; identity without a process group."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def gather_floats(value, dist=None, device="cpu"):
    """`value` of every rank, in rank order, on every rank."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return [float(value)]
    world = dist.get_world_size()
    t = torch.zeros(world, dtype=torch.float64, device=device)
    t[dist.get_rank()] = float(value)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return [float(v) for v in t.tolist()]


def aggregate_throughput(units_per_rank, seconds, dist=None, device="cpu"):
    """Whole-job units per second: every rank's units over the slowest rank's time."""
    world = dist.get_world_size() if (dist is not None and dist.is_initialized()) else 1
    return units_per_rank * world / max_over_ranks(seconds, dist, device)


def barrier(dist=None):
    if dist is not None and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


def _parse_cpulist(text):
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def bind_to_gpu_numa_node(device_index, sysfs="/sys/bus/pci/devices"):
    """Restrict this process to the CPUs next to GPU `device_index` (its PCI device's local_cpulist), so
    that the pinned host buffers it allocates afterwards are first touched on that GPU's NUMA node:
    with one rank per GPU, host <-> device copies then stay off the inter-socket link.  Best effort:
    returns the sorted CPU list it bound to, or None when the topology cannot be read (no sysfs entry,
    a container without the node files) or would leave no allowed CPU."""
    import os
    try:
        p = torch.cuda.get_device_properties(device_index)
        bdf = "%04x:%02x:%02x.0" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)
        with open(os.path.join(sysfs, bdf, "local_cpulist")) as f:
            local = _parse_cpulist(f.read())
        allowed = os.sched_getaffinity(0)
        target = local & allowed
        if not target or target == allowed:
            return None
        os.sched_setaffinity(0, target)
        return sorted(target)
    except Exception:
        return None
