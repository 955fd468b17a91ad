"""Batch replicas across the GPUs of one box: the only multi-GPU form the CNN path needs.

Images are independent, so rank g of G takes images [g*N/G, (g+1)*N/G) (remainder spread
over the first ranks), runs its own executable on its own GPU and rank 0 gathers the
outputs. There is no collective on the data path; torch.distributed only moves the
scatter/gather of host arrays and the barrier / max-over-ranks around a timed region.
The reference has no multi-device form at all (collectives are UNIMPLEMENTED,
runtime/driver/torq_device.c:235-240); this follows the benchmark configuration's
"split across GPUs by batch".
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist


def shard_bounds(n_items: int, world: int, rank: int) -> tuple[int, int]:
    """Half-open range of the items rank `rank` owns."""
    base, rem = divmod(n_items, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def _torch_dtype(np_dtype):
    return torch.from_numpy(np.zeros(1, np_dtype)).dtype


def scatter_batch(x_global: np.ndarray | None, n_items: int, item_shape, dtype, src: int = 0) -> np.ndarray:
    """Rank `src` holds the whole batch; every rank gets its shard (shards may differ by one
    item, so this is point-to-point sends rather than an equal-size scatter)."""
    world, rank = dist.get_world_size(), dist.get_rank()
    lo, hi = shard_bounds(n_items, world, rank)
    if rank == src:
        reqs = []
        for r in range(world):
            if r == src:
                continue
            rlo, rhi = shard_bounds(n_items, world, r)
            reqs.append(dist.isend(torch.from_numpy(np.ascontiguousarray(x_global[rlo:rhi])), dst=r))
        for q in reqs:
            q.wait()
        return np.ascontiguousarray(x_global[lo:hi])
    out = torch.empty((hi - lo,) + tuple(item_shape), dtype=_torch_dtype(dtype))
    dist.recv(out, src=src)
    return out.numpy()


def gather_batch(y_local: np.ndarray, n_items: int, dst: int = 0) -> np.ndarray | None:
    """Concatenate every rank's shard on rank `dst` (None elsewhere)."""
    world, rank = dist.get_world_size(), dist.get_rank()
    t = torch.from_numpy(np.ascontiguousarray(y_local))
    if rank != dst:
        dist.send(t, dst=dst)
        return None
    parts = []
    for r in range(world):
        if r == dst:
            parts.append(t)
            continue
        rlo, rhi = shard_bounds(n_items, world, r)
        buf = torch.empty((rhi - rlo,) + tuple(t.shape[1:]), dtype=t.dtype)
        dist.recv(buf, src=r)
        parts.append(buf)
    return torch.cat(parts, 0).numpy()


def max_over_ranks(value: float, device: str = "cpu") -> float:
    """Time of the slowest rank (multi-GPU timings are reported as the max)."""
    t = torch.tensor([value], dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _parse_cpulist(text: str) -> set[int]:
    cpus: set[int] = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def numa_cpus_of_gpu(pci_domain: int, pci_bus: int, pci_device: int, sysfs: str = "/sys") -> set[int]:
    """CPUs of the NUMA node the GPU hangs off (empty when the platform does not say)."""
    import os
    dev = os.path.join(sysfs, "bus", "pci", "devices", f"{pci_domain:04x}:{pci_bus:02x}:{pci_device:02x}.0")
    try:
        node = int(open(os.path.join(dev, "numa_node")).read().strip())
        if node < 0:
            return set()
        return _parse_cpulist(open(os.path.join(sysfs, "devices", "system", "node", f"node{node}", "cpulist")).read())
    except (OSError, ValueError):
        return set()


def pin_rank_to_gpu_numa_node(cuda_ordinal: int, sysfs: str = "/sys") -> list[int]:
    """Restricts this process to the CPUs next to its GPU, so that the pinned staging buffers it allocates afterwards
    (first touch) and its copy submissions stay on that node: with eight ranks feeding eight GPUs from one host, remote
    staging memory is what costs end-to-end throughput. Returns the CPUs now allowed ([] = nothing changed: the
    platform gives no node, or none of its CPUs is in this process's allowed set)."""
    import os
    if not hasattr(os, "sched_setaffinity"):
        return []
    p = torch.cuda.get_device_properties(cuda_ordinal)
    cpus = numa_cpus_of_gpu(getattr(p, "pci_domain_id", 0), getattr(p, "pci_bus_id", 0), getattr(p, "pci_device_id", 0), sysfs)
    allowed = cpus & set(os.sched_getaffinity(0))
    if not allowed:
        return []
    os.sched_setaffinity(0, allowed)
    return sorted(allowed)
