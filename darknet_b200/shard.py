"""Batch sharding across the GPUs of one box (one process per GPU).

Inference images are independent (per-image GEMM, rolling batchnorm statistics, no
cross-image layer: src/convolutional_layer.c:461-475, src/batchnorm_layer.c:151), so
the batch is cut into contiguous slices, every rank holds a full replica of the
weights, and there is no collective on the data path.  Ranks talk only to agree on
timing (max over ranks) and, when a caller wants one array, to gather outputs on
rank 0.  The reference's only multi-device code is its training loop
(src/network.c:857-875: one thread and one network per GPU); this is the same
pattern for inference.
"""
from __future__ import annotations

import numpy as np


def shard_batch(total: int, world: int, rank: int) -> tuple[int, int]:
    """(first image, image count) of `rank`'s contiguous slice; the first `total % world`
    ranks take one extra image, so any batch size is covered."""
    if world < 1 or not 0 <= rank < world or total < 0:
        raise ValueError(f"bad shard request: total={total} world={world} rank={rank}")
    base, extra = divmod(total, world)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return start, count


def max_over_ranks(value: float, device=None) -> float:
    """The job's time is its slowest rank's time."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device or "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_outputs(local: np.ndarray, total: int):
    """Concatenate every rank's output slice on rank 0 in image order (None elsewhere).
    Off the hot path: used by callers that want the whole batch in one array."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return local
    world, rank = dist.get_world_size(), dist.get_rank()
    parts = [None] * world if rank == 0 else None
    dist.gather_object(local, parts, dst=0)
    if rank != 0:
        return None
    out = np.concatenate([p for p in parts if p is not None and len(p)], axis=0)
    assert out.shape[0] == total
    return out


def cpus_near_gpu(gpu_index: int, affinity_words=None, ncpu: int | None = None) -> list[int]:
    """Host CPUs of the NUMA node the GPU hangs off, from NVML's read-only affinity query
    (`affinity_words`: the 64-bit mask words, passed in by tests).  Empty when NVML is not usable."""
    import os
    ncpu = ncpu or os.cpu_count() or 1
    if affinity_words is None:
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
            affinity_words = list(pynvml.nvmlDeviceGetCpuAffinity(h, (ncpu + 63) // 64))
        except Exception:
            return []
    cpus = [64 * w + b for w, word in enumerate(affinity_words) for b in range(64) if (int(word) >> b) & 1]
    return [c for c in cpus if c < ncpu]


def bind_near_gpu(gpu_index: int) -> list[int]:
    """One process per GPU: run this rank on the CPUs next to its GPU, so that the pinned host buffers it
    allocates afterwards (first touch) sit in that node's memory and its PCIe copies do not cross the
    socket interconnect.  Returns the CPUs chosen ([] = left as it was).  Only CPUs the process may
    already use are kept."""
    import os
    if not hasattr(os, "sched_setaffinity"):
        return []
    near = set(cpus_near_gpu(gpu_index))
    allowed = os.sched_getaffinity(0)
    chosen = sorted(near & allowed)
    if not chosen or len(chosen) == len(allowed):
        return []
    try:
        os.sched_setaffinity(0, chosen)
    except OSError:
        return []
    return chosen
