"""Batch sharding across GPUs: independent replicas, no collective on the data path.

Whole-network inference shards over the batch dimension only.  Every rank (one process per GPU)
owns a full copy of the weights and a contiguous slice of the images; the only exchange is one
all-gather of the logits after the last layer.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(total: int, rank: int, world: int):
    """Contiguous [begin, end) of `total` items for `rank`; the first total % world ranks get one more."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def gather_logits(local: torch.Tensor, total: int) -> torch.Tensor:
    """All-gather per-rank logits [n_r, classes] into [total, classes] in global image order.

    Works with any initialised process group (NCCL for CUDA tensors, gloo for CPU tensors).  Ranks
    may hold different counts (shard_range), so shards are padded to the largest count for the
    collective and trimmed afterwards.
    """
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return local
    world, rank = dist.get_world_size(), dist.get_rank()
    counts = [shard_range(total, r, world)[1] - shard_range(total, r, world)[0] for r in range(world)]
    if local.shape[0] != counts[rank]:
        raise ValueError(f"rank {rank} holds {local.shape[0]} rows, expected {counts[rank]}")
    width = max(counts)
    padded = local
    if local.shape[0] < width:
        padded = torch.zeros((width, *local.shape[1:]), dtype=local.dtype, device=local.device)
        padded[: local.shape[0]] = local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded.contiguous())
    return torch.cat([p[:c] for p, c in zip(parts, counts)], dim=0)


def bind_to_gpu_cpus(device_index: int) -> bool:
    """Pin the calling process to the CPU cores NVML reports as local to GPU `device_index` (its NUMA node), so
    that the pinned host buffers it allocates next, and the copies from them, do not cross the socket link.
    With eight replicas copying 617 MB per step each, unplaced buffers leave the host side as the bottleneck.
    Changes only this process's CPU affinity; returns False (and changes nothing) when NVML is unavailable."""
    try:
        import pynvml
        pynvml.nvmlInit()
        try:
            uuid = "GPU-" + str(torch.cuda.get_device_properties(device_index).uuid)
            handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
        except Exception:
            handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
        pynvml.nvmlDeviceSetCpuAffinity(handle)
        return True
    except Exception:
        return False

