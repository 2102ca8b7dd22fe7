"""Batch sharding of the op path over several GPUs (one process per GPU).

Every op on the path is elementwise over independent elements, and masked_select over a
batch-major tensor is the order-preserving concatenation of the per-shard results.  So a batch is
cut into contiguous blocks of its leading dimension, each rank runs the kernels on its block with
no data-path communication, and the only exchange is one all-gather of a single int64 per rank -
the number of elements its masked_select produced - from which every rank derives the offset of
its segment in the global (concatenated) result.  The reference has no multi-device support
(`webgpu_device_count = 1`, csrc/core/webgpu_device_guard.h:9).
"""
from __future__ import annotations

from typing import Sequence

import torch
import torch.distributed as dist


def shard_range(total: int, rank: int, world_size: int) -> tuple[int, int]:
    """Half-open range [lo, hi) of the leading dimension owned by `rank`.

    Blocks are contiguous and as even as possible; the first `total % world_size` ranks get one
    extra item, so any world size works, including ones larger than the batch.
    """
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError(f"rank {rank} is outside a world of {world_size}")
    base, extra = divmod(int(total), world_size)
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    return lo, hi


def exclusive_offsets(counts: Sequence[int]) -> list[int]:
    """Global output offset of each rank's segment: the exclusive prefix sum of the counts."""
    out, acc = [], 0
    for c in counts:
        out.append(acc)
        acc += int(c)
    return out


def allgather_counts(local_count: int, device: torch.device | str = "cpu", group=None) -> list[int]:
    """All-gather one int64 per rank.  With the NCCL backend `device` must be the rank's CUDA
    device (8 bytes per rank cross NVLink); with gloo it is the CPU."""
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return [int(local_count)]
    world = dist.get_world_size(group)
    mine = torch.tensor([int(local_count)], dtype=torch.int64, device=device)
    gathered = torch.empty(world, dtype=torch.int64, device=device)
    dist.all_gather_into_tensor(gathered, mine, group=group)
    return [int(v) for v in gathered.cpu().tolist()]


def global_segment(local_count: int, device: torch.device | str = "cpu", group=None) -> tuple[int, int, list[int]]:
    """(offset of this rank's segment, total selected elements, all counts)."""
    counts = allgather_counts(local_count, device, group)
    rank = dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0
    offsets = exclusive_offsets(counts)
    return offsets[rank], sum(counts), counts
