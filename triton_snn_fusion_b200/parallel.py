"""Batch sharding across ranks and the one collective of the path: the logits gather.

The reference is single-GPU and has no distributed code. Whole-network inference shards by image
(no op mixes samples once BatchNorm is folded), so each rank runs the full layer list on a
contiguous slice of the global batch and the ranks exchange nothing but their logits.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(global_batch: int, rank: int, world: int) -> Tuple[int, int]:
    """[start, stop) of the images rank `rank` owns; equal contiguous slices."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    if global_batch % world:
        raise ValueError(f"global batch {global_batch} is not divisible by {world} ranks")
    per = global_batch // world
    return rank * per, (rank + 1) * per


def gather_logits(local: torch.Tensor, out: Optional[torch.Tensor] = None, group=None) -> torch.Tensor:
    """All ranks' [B/world, classes] logits -> [B, classes] in rank order (= global image order).

    One `all_gather_into_tensor` on the default (or given) process group: NCCL on GPUs, gloo in the
    CPU tests. With a single rank (or no initialised group) the input is returned unchanged.
    """
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return local
    world = dist.get_world_size(group)
    if out is None:
        out = torch.empty((local.shape[0] * world,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    elif out.shape[0] != local.shape[0] * world:
        raise ValueError("gather_logits: output has the wrong leading size")
    dist.all_gather_into_tensor(out, local.contiguous(), group=group)
    return out
