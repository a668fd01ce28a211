"""Batch-sharded execution over the GPUs of one node: one process per GPU, replicated weights,
every rank runs its slice of the batch through the same compiled function and the outputs are
all-gathered (NCCL over NVLink on GPUs; gloo in the CPU tests).  The reference has no
distributed code; the batch symbol of its symbolic-shape machinery is what makes one compiled
plan serve the per-rank slice."""
from __future__ import annotations

from typing import Callable, List, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_bounds(total: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced split: the first ``total % world`` ranks get one extra sample."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def gather_batch(local: torch.Tensor, total: int, group=None) -> torch.Tensor:
    """All-gathers per-rank output slices (dim 0) into the full batch on every rank."""
    world = dist.get_world_size(group)
    if world == 1:
        return local
    rank = dist.get_rank(group)
    sizes = [shard_bounds(total, world, r)[1] - shard_bounds(total, world, r)[0] for r in range(world)]
    if len(set(sizes)) == 1 and local.is_cuda:
        out = local.new_empty((total,) + tuple(local.shape[1:]))
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    pad = max(sizes)
    buf = local.new_zeros((pad,) + tuple(local.shape[1:]))
    buf[: sizes[rank]] = local
    parts = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(parts, buf, group=group)
    return torch.cat([p[:n] for p, n in zip(parts, sizes)], dim=0)


class BatchShardedRunner:
    """Wraps a compiled callable: ``runner(*full_batch_inputs)`` runs this rank's slice and returns the
    gathered full-batch output.  Inputs whose leading extent is not the batch are passed whole."""

    def __init__(self, fn: Callable, group=None):
        self.fn, self.group = fn, group

    def __call__(self, *inputs: torch.Tensor) -> torch.Tensor:
        world, rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        total = inputs[0].shape[0]
        lo, hi = shard_bounds(total, world, rank)
        local = [i[lo:hi] if i.dim() > 0 and i.shape[0] == total else i for i in inputs]
        out = self.fn(*local)
        if isinstance(out, (list, tuple)):
            out = out[0]
        return gather_batch(out, total, self.group)
