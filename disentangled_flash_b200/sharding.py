"""Batch sharding for multi-GPU inference: independent sequences, no collective in the forward.

Every sequence is independent through the whole encoder, so N GPUs run N
replicas of the model on disjoint slices of the batch.  The only
communication is after the fact: gathering per-rank results (or checksums)
so that one rank can compare them with a reference.  The helpers work with
any ``torch.distributed`` backend (NCCL on GPUs, gloo in CPU tests).
"""

from __future__ import annotations

from collections.abc import Sequence

import torch
import torch.distributed as dist


def shard_indices(n_items: int, rank: int, world_size: int) -> list[int]:
    """Indices owned by ``rank``: item k goes to rank ``k mod world_size``.

    Interleaving (instead of contiguous blocks) gives every rank the same mix
    when items are ordered by cost, e.g. sequences grouped by bucket length.
    """

    if not 0 <= rank < world_size:
        raise ValueError("rank out of range")
    return list(range(rank, n_items, world_size))


def shard_buckets(bucket_sizes: dict[int, int], rank: int, world_size: int) -> dict[int, list[int]]:
    """Per-bucket interleaved shards: ``{length: [sequence indices of this rank]}``."""

    return {length: shard_indices(count, rank, world_size) for length, count in sorted(bucket_sizes.items())}


def gather_for_check(local: torch.Tensor, group=None) -> list[torch.Tensor] | None:
    """Gather equally-shaped per-rank tensors on every rank (rank order).

    Used only for checking results after the timed region.  Returns
    ``[local]`` when ``torch.distributed`` is not initialised.
    """

    if not (dist.is_available() and dist.is_initialized()):
        return [local]
    world = dist.get_world_size(group)
    out = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(out, local.contiguous(), group=group)
    return out


def reassemble(shards: Sequence[torch.Tensor], n_items: int) -> torch.Tensor:
    """Invert :func:`shard_indices`: interleave per-rank results back into item order."""

    world = len(shards)
    out = torch.empty((n_items, *shards[0].shape[1:]), dtype=shards[0].dtype, device=shards[0].device)
    for rank, shard in enumerate(shards):
        idx = shard_indices(n_items, rank, world)
        out[idx] = shard[: len(idx)]
    return out


def max_over_ranks(value: float, device: torch.device | str = "cpu", group=None) -> float:
    """Slowest rank's time: the number a multi-GPU measurement must report."""

    if not (dist.is_available() and dist.is_initialized()):
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


__all__ = ["gather_for_check", "max_over_ranks", "reassemble", "shard_buckets", "shard_indices"]
