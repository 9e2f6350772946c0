"""Partitioning of one joint-attention call over the GPUs of a node.

Every (image, head) pair is an independent attention problem (the reference itself runs
attention per image and per head, src/klein/zflux2_resident.zig:1798-1833), so the path shards
with no exchange step:

* ``images``  – one or more whole images (seeds) per rank: pointer offset ``b * tokens * ld``;
* ``heads``   – a contiguous range of heads per rank: pointer offset ``h0 * 128`` with the full
  token stride ``ld = H * 128`` (a column slice of the token-major tensors, no repacking).

The only collective is the optional all-gather of the head shards' outputs when a whole block is
timed: every rank contributes its heads in head-major form ``[heads_r, tokens, 128]`` and the
gathered buffer is head-major ``[H, tokens, 128]`` (rank order == head order).

This module is pure host logic (no CUDA): ``tests/test_shard_gloo.py`` runs it on CPU ranks.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Shard:
    rank: int
    world: int
    begin: int  # first unit (head or image) of this rank
    end: int    # one past the last

    @property
    def count(self) -> int:
        return self.end - self.begin


def split(units: int, world: int, rank: int) -> Shard:
    """Contiguous, as even as possible: the first ``units % world`` ranks get one unit more.

    30 heads over 4 ranks -> 8, 8, 7, 7; over 8 ranks -> 4, 4, 4, 4, 4, 4, 3, 3.
    """
    if world <= 0 or not (0 <= rank < world) or units < 0:
        raise ValueError("bad shard request")
    base, extra = divmod(units, world)
    begin = rank * base + min(rank, extra)
    return Shard(rank, world, begin, begin + base + (1 if rank < extra else 0))


def all_shards(units: int, world: int) -> list[Shard]:
    return [split(units, world, r) for r in range(world)]


def max_imbalance(units: int, world: int) -> float:
    """Largest shard divided by the mean shard: the bound on strong-scaling efficiency."""
    shards = all_shards(units, world)
    return max(s.count for s in shards) * world / float(units)


def all_gather_heads(local_hm, heads: int, rank: int, world: int, group=None):
    """All-gather of head-major outputs ``[heads_r, tokens, 128]`` into ``[heads, tokens, 128]``.

    Shards may differ in size (30 heads over 4 ranks), so every rank pads to the largest shard,
    one ``all_gather_into_tensor`` moves the padded blocks, and the result is compacted locally.
    Works with any ``torch.distributed`` backend (NCCL on GPUs, gloo on CPU).
    """
    import torch
    import torch.distributed as dist

    shards = all_shards(heads, world)
    biggest = max(s.count for s in shards)
    tokens, d = local_hm.shape[1], local_hm.shape[2]
    padded = local_hm
    if local_hm.shape[0] != biggest:
        padded = torch.zeros((biggest, tokens, d), dtype=local_hm.dtype, device=local_hm.device)
        padded[: local_hm.shape[0]] = local_hm
    gathered = torch.empty((world * biggest, tokens, d), dtype=local_hm.dtype, device=local_hm.device)
    dist.all_gather_into_tensor(gathered, padded.contiguous(), group=group)
    if all(s.count == biggest for s in shards):
        return gathered
    parts = [gathered[r * biggest: r * biggest + s.count] for r, s in enumerate(shards)]
    return torch.cat(parts, dim=0)
