"""Partitioning of sigmoid-attention work over the GPUs of one box.

Every (batch, head) pair is an independent attention problem (the reference's grid axis 1 is
``B * H``, ``src/triton_sigmoid/sigmoid_triton_dense.py:534``), so a multi-GPU run needs no
collective on the data path: each rank (one process per GPU) owns a contiguous block of
batches, or, when there are fewer batches than ranks, a block of heads of one batch group.
``gather_for_verification`` is the only place where ranks talk, and it is test/bench code.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch


def split_even(n: int, parts: int, idx: int) -> Tuple[int, int]:
    """Half-open range of the `idx`-th of `parts` near-equal contiguous chunks of range(n)."""
    if parts <= 0 or not (0 <= idx < parts):
        raise ValueError(f"bad partition index {idx} of {parts}")
    base, extra = divmod(n, parts)
    lo = idx * base + min(idx, extra)
    return lo, lo + base + (1 if idx < extra else 0)


@dataclass(frozen=True)
class Shard:
    """The (batch, head) block a rank owns: batches [b0, b1) x heads [h0, h1)."""

    b0: int
    b1: int
    h0: int
    h1: int

    @property
    def units(self) -> int:
        return (self.b1 - self.b0) * (self.h1 - self.h0)


def plan_shard(B: int, H: int, world: int, rank: int) -> Shard:
    """Batch-first partition of the B x H independent units over `world` ranks.

    world <= B: contiguous batch slabs (lengths and bias shard with them).
    world >  B: the ranks are divided among the batches and each group splits the heads.
    Every unit is owned by exactly one rank; a rank may own nothing when world > B * H.
    """
    if world <= B:
        b0, b1 = split_even(B, world, rank)
        return Shard(b0, b1, 0, H)
    # more ranks than batches: rank -> (batch, head block)
    b = rank * B // world
    first = -(-b * world // B)          # first rank whose batch is b  (ceil(b * world / B))
    last = -(-(b + 1) * world // B)     # first rank of the next batch
    group, pos = last - first, rank - first
    h0, h1 = split_even(H, group, pos)
    return Shard(b, b + 1, h0, h1)


def take_shard(x: torch.Tensor, s: Shard, head_dim: Optional[int] = 2) -> torch.Tensor:
    """Slice a (B, T, H, D) tensor (or a (B, ...) per-batch tensor when head_dim is None)."""
    x = x[s.b0:s.b1]
    if head_dim is not None:
        x = x.narrow(head_dim, s.h0, s.h1 - s.h0)
    return x


def gather_for_verification(local: torch.Tensor, B: int, H: int, group=None) -> Optional[torch.Tensor]:
    """Reassemble the full (B, T, H, D) tensor on rank 0 from every rank's shard.

    Verification only - never part of a timed region.  Works with any torch.distributed
    backend (gloo on CPU, nccl on GPUs).
    """
    import torch.distributed as dist

    world, rank = dist.get_world_size(group), dist.get_rank(group)
    T, D = local.shape[1], local.shape[3]
    full = torch.zeros(B, T, H, D, dtype=local.dtype, device=local.device)
    mine = plan_shard(B, H, world, rank)
    full[mine.b0:mine.b1, :, mine.h0:mine.h1] = local
    # disjoint supports: a sum is a gather
    work = full.float() if full.dtype in (torch.float16, torch.bfloat16) else full
    dist.reduce(work, dst=0, group=group)
    return work.to(local.dtype) if rank == 0 else None


def all_shards(B: int, H: int, world: int) -> List[Shard]:
    return [plan_shard(B, H, world, r) for r in range(world)]
