"""Shard planning for the multi-GPU launcher, and the verification gather over gloo (2 ranks)."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from triton_sigmoid_b200.launcher import all_shards, gather_for_verification, plan_shard, split_even, take_shard


def test_split_even_covers_range():
    for n in (0, 1, 7, 8, 33):
        for parts in (1, 2, 3, 8):
            pieces = [split_even(n, parts, i) for i in range(parts)]
            assert pieces[0][0] == 0 and pieces[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(pieces, pieces[1:]))
            assert max(b - a for a, b in pieces) - min(b - a for a, b in pieces) <= 1


@pytest.mark.parametrize("B,H,world", [(8, 32, 1), (8, 32, 2), (8, 32, 8), (4, 16, 8), (1, 16, 8), (3, 5, 8), (2, 3, 8)])
def test_every_unit_owned_exactly_once(B, H, world):
    owner = torch.zeros(B, H, dtype=torch.int32)
    for s in all_shards(B, H, world):
        owner[s.b0:s.b1, s.h0:s.h1] += 1
    assert (owner == 1).all()


def test_batch_sharding_is_preferred():
    s = plan_shard(8, 32, 4, 1)
    assert (s.b0, s.b1, s.h0, s.h1) == (2, 4, 0, 32)
    s = plan_shard(4, 16, 8, 3)  # two ranks per batch: heads split
    assert (s.b0, s.b1, s.h0, s.h1) == (1, 2, 8, 16)


def test_take_shard_slices_batch_and_heads():
    x = torch.arange(2 * 3 * 4 * 5).view(2, 3, 4, 5)
    s = plan_shard(2, 4, 4, 3)
    y = take_shard(x, s)
    assert torch.equal(y, x[1:2, :, 2:4])
    lens = torch.tensor([5, 7])
    assert torch.equal(take_shard(lens, s, head_dim=None), lens[1:2])


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, B, H):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = torch.arange(B * 6 * H * 4, dtype=torch.float32).view(B, 6, H, 4)
        mine = take_shard(full, plan_shard(B, H, world, rank)).contiguous()
        got = gather_for_verification(mine, B, H)
        if rank == 0:
            assert torch.equal(got, full)
        else:
            assert got is None
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("B,H", [(4, 2), (1, 4)])
def test_gather_for_verification_gloo_world2(B, H):
    mp.spawn(_worker, args=(2, _free_port(), B, H), nprocs=2, join=True)
