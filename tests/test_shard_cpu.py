"""Head sharding over ranks on the CPU (gloo, world size 2): slice arithmetic and the gather of output heads."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from unicaattention_b200 import shard


def test_head_slices_cover_the_heads():
    for heads, world in ((40, 1), (40, 2), (40, 8), (30, 8), (3, 4), (1, 2)):
        slices = [shard.head_slice(heads, r, world) for r in range(world)]
        assert slices[0].start == 0 and slices[-1].stop == heads
        assert all(a.stop == b.start for a, b in zip(slices, slices[1:]))
        sizes = [s.stop - s.start for s in slices]
        assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
    assert [s.stop - s.start for s in (shard.head_slice(30, r, 8) for r in range(8))] == [4, 4, 4, 4, 4, 4, 3, 3]
    with pytest.raises(ValueError):
        shard.head_slice(8, 2, 2)


def _worker(rank, world, port, heads, batch):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        whole = torch.arange(batch * heads * 5 * 128, dtype=torch.float32).reshape(batch, heads, 5, 128).bfloat16()
        mine = whole[:, shard.head_slice(heads, rank, world)].contiguous()
        out = torch.zeros_like(whole)
        shard.gather_heads(mine, out, heads, rank, world)
        assert torch.equal(out, whole), (rank, heads, batch)
        with pytest.raises(ValueError):
            shard.gather_heads(whole, out, heads, rank, world)  # not this rank's slice
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("heads,batch", [(4, 1), (5, 1), (4, 2)])
def test_gather_heads_two_ranks(heads, batch):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, heads, batch), nprocs=2, join=True)


def test_slice_heads_on_plain_tuples():
    from collections import namedtuple

    Pair = namedtuple("Pair", "codes sf")
    a, b = torch.zeros(1, 4, 3), torch.ones(1, 4, 2, 2)
    got = shard.slice_heads((a, Pair(a, b), (a, b), None, 512), slice(1, 3))
    assert got[0].shape == (1, 2, 3) and isinstance(got[1], Pair) and got[1].sf.shape == (1, 2, 2, 2)
    assert got[2][1].shape == (1, 2, 2, 2) and got[3] is None and got[4] == 512


def test_host_groups_are_small_at_both_ends():
    from unicaattention_b200.host import group_sizes

    for heads in (1, 3, 5, 7, 10, 20, 30, 40, 64):
        for largest in (None, 1, 4, 100):
            sizes = group_sizes(heads, largest)
            assert sum(sizes) == heads and all(s >= 1 for s in sizes)
            assert max(sizes) <= (largest or max(1, -(-heads // 8)))
            assert sizes[0] == 1 and sizes[-1] <= 2
            assert all(b - a <= 1 for a, b in zip(sizes, sizes[1:])), "a group's copy must fit behind the group before it"
    assert group_sizes(40) == [1, 2, 3, 4] + [5] * 5 + [3, 2]
    assert group_sizes(40, 4) == [1, 2, 3] + [4] * 8 + [2]
