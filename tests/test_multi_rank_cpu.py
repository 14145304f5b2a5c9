"""Host-side logic of the multi-GPU path, on CPU ranks (gloo, world size 2 and 3): the row / unit split and the
all-gather that assembles the shards. Compute is torch on CPU here -- the test is about the plumbing."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from emmyptx import shard


def test_split_range_covers_everything_once():
    for total, world, align in ((16384, 8, 128), (256, 8, 1), (100, 3, 1), (1000, 4, 128), (5, 8, 1), (0, 2, 1)):
        spans = [shard.split_range(total, world, r, align) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all(b % align == 0 for b, _ in spans if b < total)
    assert shard.even(16384, 8, 128) and not shard.even(1000, 4, 128)
    with pytest.raises(ValueError):
        shard.split_range(10, 2, 2)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, m: int, ragged: bool):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        a, b = torch.randn(m, 64, generator=g), torch.randn(64, 48, generator=g)
        lo, hi = shard.split_range(m, world, rank)
        local = torch.nn.functional.gelu(a[lo:hi] @ b, approximate="tanh")
        full = torch.zeros(m, 48)
        if ragged:
            shard.all_gather_ragged(full, local, m)
        else:
            shard.all_gather_rows(full, local)
        expect = torch.nn.functional.gelu(a @ b, approximate="tanh")
        assert torch.allclose(full, expect, atol=1e-5), f"rank {rank}"
        # attention units: independent (batch, head) slices gather the same way
        q = torch.randn(world * 2, 16, 8, generator=g)
        ulo, uhi = shard.split_range(world * 2, world, rank)
        o_local = torch.softmax(q[ulo:uhi] @ q[ulo:uhi].transpose(-1, -2), -1) @ q[ulo:uhi]
        o_full = shard.all_gather_rows(torch.zeros_like(q), o_local)
        assert torch.allclose(o_full, torch.softmax(q @ q.transpose(-1, -2), -1) @ q, atol=1e-5)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,m,ragged", [(2, 256, False), (3, 100, True)])
def test_row_shards_assemble_to_the_unsharded_result(world, m, ragged):
    mp.spawn(_worker, args=(world, _free_port(), m, ragged), nprocs=world, join=True)
