"""The (batch, kv-group) partition used on several GPUs: pure index logic, plus a two-process gloo run on CPU showing
that the ranks' unit ranges tile the work, that units survive the round trip, and that the per-rank checksums a rank
gathers for validation arrive in rank order."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from delta_matching_b200 import shard


def test_unit_ranges_tile_the_work():
    for B, Hk, world in ((8, 8, 1), (8, 8, 2), (8, 8, 4), (8, 8, 8), (4, 8, 8), (2, 2, 4)):
        seen = []
        for r in range(world):
            seen += list(shard.unit_range(B, Hk, world, r))
        assert seen == list(range(B * Hk))
    with pytest.raises(ValueError):
        shard.unit_range(3, 1, 2, 0)
    with pytest.raises(ValueError):
        shard.unit_range(4, 2, 2, 2)


def test_take_put_roundtrip():
    B, N, H, Hk, D = 2, 8, 6, 2, 4
    q = torch.arange(B * N * H * D, dtype=torch.float32).reshape(B, N, H, D)
    k = torch.arange(B * N * Hk * D, dtype=torch.float32).reshape(B, N, Hk, D) + 0.5
    qg, kg, vg = shard.take_units(q, k, k, shard.unit_range(B, Hk, 1, 0))
    assert qg.shape == (B * Hk, N, H // Hk, D) and kg.shape == (B * Hk, N, 1, D)
    # unit u = b * Hk + hk holds query heads hk * rep .. of batch b
    assert torch.equal(qg[3], q[1, :, 3:6])
    assert torch.equal(kg[3, :, 0], k[1, :, 1])
    assert torch.equal(shard.put_units(qg, B, Hk), q)
    assert torch.equal(shard.put_units(kg, B, Hk), k)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    B, N, H, Hk, D = 2, 4, 4, 2, 2
    g = torch.Generator().manual_seed(0)
    q = torch.randn(B, N, H, D, generator=g)
    k = torch.randn(B, N, Hk, D, generator=g)
    units = shard.unit_range(B, Hk, world, rank)
    qg, kg, _ = shard.take_units(q, k, k, units)
    # stand-in for the per-shard work: something that depends only on the unit's own data
    local = (qg.sum(dim=(1, 2, 3)) + 2 * kg.sum(dim=(1, 2, 3)))
    gathered = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(gathered, local)
    if rank == 0:
        torch.save(torch.cat(gathered), out)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo(tmp_path):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    out = str(tmp_path / "g.pt")
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    got = torch.load(out)
    B, N, H, Hk, D = 2, 4, 4, 2, 2
    g = torch.Generator().manual_seed(0)
    q = torch.randn(B, N, H, D, generator=g)
    k = torch.randn(B, N, Hk, D, generator=g)
    qg, kg, _ = shard.take_units(q, k, k, range(B * Hk))
    want = qg.sum(dim=(1, 2, 3)) + 2 * kg.sum(dim=(1, 2, 3))
    assert torch.allclose(got, want)
