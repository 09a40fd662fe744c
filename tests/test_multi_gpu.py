"""The (batch, kv-group) partition on real GPUs: two ranks (one process per GPU, NCCL) each run their units through
dm_attn_func, the per-unit hashes of (O, dQ, dK, dV) are gathered with all_gather, and rank 0 compares them with the
hashes of the unsharded run on one GPU: the same unit gives the same bits whatever the number of ranks.  No collective
touches the data path.  Skipped with fewer than two GPUs."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
B, HK, REP, N, D, SEED = 2, 2, 4, 1024, 128, 77


def _run_units(units, dev):
    import delta_matching_b200 as dm
    from delta_matching_b200 import ops, shard
    q, k, v, do = shard.make_unit_inputs(units, N, REP, D, SEED, dev, unit_rms=True)
    leaves = [t.requires_grad_() for t in (q, k, v)]
    o = dm.dm_attn_func(*leaves, causal=True, mode="matched")
    o.backward(do)
    torch.cuda.synchronize(dev)
    ops.check_status(dev)
    return shard.unit_hashes(o.detach(), leaves[0].grad, leaves[1].grad, leaves[2].grad)


def _worker(rank, world, port, out):
    from delta_matching_b200 import shard
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    h, s = _run_units(shard.unit_range(B, HK, world, rank), dev)
    H, S = shard.gather_unit_hashes(h, s, world)
    if rank == 0:
        h1, s1 = _run_units(range(B * HK), dev)
        torch.save({"gathered": H.cpu(), "single": h1.cpu(), "sums": S.cpu(), "sums_single": s1.cpu()}, out)
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_give_the_bits_of_one(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    sock = socket.socket()
    sock.bind(("127.0.0.1", 0))
    port = sock.getsockname()[1]
    sock.close()
    out = str(tmp_path / "h.pt")
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    r = torch.load(out)
    assert torch.equal(r["gathered"], r["single"])
    assert torch.equal(r["sums"], r["sums_single"]) and torch.isfinite(r["sums"]).all()
