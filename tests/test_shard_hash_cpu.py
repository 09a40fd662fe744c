"""Validation side of the multi-GPU partition on CPU: the per-unit hash depends on every bit of a unit's outputs and on
nothing else (not on the shard a unit sits in), per-unit inputs depend only on (seed, unit), and a two-rank gloo run
gathers the ranks' hashes in unit order, equal to the hashes of the unsharded run."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from delta_matching_b200 import shard

B, HK, N, REP, D, SEED = 2, 2, 32, 2, 8, 11


def _work(q, k, v, do):
    """Stand-in for the attention step with the same independence structure: unit-local, deterministic."""
    o = (q.float() * k.float().mean(dim=1, keepdim=True)).to(torch.bfloat16)
    dq = (do.float() + v.float().sum(dim=1, keepdim=True)).to(torch.bfloat16)
    dk = (k.float() * q.float().sum(dim=2, keepdim=True).mean(dim=1, keepdim=True)).to(torch.bfloat16)
    return o, dq, dk


def test_inputs_depend_on_the_unit_only():
    full = shard.make_unit_inputs(range(B * HK), N, REP, D, SEED, "cpu", unit_rms=True)
    part = shard.make_unit_inputs(shard.unit_range(B, HK, 2, 1), N, REP, D, SEED, "cpu", unit_rms=True)
    for f, p_ in zip(full, part):
        assert torch.equal(f[2:], p_)
    q, k, v, do = full
    rms = q.float().square().mean(-1).sqrt()
    assert (rms - 1).abs().max().item() < 2e-2                 # rows at unit RMS (up to bf16 rounding)
    assert (v.float().square().mean(-1).sqrt() - 1).abs().max().item() > 2e-2      # v is left Gaussian


def test_hash_sees_every_bit_and_only_the_unit():
    q, k, v, do = shard.make_unit_inputs(range(4), N, REP, D, SEED, "cpu")
    h, s = shard.unit_hashes(*_work(q, k, v, do))
    h2, s2 = shard.unit_hashes(*_work(q[1:3], k[1:3], v[1:3], do[1:3]))
    assert torch.equal(h[1:3], h2) and torch.equal(s[1:3], s2)
    o, dq, dk = _work(q, k, v, do)
    o2 = o.clone()
    o2.view(torch.int16)[2, 5, 1, 3] ^= 1                       # one mantissa bit of one element of unit 2
    h3, _ = shard.unit_hashes(o2, dq, dk)
    assert h3[2] != h[2] and torch.equal(h3[[0, 1, 3]], h[[0, 1, 3]])
    # swapping two elements changes the hash too (position enters it)
    o4 = o.clone()
    o4[0, 0, 0, 0], o4[0, 0, 0, 1] = o[0, 0, 0, 1], o[0, 0, 0, 0]
    if not torch.equal(o4, o):
        assert shard.unit_hashes(o4, dq, dk)[0][0] != h[0]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    units = shard.unit_range(B, HK, world, rank)
    h, s = shard.unit_hashes(*_work(*shard.make_unit_inputs(units, N, REP, D, SEED, "cpu")))
    H, S = shard.gather_unit_hashes(h, s, world)
    if rank == 0:
        torch.save((H, S), out)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_hash_gather(tmp_path):
    sock = socket.socket()
    sock.bind(("127.0.0.1", 0))
    port = sock.getsockname()[1]
    sock.close()
    out = str(tmp_path / "h.pt")
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    H, S = torch.load(out)
    h1, s1 = shard.unit_hashes(*_work(*shard.make_unit_inputs(range(B * HK), N, REP, D, SEED, "cpu")))
    assert torch.equal(H, h1) and torch.equal(S, s1)           # same unit => same bits at every rank count
