"""Multi-GPU partition of the attention work: one process per GPU, no collective on the data path.

Every (batch, kv-head group) unit is independent in the forward and in the backward (the GQA dK / dV reduction stays
inside a group, the K mean is per (batch, kv head)), so unit u = b * Hk + hk goes to rank u // (B * Hk / world) as a
contiguous range and each rank runs the single-GPU code on its units reshaped to a batch of groups (B' = units,
H' = H / Hk, Hk' = 1).  A unit's inputs, and therefore its output bits, do not depend on the number of ranks.
"""
from __future__ import annotations

import torch


def unit_range(B: int, Hk: int, world: int, rank: int) -> range:
    """Units [lo, hi) of `rank`; B * Hk must divide evenly (the benchmark's shapes do)."""
    units = B * Hk
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if units % world:
        raise ValueError(f"{units} (batch * kv heads) units do not divide over {world} ranks")
    per = units // world
    return range(rank * per, (rank + 1) * per)


def take_units(q, k, v, units: range):
    """q (B, N, H, D), k / v (B, N, Hk, D) -> the same tensors restricted to `units`, as a batch of groups:
    q' (U, N, H / Hk, D), k' / v' (U, N, 1, D)."""
    B, N, H, D = q.shape
    Hk = k.shape[2]
    rep = H // Hk
    idx = torch.as_tensor(list(units), device=q.device)
    qg = q.reshape(B, N, Hk, rep, D).permute(0, 2, 1, 3, 4).reshape(B * Hk, N, rep, D)
    kg = k.permute(0, 2, 1, 3).reshape(B * Hk, N, 1, D)
    vg = v.permute(0, 2, 1, 3).reshape(B * Hk, N, 1, D)
    return qg.index_select(0, idx), kg.index_select(0, idx), vg.index_select(0, idx)


def put_units(out_units, B: int, Hk: int):
    """Inverse of take_units for a full set of units: (B * Hk, N, h, D) -> (B, N, Hk * h, D)."""
    U, N, h, D = out_units.shape
    assert U == B * Hk
    return out_units.reshape(B, Hk, N, h, D).permute(0, 2, 1, 3, 4).reshape(B, N, Hk * h, D)


# ------------------------------------------------------------------------------------------------------ validation
_GOLD = -7046029254386353131          # 0x9E3779B97F4A7C15 as a signed 64-bit integer (odd)


def unit_hashes(*outs):
    """One 64-bit hash and one fp64 sum per unit over the bit patterns of `outs`, tensors whose leading dimension is
    the unit (for instance O, dQ, dK, dV of a rank's shard): returns (int64 (U,), float64 (U,)).  The hash is a sum
    modulo 2^64 of (bits + 1) * (2 * position + 1) * odd constant per tensor, mixed across tensors with another odd
    multiplier: it depends on every bit and on where it sits, not on the device, the rank or the number of units in the
    shard.  Runs on the tensors' device without a host round trip."""
    if not outs:
        raise ValueError("unit_hashes needs at least one tensor")
    U = outs[0].shape[0]
    h = torch.zeros(U, dtype=torch.int64, device=outs[0].device)
    s = torch.zeros(U, dtype=torch.float64, device=outs[0].device)
    for t in outs:
        if t.shape[0] != U:
            raise ValueError("every tensor must have the unit as its leading dimension")
        flat = t.contiguous().reshape(U, -1)
        if flat.dtype in (torch.bfloat16, torch.float16):
            bits = flat.view(torch.int16).to(torch.int64) & 0xFFFF
        elif flat.dtype == torch.float32:
            bits = flat.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
        else:
            bits = flat.to(torch.int64)
        pos = torch.arange(flat.shape[1], device=flat.device, dtype=torch.int64) * 2 + 1
        part = ((bits + 1) * pos * _GOLD).sum(dim=1)          # int64 arithmetic wraps: sums modulo 2^64
        h = (h * 1000003) ^ part
        s = s + flat.to(torch.float64).sum(dim=1)
    return h, s


def gather_unit_hashes(h: torch.Tensor, s: torch.Tensor, world: int):
    """all_gather of the ranks' (hash, sum) vectors in rank order = unit order (every rank holds the same number of
    units).  The only collective of the multi-GPU path, and it runs after the timed region: validation, not data."""
    import torch.distributed as dist
    if world == 1:
        return h, s
    hs = [torch.empty_like(h) for _ in range(world)]
    ss = [torch.empty_like(s) for _ in range(world)]
    dist.all_gather(hs, h)
    dist.all_gather(ss, s)
    return torch.cat(hs), torch.cat(ss)


def make_unit_inputs(units, N: int, rep: int, D: int, seed: int, device, unit_rms: bool = False):
    """Synthetic inputs of `units` as a batch of groups: q, dO (U, N, rep, D), k, v (U, N, 1, D) bf16, unit u drawn
    from torch.Generator(device).manual_seed(seed + u) in the order q, k, v, dO, so that a unit's inputs (and therefore
    its output bits) do not depend on which rank owns it or on how many ranks there are.  unit_rms=True divides every
    q and k row by its RMS over D (rows of unit RMS, like a qk-norm)."""
    units = list(units)
    q = torch.empty(len(units), N, rep, D, device=device, dtype=torch.bfloat16)
    do = torch.empty_like(q)
    k = torch.empty(len(units), N, 1, D, device=device, dtype=torch.bfloat16)
    v = torch.empty_like(k)
    for i, u in enumerate(units):
        g = torch.Generator(device=device).manual_seed(seed + u)
        for dst, h, norm in ((q, rep, unit_rms), (k, 1, unit_rms), (v, 1, False), (do, rep, False)):
            x = torch.randn(N, h, D, generator=g, device=device, dtype=torch.float32)
            if norm:
                x = x * torch.rsqrt(x.square().mean(dim=-1, keepdim=True))
            dst[i] = x.to(torch.bfloat16)
    return q, k, v, do
