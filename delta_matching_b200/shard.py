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
