"""The two-pass backward (dK / dV kernel stores the dS codes, dQ streams them) against the backward that recomputes:
bit-identical outputs, also when the workspace bound splits the call over batches or kv-head groups."""
import pytest
import torch

from .helpers import run_ops

pytestmark = pytest.mark.gpu
NAMES = ("dQ", "dK", "dV")


def _bwd(oracle, monkeypatch, cap_mb, B, N, H, Hk, causal, mode, seed, D=128):
    q, k, v, do = oracle.make_inputs(B, N, H, Hk, D, seed=seed, device="cuda")
    if cap_mb is None:
        monkeypatch.delenv("DM_BWD_WORKSPACE_MB", raising=False)
    else:
        monkeypatch.setenv("DM_BWD_WORKSPACE_MB", str(cap_mb))
    return run_ops(q, k, v, do, causal, mode)


@pytest.mark.parametrize("B,N,H,Hk,causal,mode", [(2, 1024, 8, 2, True, "matched"), (1, 512, 4, 4, False, "stale"),
                                                  (3, 768, 6, 3, True, "stale")])
def test_two_pass_equals_recompute(B, N, H, Hk, causal, mode, oracle, monkeypatch):
    ref = _bwd(oracle, monkeypatch, 0, B, N, H, Hk, causal, mode, seed=31)            # 0: recomputing kernel
    got = _bwd(oracle, monkeypatch, None, B, N, H, Hk, causal, mode, seed=31)         # default: two-pass
    for nm in NAMES:
        assert torch.equal(got[nm], ref[nm]), nm


@pytest.mark.parametrize("B,N,H,Hk,causal,mode", [(1, 512, 4, 2, True, "matched"), (2, 384, 2, 2, False, "stale")])
def test_two_pass_equals_recompute_hd256(B, N, H, Hk, causal, mode, oracle, monkeypatch):
    ref = _bwd(oracle, monkeypatch, 0, B, N, H, Hk, causal, mode, seed=34, D=256)
    got = _bwd(oracle, monkeypatch, None, B, N, H, Hk, causal, mode, seed=34, D=256)
    for nm in NAMES:
        assert torch.equal(got[nm], ref[nm]), nm


@pytest.mark.parametrize("cap_mb", [1, 3, 7])
def test_workspace_bound_splits_the_call(cap_mb, oracle, monkeypatch):
    """N = 1024: one kv group of 2 query heads needs 2 x 64 tiles x 16 KiB = 2 MiB; caps of 1 / 3 / 7 MiB give the
    recomputing kernel, one group per call, and whole batches of two groups."""
    B, N, H, Hk = 3, 1024, 4, 2
    ref = _bwd(oracle, monkeypatch, 0, B, N, H, Hk, True, "matched", seed=32)
    got = _bwd(oracle, monkeypatch, cap_mb, B, N, H, Hk, True, "matched", seed=32)
    for nm in NAMES:
        assert torch.equal(got[nm], ref[nm]), nm


def test_parts_share_a_workspace(oracle):
    from delta_matching_b200 import ops
    B, N, H, Hk = 1, 512, 4, 2
    q, k, v, do = oracle.make_inputs(B, N, H, Hk, 128, seed=33, device="cuda")
    r = run_ops(q, k, v, do, True, "matched")
    ws = torch.empty(ops.bwd_workspace_bytes(B, N, H, 128), device="cuda", dtype=torch.uint8)
    args = (r["q8"], r["k8"], r["v8"], r["do8"], r["qs"], r["ks"], r["vs"], r["dos"], r["LSE"], r["delta"], True)
    _, dk, dv = ops.bwd_fp8(*args, parts=1, workspace=ws)
    dq, _, _ = ops.bwd_fp8(*args, parts=2, workspace=ws)
    torch.cuda.synchronize()
    assert torch.equal(dq, r["dQ"]) and torch.equal(dk, r["dK"]) and torch.equal(dv, r["dV"])
    with pytest.raises(RuntimeError):
        ops.bwd_fp8(*args, workspace=ws[:1000])


def test_workspace_bytes():
    from delta_matching_b200 import ops
    assert ops.bwd_workspace_bytes(4, 4096, 32, 128) == 4 * 32 * 32 * 32 * (16384 + 16)
    assert ops.bwd_workspace_bytes(2, 1024, 4, 256) == 2 * 4 * 8 * 8 * (16384 + 16)      # the tile does not depend on head_dim
    assert ops.bwd_workspace_bytes(2, 1000, 4, 128) == 0
