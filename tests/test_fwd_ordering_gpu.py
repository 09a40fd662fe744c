"""The forward issues S = Q K^T of key tile i + 1 into the TMEM columns from which the block-scaled PV chain of tile i
reads its scale-factor words.  The production kernel waits for the PV chain first (a commit and an mbarrier wait, as
the reference's kernel does: delta_matching/sm100/dm_fwd_sm100.py:636-645); the hook dm_dbg_fwd_unordered leaves the
wait out and relies on MMAs executing in issue order.  Both must give the same bits, every time: on the headline
shape and on the logit-range case whose running maximum moves by hundreds of binades between key tiles."""
import pytest
import torch

pytestmark = pytest.mark.gpu
REPEATS = 20


def _codes(oracle, B, N, H, Hk, D, seed, qk_scale=1.0):
    from delta_matching_b200 import ops
    q, k, v, _ = oracle.make_inputs(B, N, H, Hk, D, seed=seed, device="cuda", qk_scale=qk_scale)
    return ops.quant_qkv(*(t.transpose(1, 2) for t in (q, k, v)))[:6]


@pytest.mark.parametrize("B,N,H,Hk,D,causal,s", [(4, 4096, 32, 8, 128, True, 1.0), (8, 2048, 16, 16, 128, False, 30.0),
                                                 (1, 2048, 4, 4, 256, True, 1.0), (2, 1024, 8, 8, 256, True, 1.0)])
def test_ordered_and_unordered_forward_agree_bitwise(B, N, H, Hk, D, causal, s, oracle):
    from delta_matching_b200 import ops
    q8, qs, k8, ks, v8, vs = _codes(oracle, B, N, H, Hk, D, seed=51, qk_scale=s)
    o0, l0 = ops.fwd_fp8(q8, k8, v8, qs, ks, vs, causal)
    torch.cuda.synchronize()
    assert torch.isfinite(o0.float()).all() and torch.isfinite(l0).all()
    for i in range(REPEATS):
        o1, l1 = ops.fwd_fp8(q8, k8, v8, qs, ks, vs, causal)
        o2, l2 = ops.fwd_fp8(q8, k8, v8, qs, ks, vs, causal, unordered=True)
        torch.cuda.synchronize()
        assert torch.equal(o1, o0) and torch.equal(l1, l0), f"ordered, repeat {i}"
        assert torch.equal(o2, o0) and torch.equal(l2, l0), f"unordered, repeat {i}"
    ops.check_status("cuda")
