"""The numerics arms besides the contract: "sm100-mx-ds32" (dS scaled per 32 queries x 32 keys; "sm100-mx-d256-ds32" at
head_dim 256) and "sm100-mx-nonorm" (matched delta = sum P dP without the division), both presets of the reference's
emulation (delta_matching/reference.py:620, 625, 630).  Same gates as the contract's tests: distance to the oracle run
with the same arm on the kernel's own K mean, error against exact attention at most 1 % above the emulation's, the
committed golden vectors of the reference's emulation, and agreement of the two backward forms."""
import pytest
import torch

from .conftest import load_golden
from .helpers import record, run_api, run_ops

pytestmark = pytest.mark.gpu

NAMES = ("O", "dQ", "dK", "dV")
EMU_DIST = {"O": 3e-4, "dQ": 5e-3, "dK": 5e-3, "dV": 5e-3}
TOL_EXACT = {"O": 0.08, "dQ": 0.12, "dK": 0.12, "dV": 0.08}
CASES = [  # B, N, H, Hk, D, causal, mode, numerics
    (1, 256, 2, 2, 128, True, "matched", "sm100-mx-ds32"),
    (2, 1152, 4, 2, 128, True, "matched", "sm100-mx-ds32"),
    (1, 1408, 4, 4, 128, False, "stale", "sm100-mx-ds32"),
    (1, 2048, 8, 2, 128, True, "stale", "sm100-mx-ds32"),
    (1, 384, 4, 2, 256, True, "matched", "sm100-mx-d256-ds32"),
    (1, 1024, 2, 1, 256, True, "stale", "sm100-mx-d256-ds32"),
    (2, 1152, 4, 2, 128, True, "matched", "sm100-mx-nonorm"),
    (1, 384, 4, 2, 256, True, "matched", "sm100-mx-nonorm"),
]


@pytest.mark.parametrize("B,N,H,Hk,D,causal,mode,numerics", CASES)
def test_arm_matches_its_emulation(B, N, H, Hk, D, causal, mode, numerics, oracle):
    q, k, v, do = oracle.make_inputs(B, N, H, Hk, D, seed=11, device="cuda")
    got = run_ops(q, k, v, do, causal, mode, numerics=numerics)
    em = oracle.dm_oracle(q, k, v, do, causal, mode, k_mean=got["kmean"], o_for_stale=got["O"] if mode == "stale" else None,
                          numerics=numerics)
    ex = oracle.attention_exact(q, k, v, do, causal)
    case = f"{numerics}_{B}_{N}_{H}_{Hk}_{D}_{int(causal)}_{mode}"
    assert oracle.rel_l2(got["delta"], em["delta"]) <= 1e-4, "delta"
    for nm in NAMES:
        e_c, e_e = oracle.rel_l2(got[nm], ex[nm]), oracle.rel_l2(em[nm], ex[nm])
        dist = oracle.rel_l2(got[nm], em[nm])
        record("arms", case, nm, dist)
        assert e_c <= 1.01 * e_e + 1e-5, f"{nm}: err vs exact {e_c:.3e}, emulation {e_e:.3e}"
        assert dist <= EMU_DIST[nm], f"{nm}: dist to emulation {dist:.3e}"
        assert e_c < TOL_EXACT[nm], nm


@pytest.mark.parametrize("B,N,H,Hk,D,causal,mode,numerics", CASES[:2] + CASES[4:5])
def test_arm_differs_from_the_contract(B, N, H, Hk, D, causal, mode, numerics, oracle):
    """The flag reaches the kernels: dQ / dK of the ds32 arm are not the contract's (dV and O do not depend on dS)."""
    q, k, v, do = oracle.make_inputs(B, N, H, Hk, D, seed=11, device="cuda")
    a = run_ops(q, k, v, do, causal, mode, numerics=numerics)
    b = run_ops(q, k, v, do, causal, mode)
    assert torch.equal(a["O"], b["O"]) and torch.equal(a["dV"], b["dV"]) and torch.equal(a["delta"], b["delta"])
    assert not torch.equal(a["dQ"], b["dQ"]) and not torch.equal(a["dK"], b["dK"])


@pytest.mark.parametrize("case", ["c1_matched_ds32", "c1_stale_ds32", "c1_matched_nonorm", "hd256_matched_ds32"])
def test_arm_golden_vectors(case, oracle):
    """Against the committed outputs of the reference's own emulation for the arm (generated with its default K mean)."""
    g = load_golden(case)
    d = g["dims"]
    q, k, v, do = (g[n].cuda() for n in ("q", "k", "v", "do"))
    got = run_ops(q, k, v, do, d["causal"], g["mode"], numerics=g["preset"])
    assert oracle.rel_l2(got["O"].cpu(), g["O"]) <= 2e-3
    assert oracle.rel_l2(got["delta"].cpu(), g["delta"]) <= 2e-3
    for nm in ("dQ", "dK") + (("dV",) if "dV" in g else ()):
        dist = oracle.rel_l2(got[nm].cpu(), g[nm])
        record("golden", case, nm, dist)
        assert dist <= 1e-2, (nm, dist)


@pytest.mark.parametrize("D,N", [(128, 1024), (256, 512)])
def test_ds32_both_backward_forms_agree_bitwise(D, N, oracle):
    """The two-pass backward (dS tiles stored, dQ streams them) and the one that recomputes give the same bits."""
    name = "sm100-mx-ds32" if D == 128 else "sm100-mx-d256-ds32"
    q, k, v, do = oracle.make_inputs(1, N, 4, 2, D, seed=12, device="cuda")
    a = run_ops(q, k, v, do, True, "matched", numerics=name, two_pass=True)
    b = run_ops(q, k, v, do, True, "matched", numerics=name, two_pass=False)
    for nm in ("dQ", "dK", "dV"):
        assert torch.equal(a[nm], b[nm]), nm


def test_nonorm_delta_is_the_numerator(oracle):
    """delta(nonorm) = delta(contract) * sum_j P_ij: the same pass 0 with the division left out."""
    from delta_matching_b200 import ops
    q, k, v, do = oracle.make_inputs(1, 1024, 4, 2, 128, seed=13, device="cuda")
    a = run_ops(q, k, v, do, True, "matched")
    n = ops.delta_fp8(a["q8"], a["k8"], a["v8"], a["do8"], a["qs"], a["ks"], a["vs"], a["dos"], a["LSE"], True, norm=False)
    em = oracle.dm_oracle(q, k, v, do, True, "matched", k_mean=a["kmean"], numerics="sm100-mx-nonorm")
    assert oracle.rel_l2(n, em["delta"]) <= 1e-4
    # sum_j P_ij is 1 up to the forward's quantisation of l, so the two deltas are close but not equal
    assert not torch.equal(n, a["delta"])
    assert oracle.rel_l2(n, a["delta"]) <= 2e-2


def test_api_numerics_argument(oracle):
    import delta_matching_b200 as dm
    q, k, v, do = oracle.make_inputs(1, 512, 4, 2, 128, seed=14, device="cuda")
    a = run_api(q, k, v, do, True, "matched", numerics="sm100-mx-ds32")
    b = run_ops(q, k, v, do, True, "matched", numerics="sm100-mx-ds32")
    for nm in NAMES:
        assert torch.equal(a[nm], b[nm]), nm
    with pytest.raises(ValueError, match="numerics must be one of"):
        dm.dm_attn_func(q, k, v, causal=True, numerics="sm90")
    with pytest.raises(ValueError, match="head_dim-256 name"):
        dm.dm_attn_func(q, k, v, causal=True, numerics="sm100-mx-d256-ds32")
    assert set(dm.kernel_version()["numerics_arms"]) == set(dm.NUMERICS_ARMS)
