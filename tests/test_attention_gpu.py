"""The CUDA forward / matched-delta / backward against the oracle (the reference's emulation restated) and against exact
attention, through the public API.  Gates are the reference's own for its Blackwell kernels (tests/test_sm100.py:61,
79-129 of the reference): distance to the emulation run on the kernel's own K mean, error against exact attention at
most 1% above the emulation's, the matched-mode identity measured inside the backward, bitwise determinism."""
import pytest
import torch

from .conftest import load_golden
from .helpers import record, run_api, run_ops

pytestmark = pytest.mark.gpu

D = 128
NAMES = ("O", "dQ", "dK", "dV")
EMU_DIST = {"O": 3e-4, "dQ": 5e-3, "dK": 5e-3, "dV": 5e-3}          # rel L2(kernel, emulation)
TOL_EXACT = {"O": 0.08, "dQ": 0.12, "dK": 0.12, "dV": 0.08}        # rel L2 against fp32 attention
# B, N, H, Hk, causal: MHA / GQA / MQA, one tile, odd numbers of 128-row tiles
SHAPES = [(1, 128, 2, 2, True), (2, 256, 4, 1, True), (1, 384, 4, 4, False), (1, 1152, 4, 4, True),
          (2, 1408, 8, 2, False), (1, 2048, 8, 2, True)]


def _kmean(k):
    from delta_matching_b200 import ops
    return ops.kmean(k.transpose(1, 2))


@pytest.mark.parametrize("mode", ["matched", "stale"])
@pytest.mark.parametrize("B,N,H,Hk,causal", SHAPES)
def test_matches_emulation(B, N, H, Hk, causal, mode, oracle):
    if mode == "matched" and not causal:
        pytest.skip("matched needs causal")
    q, k, v, do = oracle.make_inputs(B, N, H, Hk, D, seed=0, device="cuda")
    got = run_ops(q, k, v, do, causal, mode)
    for nm in NAMES:
        assert torch.isfinite(got[nm].float()).all(), nm
    em = oracle.dm_oracle(q, k, v, do, causal, mode, k_mean=got["kmean"], o_for_stale=got["O"] if mode == "stale" else None)
    ex = oracle.attention_exact(q, k, v, do, causal)
    case = f"{B}_{N}_{H}_{Hk}_{int(causal)}_{mode}"
    record("emu", case, "LSE", oracle.rel_l2(got["LSE"], em["LSE"]))
    record("emu", case, "delta", oracle.rel_l2(got["delta"], em["delta"]))
    fails = []
    for nm in NAMES:
        e_c, e_e = oracle.rel_l2(got[nm], ex[nm]), oracle.rel_l2(em[nm], ex[nm])
        dist = oracle.rel_l2(got[nm], em[nm])
        record("emu", case, nm, dist)
        record("exact", case, nm, e_c)
        if not e_c <= 1.01 * e_e + 1e-5:
            fails.append(f"{nm}: err vs exact {e_c:.3e}, emulation {e_e:.3e}")
        if not dist <= EMU_DIST[nm]:
            fails.append(f"{nm}: dist to emulation {dist:.3e} > {EMU_DIST[nm]:.1e}")
        if not e_c < TOL_EXACT[nm]:
            fails.append(f"{nm}: err vs exact {e_c:.3e} >= {TOL_EXACT[nm]}")
    assert (got["LSE"] - em["LSE"]).abs().max().item() <= 1e-4 + 1e-5 * em["LSE"].abs().max().item(), "LSE"
    assert not fails, "; ".join(fails)


@pytest.mark.parametrize("mode", ["matched", "stale"])
@pytest.mark.parametrize("B,N,H,Hk,causal", [(1, 128, 2, 2, True), (1, 384, 4, 2, True), (1, 256, 2, 1, False),
                                             (1, 1024, 2, 1, True)])
def test_matches_emulation_hd256(B, N, H, Hk, causal, mode, oracle):
    """head_dim 256 (the reference's gates for its hd256 kernels: tests/test_sm100_hd256.py:97, 122-147)."""
    if mode == "matched" and not causal:
        pytest.skip("matched needs causal")
    q, k, v, do = oracle.make_inputs(B, N, H, Hk, 256, seed=7, device="cuda")
    got = run_ops(q, k, v, do, causal, mode)
    em = oracle.dm_oracle(q, k, v, do, causal, mode, k_mean=got["kmean"], o_for_stale=got["O"] if mode == "stale" else None)
    ex = oracle.attention_exact(q, k, v, do, causal)
    case = f"hd256_{B}_{N}_{H}_{Hk}_{int(causal)}_{mode}"
    assert (got["LSE"] - em["LSE"]).abs().max().item() <= 1e-4 + 1e-5 * em["LSE"].abs().max().item(), "LSE"
    for nm in NAMES:
        e_c, e_e = oracle.rel_l2(got[nm], ex[nm]), oracle.rel_l2(em[nm], ex[nm])
        dist = oracle.rel_l2(got[nm], em[nm])
        record("emu", case, nm, dist)
        assert e_c <= 1.01 * e_e + 1e-5, f"{nm}: err vs exact {e_c:.3e}, emulation {e_e:.3e}"
        assert dist <= EMU_DIST[nm], f"{nm}: dist to emulation {dist:.3e}"
        assert e_c < TOL_EXACT[nm], nm


@pytest.mark.parametrize("case", ["c1_matched", "c1_stale", "gqa_noncausal_stale", "hd256_matched"])
def test_golden_vectors(case, oracle):
    """Against the committed outputs of the reference's own emulation (generated with its default K mean)."""
    g = load_golden(case)
    d = g["dims"]
    q, k, v, do = (g[n].cuda() for n in ("q", "k", "v", "do"))
    got = run_ops(q, k, v, do, d["causal"], g["mode"])
    assert oracle.rel_l2(got["O"].cpu(), g["O"]) <= 2e-3
    assert (got["LSE"].cpu() - g["LSE"]).abs().max().item() <= 2e-4
    for nm in ("dQ", "dK") + (("dV",) if "dV" in g else ()):
        dist = oracle.rel_l2(got[nm].cpu(), g[nm])
        record("golden", case, nm, dist)
        assert dist <= 1e-2, (nm, dist)


@pytest.mark.parametrize("B,N,H,Hk,causal", [(1, 1024, 4, 4, True), (1, 2048, 8, 2, True)])
def test_identity_in_kernel(B, N, H, Hk, causal, oracle):
    """Matched mode: per-row |sum_j dS_ij| / sum_j |P dP|, accumulated in the backward before dS is quantised, is at
    fp32 round-off (reference gate: max <= 1e-5, mean <= 2e-7)."""
    import delta_matching_b200 as dm
    q, k, v, do = oracle.make_inputs(B, N, H, Hk, D, seed=1, device="cuda")
    d = dm.dm_attn_debug(q, k, v, do, causal=causal, mode="matched", identity=True)
    torch.cuda.synchronize()
    live = d["sum_abs_PdP"] > 0
    r = (d["rowsum_dS"].double().abs() / d["sum_abs_PdP"].double().clamp_min(1e-300))[live]
    record("identity", f"{B}_{N}_{H}_{Hk}", "max", r.max().item())
    record("identity", f"{B}_{N}_{H}_{Hk}", "mean", r.mean().item())
    assert r.max().item() <= 1e-5 and r.mean().item() <= 2e-7, (r.max().item(), r.mean().item())
    assert torch.isfinite(d["delta"]).all() and torch.isfinite(d["lse"]).all()
    # the stale delta breaks the identity by orders of magnitude on the same inputs
    s = dm.dm_attn_debug(q, k, v, do, causal=causal, mode="stale", identity=True)
    rs = (s["rowsum_dS"].double().abs() / s["sum_abs_PdP"].double().clamp_min(1e-300))[live]
    assert rs.mean().item() > 100 * r.mean().item()


@pytest.mark.parametrize("mode", ["matched", "stale"])
def test_deterministic_and_strided(mode, oracle):
    """Repeat calls and q / k / v given as strided views of one packed tensor give bitwise equal outputs."""
    B, N, H, Hk = 1, 2048, 8, 2
    q, k, v, do = oracle.make_inputs(B, N, H, Hk, D, seed=2, device="cuda")
    a = run_api(q, k, v, do, True, mode)
    b = run_api(q, k, v, do, True, mode)
    qkv = torch.cat([q, k, v], dim=2)
    s = run_api(qkv[:, :, :H], qkv[:, :, H:H + Hk], qkv[:, :, H + Hk:], do, True, mode)
    for nm in NAMES:
        assert torch.equal(a[nm], b[nm]), f"repeat {nm}"
        assert torch.equal(a[nm], s[nm]), f"strided {nm}"


def test_matched_and_stale_share_forward(oracle):
    """The forward does not depend on the mode; dV = P^T dO does not use delta, so it is equal too."""
    q, k, v, do = oracle.make_inputs(1, 1024, 4, 4, D, seed=3, device="cuda")
    m, s = run_api(q, k, v, do, True, "matched"), run_api(q, k, v, do, True, "stale")
    assert torch.equal(m["O"], s["O"]) and torch.equal(m["dV"], s["dV"])
    assert not torch.equal(m["dQ"], s["dQ"]) and not torch.equal(m["dK"], s["dK"])


def test_all_zero_inputs(oracle):
    """All-zero q, k, v: O, dQ, dK exactly 0; dV is the uniform-causal average of dO (reference tests/test_api.py:276-294)."""
    B, N, H = 1, 256, 2
    z = torch.zeros(B, N, H, D, dtype=torch.bfloat16, device="cuda")
    do = oracle.make_inputs(B, N, H, H, D, seed=4, device="cuda")[3]
    got = run_api(z, z, z, do, True, "matched")
    for nm in ("O", "dQ", "dK"):
        assert got[nm].float().abs().max().item() == 0.0, nm
    w = torch.tril(torch.ones(N, N, device="cuda")) / torch.arange(1, N + 1, device="cuda")[:, None]
    want = torch.einsum("ij,bihd->bjhd", w, do.float())
    assert oracle.rel_l2(got["dV"], want) < 0.06


def test_expanded_grad_and_api_forms(oracle):
    """o.sum().backward() hands an expanded (stride-0) gradient; flash_attn_func and dm_attn_func_bhnd agree bitwise."""
    import delta_matching_b200 as dm
    q, k, v, _ = oracle.make_inputs(1, 256, 4, 2, D, seed=6, device="cuda")
    leaves = [t.detach().clone().requires_grad_() for t in (q, k, v)]
    dm.dm_attn_func(*leaves, causal=True, mode="matched").sum().backward()
    ones = torch.ones(1, 256, 4, D, dtype=torch.bfloat16, device="cuda")
    ref = run_api(q, k, v, ones, True, "matched")
    assert torch.equal(leaves[0].grad, ref["dQ"]) and torch.equal(leaves[2].grad, ref["dV"])
    o1 = dm.flash_attn_func(q, k, v, causal=True, mode="stale", deterministic=True)
    o2 = dm.dm_attn_func_bhnd(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), causal=True, delta_mode="stale")
    assert torch.equal(o1, o2) and o2.is_contiguous() and tuple(o2.shape) == (1, 256, 4, D)
