"""The CPU oracle against the golden vectors produced by the reference's own emulation (tests/golden/make_golden.py).
Producer codes and scales must be bit-identical; the floating-point outputs must agree to fp32 round-off."""
import pytest
import torch

from .conftest import GOLDEN_CASES, load_golden


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_inputs_reproducible(case, oracle):
    """The seeded input generator regenerates the stored inputs bit for bit."""
    g = load_golden(case)
    d = g["dims"]
    q, k, v, do = oracle.make_inputs(d["B"], d["N"], d["H"], d["Hk"], d["D"], seed=d["seed"])
    for name, t in (("q", q), ("k", k), ("v", v), ("do", do)):
        assert torch.equal(t.view(torch.int16), g[name].view(torch.int16)), name


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_producers_bit_exact(case, oracle):
    g = load_golden(case)
    p = oracle.producers(g["q"], g["k"], g["v"], g["do"])
    assert torch.equal(p["kmean"], g["kmean"])
    for nm in ("q", "k", "v", "do"):
        codes = p[nm + "_codes"].to(torch.float8_e4m3fn).view(torch.uint8)
        assert torch.equal(codes, g[nm + "_codes"]), nm
        assert torch.equal(p[nm + "_scales"], g[nm + "_scales"]), nm


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_engine_matches_reference(case, oracle):
    g = load_golden(case)
    d = g["dims"]
    r = oracle.dm_oracle(g["q"], g["k"], g["v"], g["do"], d["causal"], g["mode"], aux=True, numerics=g["preset"])
    assert torch.equal(r["O"].view(torch.int16), g["O"].view(torch.int16))
    tol = 2e-6
    assert oracle.rel_l2(r["LSE"], g["LSE"]) <= tol
    assert oracle.rel_l2(r["delta"], g["delta"]) <= 1e-5
    for nm in ("dQ", "dK") + (("dV",) if "dV" in g else ()):
        assert oracle.rel_l2(r[nm], g[nm]) <= tol, nm
    assert oracle.rel_l2(r["sum_absPdP"], g["sum_absPdP"]) <= 1e-6
    if g["mode"] == "matched":
        live = g["sum_absPdP"] > 0
        resid = (r["rowsum_dS"].abs() / r["sum_absPdP"].clamp_min(1e-300))[live]
        assert resid.max().item() <= 1e-5 and resid.mean().item() <= 2e-7


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_reference_error_bounds(case, oracle):
    """The emulation itself sits inside the reference's accuracy gates against exact attention (O, dV < 0.08;
    dQ, dK < 0.12: tests/test_dm_attn.py:15 of the reference), and the oracle reproduces the stored distances."""
    g = load_golden(case)
    d = g["dims"]
    r = oracle.dm_oracle(g["q"], g["k"], g["v"], g["do"], d["causal"], g["mode"], numerics=g["preset"])
    ex = oracle.attention_exact(g["q"], g["k"], g["v"], g["do"], d["causal"])
    for i, (nm, bound) in enumerate((("O", 0.08), ("dQ", 0.12), ("dK", 0.12), ("dV", 0.08))):
        e = oracle.rel_l2(r[nm], ex[nm])
        assert e < bound, (nm, e)
        assert abs(e - float(g["err_vs_fp32"][i])) < 1e-4, (nm, e, float(g["err_vs_fp32"][i]))
