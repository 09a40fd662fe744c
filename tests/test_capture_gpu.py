"""torch.compile and CUDA-graph capture around the public API, as the reference tests them (tests/test_api.py:304-332):
the compiled / replayed results equal the eager ones bit for bit, and the compiler traces through the API without a
graph break.  The backward is captured too (the reference captures the forward only)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _inputs(oracle, seed, B=1, N=1024, H=8, Hk=2, D=128):
    return oracle.make_inputs(B, N, H, Hk, D, seed=seed, device="cuda")


def test_cuda_graph_capture_of_the_forward(oracle):
    from delta_matching_b200 import dm_attn_func
    q, k, v, _ = _inputs(oracle, 41)
    dm_attn_func(q, k, v, causal=True)                 # warm-up outside the capture
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        o = dm_attn_func(q, k, v, causal=True)
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(o, dm_attn_func(q, k, v, causal=True))


@pytest.mark.parametrize("mode", ["matched", "stale"])
def test_cuda_graph_capture_of_forward_and_backward(mode, oracle):
    from delta_matching_b200 import dm_attn_func
    q, k, v, do = _inputs(oracle, 42)

    def step(leaves):
        o = dm_attn_func(*leaves, causal=True, mode=mode)
        grads = torch.autograd.grad(o, leaves, do)
        return (o.detach(),) + tuple(grads)

    leaves = [t.detach().clone().requires_grad_() for t in (q, k, v)]
    want = step(leaves)                                # also the warm-up
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        got = step(leaves)
    for _ in range(2):
        g.replay()
    torch.cuda.synchronize()
    for a, b in zip(got, want):
        assert torch.equal(a, b)


def test_torch_compile_matches_eager(oracle):
    from delta_matching_b200 import dm_attn_func
    q, k, v, go = _inputs(oracle, 43)

    def f(q, k, v):
        return dm_attn_func(q * 1.0, k, v, causal=True, mode="matched")
    qa, ka, va = (x.detach().clone().requires_grad_(True) for x in (q, k, v))
    qb, kb, vb = (x.detach().clone().requires_grad_(True) for x in (q, k, v))
    try:
        compiled = torch.compile(f)
        oa = compiled(qa, ka, va)
    except Exception as e:                              # no working inductor toolchain on this machine
        pytest.skip(f"torch.compile is not usable here: {type(e).__name__}: {str(e)[:300]}")
    oa.backward(go)
    ob = f(qb, kb, vb)
    ob.backward(go)
    torch.cuda.synchronize()
    assert torch.equal(oa, ob) and torch.equal(qa.grad, qb.grad) and torch.equal(ka.grad, kb.grad) and torch.equal(va.grad, vb.grad)


def test_torch_compile_traces_without_a_graph_break(oracle):
    """The API is made of registered ops with fake implementations (torch.ops.delta_matching_b200.*), so dynamo traces
    through dm_attn_func instead of falling back to eager around it (reference: tests/test_api.py:304-317)."""
    import torch._dynamo
    from delta_matching_b200 import dm_attn_func
    q, k, v, _ = _inputs(oracle, 44)

    def f(q, k, v):
        return dm_attn_func(q * 1.0, k, v, causal=True, mode="matched") + 0.0
    torch._dynamo.reset()
    ex = torch._dynamo.explain(f)(q.detach().requires_grad_(True), k, v)
    assert ex.graph_break_count == 0, ex.break_reasons
    assert ex.graph_count == 1
    names = {str(n.target) for g in ex.graphs for n in g.graph.nodes}
    assert any("autograd_function_apply" in n or "delta_matching_b200" in n for n in names), names
