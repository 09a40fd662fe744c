"""The host-memory training step (pinned CPU tensors in, pinned CPU tensors out, copies pipelined over batch chunks) must
return exactly what one call of the public API on CUDA tensors returns."""
import pytest
import torch

from .helpers import run_api

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("chunks", [None, 1, 2, 3, 6])
@pytest.mark.parametrize("mode,causal", [("matched", True), ("stale", False)])
def test_host_step_is_bit_identical(chunks, mode, causal, oracle):
    from delta_matching_b200.host import attn_step_host
    B, N, H, Hk, D = 3, 512, 4, 2, 128
    q, k, v, do = oracle.make_inputs(B, N, H, Hk, D, seed=21, device="cuda")
    want = run_api(q, k, v, do, causal, mode)
    host = [t.cpu().pin_memory() for t in (q, k, v, do)]
    for _ in range(2):                                    # second call reuses streams and cached blocks
        o, dq, dk, dv = attn_step_host(*host, causal=causal, mode=mode, chunks=chunks)
        torch.cuda.synchronize()
        for name, got in (("O", o), ("dQ", dq), ("dK", dk), ("dV", dv)):
            assert got.is_pinned() and got.device.type == "cpu"
            assert torch.equal(got, want[name].cpu()), name


def test_host_step_fills_out_tensors(oracle):
    from delta_matching_b200.host import attn_step_host
    B, N, H, Hk, D = 2, 256, 2, 2, 128
    q, k, v, do = oracle.make_inputs(B, N, H, Hk, D, seed=22, device="cuda")
    want = run_api(q, k, v, do, True, "matched")
    host = [t.cpu().pin_memory() for t in (q, k, v, do)]
    out = tuple(torch.zeros(t.shape, dtype=torch.bfloat16).pin_memory() for t in (q, q, k, v))
    res = attn_step_host(*host, out=out)
    torch.cuda.synchronize()
    assert all(a is b for a, b in zip(res, out))
    for name, got in zip(("O", "dQ", "dK", "dV"), out):
        assert torch.equal(got, want[name].cpu()), name


def test_host_step_argument_errors():
    from delta_matching_b200.host import attn_step_host
    q = torch.zeros(2, 256, 2, 128, dtype=torch.bfloat16).pin_memory()
    with pytest.raises(ValueError):
        attn_step_host(q, q, q, q, chunks=3)
    with pytest.raises(ValueError):
        attn_step_host(q, q, q, torch.zeros(2, 256, 2, 128, dtype=torch.bfloat16))        # not pinned
    with pytest.raises(ValueError):
        attn_step_host(q.cuda(), q, q, q)
