"""The boundary on caller-chosen streams and devices, after the reference's tests (tests/test_api.py:72-82: a call on a
device that is not the current one; tests/test_sm100_hd256.py:151-163: two caller streams give bitwise equal results)."""
import pytest
import torch

from .helpers import run_api

pytestmark = pytest.mark.gpu
NAMES = ("O", "dQ", "dK", "dV")


def _run_on_stream(q, k, v, do, stream):
    import delta_matching_b200 as dm
    with torch.cuda.stream(stream):
        leaves = [t.detach().clone().requires_grad_() for t in (q, k, v)]
        o = dm.dm_attn_func(*leaves, causal=True, mode="matched")
        o.backward(do)
    return {"O": o.detach(), "dQ": leaves[0].grad, "dK": leaves[1].grad, "dV": leaves[2].grad}


@pytest.mark.parametrize("D,N", [(128, 1024), (256, 512)])
def test_two_caller_streams_bitwise(D, N, oracle):
    """Forward + backward issued on two side streams at the same time (kernels of the two calls may overlap on the GPU)
    equal the call on the default stream bit for bit."""
    from delta_matching_b200 import ops
    q, k, v, do = oracle.make_inputs(2, N, 4, 2, D, seed=41, device="cuda")
    ref = run_api(q, k, v, do, True, "matched")
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    cur = torch.cuda.current_stream()
    s1.wait_stream(cur)
    s2.wait_stream(cur)
    a = _run_on_stream(q, k, v, do, s1)
    b = _run_on_stream(q, k, v, do, s2)
    cur.wait_stream(s1)
    cur.wait_stream(s2)
    torch.cuda.synchronize()
    ops.check_status(q.device)
    for nm in NAMES:
        assert torch.equal(a[nm], ref[nm]), f"stream 1 {nm}"
        assert torch.equal(b[nm], ref[nm]), f"stream 2 {nm}"


def test_non_current_device(oracle):
    """Inputs on cuda:1 while cuda:0 is current: the call runs on the tensors' device and gives the bits of the same call
    made with that device current."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from delta_matching_b200 import ops
    q, k, v, do = (t.to("cuda:1") for t in oracle.make_inputs(1, 512, 4, 2, 128, seed=42, device="cuda:0"))
    with torch.cuda.device(1):
        ref = run_api(q, k, v, do, True, "matched")
    assert torch.cuda.current_device() == 0
    got = run_api(q, k, v, do, True, "matched")
    torch.cuda.synchronize(1)
    ops.check_status("cuda:1")
    for nm in NAMES:
        assert got[nm].device == q.device
        assert torch.equal(got[nm], ref[nm]), nm
