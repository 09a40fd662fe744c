"""A bounded wait that runs out: the kernel returns (nothing hangs, nothing faults), leaves its status code, the op layer
turns the code into RuntimeError, and the next launch works.  The probe kernel is launched with its MMA role told to
skip the commit that the other threads wait for and with a wait limit of 100 microseconds (the attention kernels use
the same wait routine with a limit of two seconds)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_expired_wait_returns_a_status_and_raises():
    from delta_matching_b200 import ops
    dev = torch.device("cuda")
    ops.check_status(dev)                               # nothing pending
    a = torch.randint(0, 120, (128, 128), device=dev, dtype=torch.uint8)
    out = ops.wait_expiry_probe(a, a, limit_us=100)     # returns: the kernel gave up waiting and left
    torch.cuda.synchronize()
    assert int(ops.status_word(dev)[0]) == 4            # kStatusTimeoutProbe, visible to the host without a copy
    with pytest.raises(RuntimeError, match="status 4"):
        ops.check_status(dev)
    ops.check_status(dev)                               # the word was cleared by the raise
    del out
    # the same kernel, normally: a correct product, status stays 0
    g = torch.Generator().manual_seed(5)
    x = torch.randint(-4, 5, (128, 128), generator=g).float()
    y = torch.randint(-4, 5, (128, 128), generator=g).float()
    got = ops.mma_tile(x.to(torch.float8_e4m3fn).cuda(), y.to(torch.float8_e4m3fn).cuda())
    torch.cuda.synchronize()
    ops.check_status(dev)
    assert torch.equal(got.cpu(), x @ y.T)              # small integers: every product and sum is exact


def test_next_op_raises_without_a_sync(oracle):
    """A non-zero status word makes the NEXT op call raise at its entry (the word lives in pinned host memory that the
    kernels write directly), so a timed-out kernel cannot feed a training step silently."""
    from delta_matching_b200 import ops
    dev = torch.device("cuda")
    a = torch.randint(0, 120, (128, 128), device=dev, dtype=torch.uint8)
    ops.wait_expiry_probe(a, a, limit_us=100)
    torch.cuda.synchronize()
    q, k, v, _ = oracle.make_inputs(1, 256, 2, 2, 128, seed=0, device="cuda")
    with pytest.raises(RuntimeError, match="status 4"):
        ops.quant_qkv(*(t.transpose(1, 2) for t in (q, k, v)))
    ops.quant_qkv(*(t.transpose(1, 2) for t in (q, k, v)))        # cleared: works again
    torch.cuda.synchronize()
    ops.check_status(dev)
