"""dm_kmean_static: the K mean for callers that cannot allocate (the scratch lives inside the library).

Collected last on purpose.  Calls the entry point through the C ABI and checks it against dm_kmean, which takes a
caller-allocated workspace: same kernels, same summation order, so the means must be bit-identical, on two calls in a row
that reuse the built-in scratch with different shapes (the second call must not be disturbed by what the first left
behind).  Problems beyond the built-in scratch are refused with a message."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _static_kmean(k):
    """k (B, Hk, N, D) bf16 CUDA -> (rc, mean, message) through dm_kmean_static."""
    from delta_matching_b200 import _lib
    L = _lib.lib()
    B, Hk, N, D = k.shape
    mean = torch.full((B, Hk, D), float("nan"), device=k.device, dtype=torch.float32)
    err = ctypes.create_string_buffer(512)
    before = torch.cuda.memory_allocated(k.device)
    rc = L.dm_kmean_static(ctypes.c_void_p(k.data_ptr()), k.stride(0), k.stride(1), k.stride(2), B, N, Hk, D,
                           ctypes.c_void_p(mean.data_ptr()),
                           ctypes.c_void_p(torch.cuda.current_stream(k.device).cuda_stream), err, 512)
    assert torch.cuda.memory_allocated(k.device) == before
    return rc, mean, err.value.decode()


def test_matches_workspace_version_twice_in_a_row():
    from delta_matching_b200 import ops
    g = torch.Generator(device="cpu").manual_seed(11)
    for (B, Hk, N, D) in ((2, 2, 1024, 128), (1, 3, 384, 256)):
        k = (torch.randn(B, Hk, N, D, generator=g) + 0.25).to(torch.bfloat16).cuda()
        rc, got, msg = _static_kmean(k)
        assert rc == 0, msg
        want = ops.kmean(k)
        torch.cuda.synchronize()
        assert torch.equal(got, want), (B, Hk, N, D)
    # strided input (token-major storage viewed head-major), as the attention API passes it
    k = torch.randn(1, 512, 2, 128, generator=g).to(torch.bfloat16).cuda().transpose(1, 2)
    rc, got, msg = _static_kmean(k)
    assert rc == 0, msg
    assert torch.equal(got, ops.kmean(k))


def test_refuses_what_does_not_fit():
    k = torch.zeros(1, 1, 128, 128, dtype=torch.bfloat16, device="cuda")
    from delta_matching_b200 import _lib
    L = _lib.lib()
    err = ctypes.create_string_buffer(512)
    mean = torch.zeros(1, 1, 128, device="cuda")
    # B * Hk * (N / 64) * D = 64 * 8 * 512 * 128 floats: far beyond the 1 Mi-float scratch; nothing is launched
    rc = L.dm_kmean_static(ctypes.c_void_p(k.data_ptr()), 8, 8, 128, 64, 32768, 8, 128, ctypes.c_void_p(mean.data_ptr()),
                           None, err, 512)
    assert rc < 0 and "built-in scratch" in err.value.decode()
    rc = L.dm_kmean_static(None, 8, 8, 128, 1, 128, 1, 128, ctypes.c_void_p(mean.data_ptr()), None, err, 512)
    assert rc < 0 and "NULL" in err.value.decode()
    # a host pointer, or memory that is not CUDA memory, is refused before any launch
    host = torch.zeros(1, 1, 128, 128, dtype=torch.bfloat16).pin_memory()
    rc = L.dm_kmean_static(ctypes.c_void_p(host.data_ptr()), 8, 8, 128, 1, 128, 1, 128, ctypes.c_void_p(mean.data_ptr()),
                           None, err, 512)
    assert rc < 0 and "CUDA memory" in err.value.decode()
    rc = L.dm_kmean_static(ctypes.c_void_p(k.data_ptr()), 8, 8, 128, 1, 128, 1, 128,
                           ctypes.c_void_p(mean.data_ptr() + 4), None, err, 512)
    assert rc < 0 and "aligned" in err.value.decode()
