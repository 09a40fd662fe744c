"""The registered ops (torch.ops.delta_matching_b200.*) without a GPU: every op exists, and its fake implementation
states the shapes, dtypes and devices that the op layer documents (run on fake CUDA tensors, which need no device)."""
import torch
from torch._subclasses.fake_tensor import FakeTensorMode

import delta_matching_b200  # noqa: F401  (registers the ops)

E4M3, F32, BF16 = torch.float8_e4m3fn, torch.float32, torch.bfloat16


def _meta(t):
    return tuple(t.shape), t.dtype, t.device.type


def test_ops_are_registered():
    ns = torch.ops.delta_matching_b200
    for name in ("quant_qkv", "fwd_fp8", "quant_do", "delta_fp8", "bwd_fp8"):
        assert hasattr(ns, name), name


def test_fake_implementations_state_the_layout():
    ns = torch.ops.delta_matching_b200
    B, H, Hk, N, D = 2, 8, 2, 512, 128
    with FakeTensorMode():
        q = torch.empty(B, H, N, D, device="cuda", dtype=BF16)
        k = torch.empty(B, Hk, N, D, device="cuda", dtype=BF16)
        q8, qs, k8, ks, v8, vs, km = ns.quant_qkv(q, k, k)
        assert _meta(q8) == ((B, H, N, D), E4M3, "cuda") and _meta(k8) == ((B, Hk, N, D), E4M3, "cuda")
        assert _meta(qs) == ((B, H, N // 32), F32, "cuda") and _meta(vs) == ((B, Hk, N // 32), F32, "cuda")
        assert _meta(km) == ((B, Hk, D), F32, "cuda") and _meta(v8) == _meta(k8) and _meta(ks) == _meta(vs)
        o, lse = ns.fwd_fp8(q8, k8, v8, qs, ks, vs, True)
        assert _meta(o) == ((B, N, H, D), BF16, "cuda") and o.is_contiguous()
        assert _meta(lse) == ((B, H, N), F32, "cuda")
        do = torch.empty(B, N, H, D, device="cuda", dtype=BF16).permute(0, 2, 1, 3)
        do8, dos, none = ns.quant_do(do, do, False)
        assert _meta(do8) == _meta(q8) and _meta(dos) == _meta(qs) and none.numel() == 0
        _, _, stale = ns.quant_do(do, o.permute(0, 2, 1, 3), True)
        assert _meta(stale) == ((B, H, N), F32, "cuda")
        delta = ns.delta_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, True, True)
        assert _meta(delta) == _meta(lse)
        dq, dk, dv = ns.bwd_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, delta, True, False)
        assert _meta(dq) == ((B, N, H, D), BF16, "cuda")
        assert _meta(dk) == ((B, N, Hk, D), BF16, "cuda") and _meta(dv) == _meta(dk)
