"""The exception contract of the public API (types and the message fragments the reference's tests match:
tests/test_dm_attn.py:126-143, tests/test_api.py:117-149 of the reference).  The checks that precede the device check
run without a GPU; the rest are GPU tests."""
import pytest
import torch

import delta_matching_b200 as dm

BF = torch.bfloat16


def _cpu(B=1, N=256, H=2, Hk=2, D=128, dtype=BF):
    return [torch.zeros(B, N, h, D, dtype=dtype) for h in (H, Hk, Hk)]


def test_public_names():
    for name in ("dm_attn_func", "dm_attn_func_bhnd", "dm_attn_func_plain", "flash_attn_func", "blocks", "kernel_version",
                 "__version__", "KERNEL_NUMERICS"):
        assert hasattr(dm, name), name
    assert set(dm.__all__) >= {"dm_attn_func", "dm_attn_func_bhnd", "flash_attn_func", "kernel_version"}
    assert dm.blocks(128) == (32, 32) and dm.blocks(256) == (32, 32)
    v = dm.kernel_version()
    assert set(v) >= {"version", "code_sha", "fa_src_commit", "numerics"}
    assert len(v["code_sha"]) == 12 and set(v["numerics"]) == {"128", "256"}
    assert v["numerics"]["128"] == "sm100-mx" and v["bf16_dp"] is False


def test_cpu_side_refusals():
    q, k, v = _cpu()
    with pytest.raises(ValueError, match="4-D"):
        dm.dm_attn_func(q[0], k, v, causal=True)
    with pytest.raises(ValueError, match="4-D"):
        dm.dm_attn_func("q", k, v, causal=True)
    with pytest.raises(TypeError):
        dm.dm_attn_func_bhnd("q", k, v)
    with pytest.raises(ValueError, match="4-D"):
        dm.dm_attn_func_bhnd(q[0], k, v)
    with pytest.raises(ValueError, match="CUDA"):
        dm.dm_attn_func(q, k, v, causal=True)
    with pytest.raises(TypeError, match="unexpected keyword"):
        dm.dm_attn_func(q, k, v, causal=True, window=3)


def test_flash_attn_func_refusals():
    q, k, v = _cpu()
    with pytest.raises(NotImplementedError, match="dropout"):
        dm.flash_attn_func(q, k, v, dropout_p=0.1)
    with pytest.raises(NotImplementedError, match="window"):
        dm.flash_attn_func(q, k, v, window_size=(128, 0))
    with pytest.raises(NotImplementedError, match="softcap"):
        dm.flash_attn_func(q, k, v, softcap=30.0)
    with pytest.raises(NotImplementedError, match="alibi"):
        dm.flash_attn_func(q, k, v, alibi_slopes=torch.zeros(2))
    with pytest.raises(NotImplementedError, match="return_attn_probs"):
        dm.flash_attn_func(q, k, v, return_attn_probs=True)
    with pytest.raises(ValueError, match="CUDA"):        # `deterministic` is accepted; the next check is the device
        dm.flash_attn_func(q, k, v, causal=True, deterministic=True)


@pytest.mark.gpu
def test_gpu_side_refusals():
    def t(B=1, N=256, H=2, Hk=2, D=128, dtype=BF):
        return [torch.zeros(B, N, h, D, dtype=dtype, device="cuda") for h in (H, Hk, Hk)]
    q, k, v = t()
    with pytest.raises(TypeError, match="bfloat16"):
        dm.dm_attn_func(*t(dtype=torch.float16), causal=True)
    with pytest.raises(ValueError, match="mode"):
        dm.dm_attn_func(q, k, v, causal=True, mode="fresh")
    with pytest.raises(ValueError, match="causal"):
        dm.dm_attn_func(q, k, v)                          # the bare call: matched + causal=False
    with pytest.raises(ValueError, match="shape"):
        dm.dm_attn_func(q, k, v[:, :, :1], causal=True)
    with pytest.raises(ValueError, match="seqlen"):
        dm.dm_attn_func(q, k[:, :128], v[:, :128], causal=True)
    with pytest.raises(ValueError, match="nheads"):
        dm.dm_attn_func(*t(H=3, Hk=2), causal=True)
    with pytest.raises(ValueError, match="head_dim"):
        dm.dm_attn_func(*t(D=64), causal=True)
    with pytest.raises(ValueError, match="256"):
        dm.dm_attn_func(*t(N=128), causal=True)
    with pytest.raises(ValueError, match="seqlen"):
        dm.dm_attn_func(*t(N=320), causal=True)
    with pytest.raises(NotImplementedError, match="softmax_scale"):
        dm.dm_attn_func(q, k, v, softmax_scale=0.5, causal=True)
    dm.dm_attn_func(q, k, v, softmax_scale=128 ** -0.5, causal=True)      # the fixed value is accepted
    with pytest.raises(ValueError):
        dm.dm_attn_func(q, k.cpu(), v, causal=True)


@pytest.mark.gpu
def test_op_level_misuse():
    """The op layer raises RuntimeError before any launch (reference tests/test_api.py:171-191)."""
    from delta_matching_b200 import ops
    q = torch.zeros(1, 2, 256, 128, dtype=BF, device="cuda")
    q8, qs, k8, ks, v8, vs, _ = ops.quant_qkv(q, q, q)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.fwd_fp8(q8.cpu(), k8, v8, qs, ks, vs, True)
    with pytest.raises(RuntimeError, match="e4m3"):
        ops.fwd_fp8(q8.view(torch.uint8), k8, v8, qs, ks, vs, True)
    with pytest.raises(RuntimeError, match="fp32"):
        ops.fwd_fp8(q8, k8, v8, qs.half(), ks, vs, True)
    with pytest.raises(RuntimeError, match="empty"):
        ops.quant_rows(q[:, :0])
    with pytest.raises(RuntimeError, match="contiguous"):
        ops.fwd_fp8(q8.transpose(1, 2), k8, v8, qs, ks, vs, True)
    if torch.cuda.device_count() > 1:
        with pytest.raises(RuntimeError, match="same device"):
            ops.fwd_fp8(q8, k8.to("cuda:1"), v8, qs, ks, vs, True)
    # the C ABI itself refuses bad arguments with a message (no launch)
    from delta_matching_b200 import _lib
    import ctypes
    L = _lib.lib()
    rc = L.dm_fwd(None, None, None, None, None, None, 1, 100, 2, 2, 128, 1, None, 0, 0, 0, None, None, None)
    assert rc < 0 and "multiple of 128" in _lib.last_error()
    rc = L.dm_fwd(None, None, None, None, None, None, 1, 256, 2, 2, 128, 1, None, 0, 0, 0, None, None, None)
    assert rc < 0 and "NULL" in _lib.last_error()
    host = ctypes.create_string_buffer(1 << 16)
    p = ctypes.cast(host, ctypes.c_void_p)
    rc = L.dm_fwd(p, p, p, p, p, p, 1, 256, 2, 2, 128, 1, p, 0, 0, 0, p, None, None)
    assert rc < 0 and "CUDA memory" in _lib.last_error()
