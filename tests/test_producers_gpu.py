"""Quantisation producers on the GPU, through the C ABI: bit-exact codes and scales against the reference's golden
vectors and against the oracle on larger seeded inputs; K mean to fp32 round-off; stale delta; strided inputs."""
import pytest
import torch

from .conftest import GOLDEN_CASES, load_golden

pytestmark = pytest.mark.gpu


def _bits(c):
    return c.view(torch.uint8)


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_golden_codes_and_scales(case, oracle):
    from delta_matching_b200 import ops
    g = load_golden(case)
    q, k, v, do = (g[n].cuda().transpose(1, 2) for n in ("q", "k", "v", "do"))
    q8, qs, k8, ks, v8, vs, km = ops.quant_qkv(q, k, v)
    do8, dos, _ = ops.quant_do(do)
    torch.cuda.synchronize()
    for nm, c, s in (("q", q8, qs), ("v", v8, vs), ("do", do8, dos)):
        assert torch.equal(_bits(c).cpu(), g[nm + "_codes"]), nm
        assert torch.equal(s.cpu(), g[nm + "_scales"]), nm
    # K mean: same chunked order, within-chunk order differs from torch's -> fp32 round-off
    assert (km.cpu() - g["kmean"]).abs().max().item() <= 4e-7 * max(1.0, g["kmean"].abs().max().item()) + 1e-6
    # K codes: bit-exact against the oracle's quantiser run on the kernel's own mean
    p = oracle.producers(g["q"], g["k"], g["v"], None, k_mean=km.cpu())
    assert torch.equal(_bits(k8).cpu(), p["k_codes"].to(torch.float8_e4m3fn).view(torch.uint8))
    assert torch.equal(ks.cpu(), p["k_scales"])


@pytest.mark.parametrize("B,N,H,Hk,D", [(2, 512, 4, 2, 128), (1, 384, 3, 1, 256), (1, 4096, 2, 1, 128)])
def test_against_oracle(B, N, H, Hk, D, oracle):
    from delta_matching_b200 import ops
    q, k, v, do = oracle.make_inputs(B, N, H, Hk, D, seed=5, device="cuda")
    q8, qs, k8, ks, v8, vs, km = ops.quant_qkv(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
    do8, dos, _ = ops.quant_do(do.transpose(1, 2))
    p = oracle.producers(q, k, v, do, k_mean=km)
    for nm, c, s in (("q", q8, qs), ("k", k8, ks), ("v", v8, vs), ("do", do8, dos)):
        assert torch.equal(_bits(c), p[nm + "_codes"].to(torch.float8_e4m3fn).view(torch.uint8)), nm
        assert torch.equal(s, p[nm + "_scales"]), nm
    ref_mean = oracle.kmean_chunked(k.float().transpose(1, 2))
    assert (km - ref_mean).abs().max().item() <= 1e-6


def test_edge_blocks(oracle):
    """All-zero blocks (scale 1, codes 0), a block with one huge outlier, and values at the e4m3 rounding boundary."""
    from delta_matching_b200 import ops
    x = torch.zeros(1, 1, 128, 128, dtype=torch.bfloat16, device="cuda")
    x[0, 0, 32:64] = torch.randn(32, 128, device="cuda").to(torch.bfloat16)
    x[0, 0, 40, 7] = 3.0e4
    x[0, 0, 64:96] = 1.75 * 256            # mantissa exactly 1.75: scale 2^(E-8)
    x[0, 0, 96:128] = 1.7578125 * 256      # just above: scale 2^(E-7)
    c, s = ops.quant_rows(x)
    rc, rs = oracle.quant_tokens(x.float())
    assert torch.equal(s, rs)
    assert torch.equal(_bits(c), rc.to(torch.float8_e4m3fn).view(torch.uint8))
    assert s[0, 0, 0].item() == 1.0 and int(_bits(c)[0, 0, :32].max()) == 0


def test_stale_delta_and_strides(oracle):
    from delta_matching_b200 import ops
    B, N, H, D = 2, 256, 4, 128
    g = torch.Generator(device="cpu").manual_seed(3)
    packed = torch.randn(B, N, 3 * H, D, generator=g).to(torch.bfloat16).cuda()
    do = packed[:, :, :H].transpose(1, 2)            # strided (B, H, N, D) views of one packed tensor
    o = packed[:, :, H:2 * H].transpose(1, 2)
    c1, s1, d1 = ops.quant_do(do, o)
    c2, s2, d2 = ops.quant_do(do.contiguous(), o.contiguous())
    assert torch.equal(_bits(c1), _bits(c2)) and torch.equal(s1, s2) and torch.equal(d1, d2)
    want = (do.float() * o.float()).sum(-1)
    assert (d1 - want).abs().max().item() <= 1e-4 * want.abs().max().item()
    # a misaligned view is copied, not misread
    odd = torch.randn(B, H, N, D + 8, generator=g).to(torch.bfloat16).cuda()[..., 4:D + 4]
    c3, s3 = ops.quant_rows(odd)
    c4, s4 = ops.quant_rows(odd.contiguous())
    assert torch.equal(_bits(c3), _bits(c4)) and torch.equal(s3, s4)
