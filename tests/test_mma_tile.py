"""The tcgen05 building blocks (TMA 128-byte-swizzled tiles as K-major / MN-major operands, A from TMEM, plain and
block-scaled fp8 MMA, the TMEM scale-word placement) against a host matmul, through the C ABI (dm_dbg_mma_tile).
Inputs are small integers in e4m3, so every product and sum is exact in fp32 and the comparison is bit-exact."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _codes(seed, lo=-4, hi=4):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (128, 128), generator=g).float()


def _run(a, b, **kw):
    from delta_matching_b200 import ops
    a8 = a.to(torch.float8_e4m3fn).cuda()
    b8 = b.to(torch.float8_e4m3fn).cuda()
    out = ops.mma_tile(a8, b8, **kw)
    torch.cuda.synchronize()
    ops.check_status("cuda")
    return out.cpu()


@pytest.mark.parametrize("nk", [1, 2, 4])
def test_ss_kmajor(nk):
    a, b = _codes(1), _codes(2)
    got = _run(a, b, nk=nk)
    assert torch.equal(got, a[:, :32 * nk] @ b[:, :32 * nk].T)


@pytest.mark.parametrize("nk", [1, 4])
def test_ss_b_mn_major(nk):
    """B tile rows are the contraction index (how V, dO, Q and K feed the second matmuls)."""
    a, b = _codes(3), _codes(4)
    got = _run(a, b, b_mn=True, nk=nk)
    assert torch.equal(got, a[:, :32 * nk] @ b[:32 * nk, :])


def test_ss_a_mn_major():
    a, b = _codes(5), _codes(6)
    got = _run(a, b, a_mn=True, nk=4)
    assert torch.equal(got, a.T @ b.T)


@pytest.mark.parametrize("b_mn", [False, True])
def test_ts_a_from_tmem(b_mn):
    a, b = _codes(7), _codes(8)
    got = _run(a, b, a_tmem=True, b_mn=b_mn, nk=4)
    assert torch.equal(got, a @ (b if b_mn else b.T))


def _scale_words(seed, uniform_rows):
    """(128, 4) int32 words whose byte k is the UE8M0 scale of contraction step k; every column holds the row's word."""
    g = torch.Generator().manual_seed(seed)
    if uniform_rows:
        by = torch.randint(120, 134, (1, 4), generator=g).expand(128, 4)
    else:
        by = torch.randint(120, 134, (128, 4), generator=g)
    word = (by[:, 0] | (by[:, 1] << 8) | (by[:, 2] << 16) | (by[:, 3] << 24)).to(torch.int32)
    return word[:, None].expand(128, 4).contiguous(), (by.float() - 127).exp2()


def test_block_scaled_a_mn_major():
    """Both operands MN-major with per-step scales that are the same for every row (the dS^T tile of the second backward
    pass): out = sum_k s[k] A_k^T B_k."""
    a, b = _codes(13), _codes(14)
    sfa, sa = _scale_words(15, uniform_rows=True)
    sfb, sb = _scale_words(16, uniform_rows=True)
    got = _run(a, b, sfa=sfa.cuda(), sfb=sfb.cuda(), a_mn=True, b_mn=True, nk=4)
    want = torch.zeros(128, 128, dtype=torch.float64)
    for k in range(4):
        blk = a[32 * k:32 * k + 32, :].double().T @ b[32 * k:32 * k + 32, :].double()
        want += sa[0, k].double() * sb[0, k].double() * blk
    assert torch.equal(got.double(), want)


@pytest.mark.parametrize("a_tmem", [True, False])
def test_block_scaled(a_tmem):
    """Per-row, per-step A scales (the P / P^T / dS^T scale words) and a per-step B scale shared by all columns (the V
    scale word): out = sum_k sa[i, k] sb[k] A_k B_k."""
    a, b = _codes(9), _codes(10)
    sfa, sa = _scale_words(11, uniform_rows=False)
    sfb, sb = _scale_words(12, uniform_rows=True)
    got = _run(a, b, sfa=sfa.cuda(), sfb=sfb.cuda(), a_tmem=a_tmem, b_mn=True, nk=4)
    want = torch.zeros(128, 128, dtype=torch.float64)
    for k in range(4):
        blk = a[:, 32 * k:32 * k + 32].double() @ b[32 * k:32 * k + 32, :].double()
        want += sa[:, k:k + 1].double() * sb[0, k].double() * blk
    assert torch.equal(got.double(), want)
