"""CPU restatement of the reference's fp8 attention numerics (its Blackwell contract, emulation preset "sm100-mx", and the
arms "sm100-mx-ds32" and "sm100-mx-nonorm" of the same preset table).

TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA kernels: tests/, the smoke entry and the CPU-baseline
leg of the benchmark may import it; the product package never does.  Every function restates, in its own code, what
delta_matching/reference.py (the reference's pure-PyTorch emulation) computes for preset "sm100-mx"; the cited lines are
the ones each function follows.  Parity of this file with the reference itself is pinned by tests/golden/ (vectors
produced by running the reference in the build container, script tests/golden/make_golden.py).

Plain torch ops on whatever device the inputs live on (CPU by default), fp32 unless noted.  Layout as the reference:
q (B, N, H, D), k / v (B, N, Hk, D), do (B, N, H, D); results in the same layout.

What the restatement is exact about: every quantisation point (which tensor, which block, which scale, RNE e4m3 with
saturation).  What it is not: tensor-core accumulation order and the hardware exp2 approximation, so a correct kernel
sits at fp32 round-off (times the few fp8 code flips that causes) from it.
"""
from __future__ import annotations

import math

import torch

E4M3 = torch.float8_e4m3fn
E4M3_MAX = 448.0
LOG2E = 1.4426950408889634
BLK = 32          # tokens per input scale; keys per forward-P block; queries per P^T block; keys per dS block
DS_ROWS = 128     # queries per dS block of the contract
# numerics arm -> (queries per dS block, matched delta divided by sum P): delta_matching/reference.py:613, 620, 625, 629-630
NUMERICS = {
    "sm100-mx": (128, True),
    "sm100-mx-d256": (128, True),
    "sm100-mx-ds32": (32, True),
    "sm100-mx-d256-ds32": (32, True),
    "sm100-mx-nonorm": (128, False),
}


# ----------------------------------------------------------------------------------------------------- quantisers
def to_e4m3(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> nearest e4m3 value (RNE, saturating at +-448), kept as fp32.  reference.py:36-38."""
    return x.clamp(-E4M3_MAX, E4M3_MAX).to(E4M3).to(torch.float32)


def pow2_ceil_scale(amax: torch.Tensor, zero_to_one: bool, min_byte: int = 0) -> torch.Tensor:
    """Smallest power of two s with amax <= 448 s, from the fp32 bit pattern of amax = m 2^E: 2^(E-8) when m <= 1.75,
    else 2^(E-7), exponent byte clamped to [min_byte, 254].  amax == 0 gives 1 (zero_to_one) or 2^-127.
    reference.py:54-71 ("ceil", clamp to 2^-127 .. 2^127) and :96-99; the bit rule and the producers' lower clamp of 1
    are delta_matching/sm100/quant.py:160-176."""
    a = amax.to(torch.float32).contiguous()
    bits = a.view(torch.int32)
    eb = ((bits >> 23) & 0xFF) - 8 + ((bits & 0x7FFFFF) > 0x600000).to(torch.int32)
    eb = eb.clamp(min_byte, 254)
    eb = torch.where(a > 0, eb, torch.full_like(eb, 127 if zero_to_one else 0))
    return torch.exp2((eb - 127).to(torch.float32))


def quant_tokens(x: torch.Tensor):
    """Producer quantiser: x (..., N, D) fp32 -> (codes as fp32-valued e4m3, scales (..., N/32)); one power-of-two scale
    per 32 tokens over all D, all-zero block -> scale 1.  reference.py:102-107 (fake_blockrows_pow2)."""
    *lead, N, D = x.shape
    xb = x.reshape(*lead, N // BLK, BLK * D)
    s = pow2_ceil_scale(xb.abs().amax(-1), True, 1)
    codes = to_e4m3(xb / s.unsqueeze(-1)).reshape(*lead, N, D)
    return codes, s


def dequant_tokens(codes: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    return codes * s.repeat_interleave(BLK, dim=-1).unsqueeze(-1)


def kmean_chunked(k: torch.Tensor) -> torch.Tensor:
    """K mean over tokens, k (..., N, D) fp32 -> (..., D): fp32 sums of 64-token chunks folded serially in chunk order,
    divided by N.  reference.py:328-338 (kmean_sm90)."""
    N = k.shape[-2]
    if N % 64:
        return k.mean(-2)
    chunk = k.reshape(*k.shape[:-2], N // 64, 64, k.shape[-1]).sum(-2)
    run = torch.zeros_like(chunk[..., 0, :])
    for j in range(chunk.shape[-2]):
        run = run + chunk[..., j, :]
    return run / N


def quant_p_forward(S: torch.Tensor, row_max: torch.Tensor) -> torch.Tensor:
    """Forward P-hat in units of exp(S - row_max): per (row, 32-key block) k = floor(max x) with x = S log2e,
    code = e4m3(2^(x - k + 7)), value = code 2^(k - 7 - row_max log2e).  Blocks with no live key give zeros.
    reference.py:159-171 (mx_pfwd)."""
    R, C = S.shape[-2:]
    x = S * LOG2E
    xb = x.reshape(*x.shape[:-1], C // BLK, BLK)
    kb = torch.floor(xb.amax(-1, keepdim=True))
    xm = (row_max * LOG2E).unsqueeze(-1)
    kb = torch.where(torch.isfinite(kb), kb, xm.expand_as(kb))
    ph = to_e4m3(torch.exp2(xb - kb + 7)) * torch.exp2(kb - 7 - xm)
    return ph.reshape(x.shape)


def quant_rows_of_queries(P: torch.Tensor) -> torch.Tensor:
    """Backward P^T for dV: power-of-two scale per (key, 32 queries), all-zero block -> 2^-127.
    reference.py:74-93 (fake_mx along the query axis, "ceil" rounding) via scheme "mx:queries:32"."""
    R, C = P.shape[-2:]
    t = P.reshape(*P.shape[:-2], R // BLK, BLK, C)
    s = pow2_ceil_scale(t.abs().amax(-2, keepdim=True), False)
    return (to_e4m3(t / s) * s).reshape(P.shape)


def quant_ds(dS: torch.Tensor, rows: int = DS_ROWS) -> torch.Tensor:
    """dS codes (one set for dK and dQ): power-of-two scale per (`rows` queries x 32 keys), all-zero block -> 1.
    reference.py:110-116 (fake_mx2d) via scheme "mx2d:128x32" (the contract) or "mx2d:32x32" (the ds32 arms)."""
    R, C = dS.shape[-2:]
    t = dS.reshape(*dS.shape[:-2], R // rows, rows, C // BLK, BLK)
    s = pow2_ceil_scale(t.abs().amax(dim=(-3, -1), keepdim=True), True)
    return (to_e4m3(t / s) * s).reshape(dS.shape)


# ----------------------------------------------------------------------------------------------------- exact attention
def attention_exact(q, k, v, do, causal=True, dtype=torch.float32):
    """Unquantised attention with autograd gradients (fp32 or fp64).  reference.py:357-376 (attention_fp32)."""
    B, N, H, D = q.shape
    Hk = k.shape[2]
    qf = q.to(dtype).transpose(1, 2).detach().requires_grad_(True)
    kf = k.to(dtype).transpose(1, 2).detach().requires_grad_(True)
    vf = v.to(dtype).transpose(1, 2).detach().requires_grad_(True)
    s = (qf @ kf.repeat_interleave(H // Hk, dim=1).transpose(-1, -2)) * (D ** -0.5)
    if causal:
        s = s.masked_fill(~torch.ones(N, N, device=q.device, dtype=torch.bool).tril(), float("-inf"))
    o = torch.softmax(s, dim=-1) @ vf.repeat_interleave(H // Hk, dim=1)
    o.backward(do.to(dtype).transpose(1, 2))
    return {"O": o.detach().transpose(1, 2), "LSE": torch.logsumexp(s.detach(), -1), "dQ": qf.grad.transpose(1, 2),
            "dK": kf.grad.transpose(1, 2), "dV": vf.grad.transpose(1, 2)}


# ----------------------------------------------------------------------------------------------------- the emulation
def producers(q, k, v, do=None, k_mean=None):
    """Dequantised operands in (B, H, N, D): Q (softmax scale baked in), centred K, V, dO, plus the K mean used.
    reference.py:408-433 with q = k = v = do = "blockrows_pow2:32"."""
    f32 = torch.float32
    D = q.shape[-1]
    qh = q.to(f32).transpose(1, 2) * (D ** -0.5)
    kh = k.to(f32).transpose(1, 2)
    km = kmean_chunked(kh) if k_mean is None else k_mean.to(f32).reshape(kh.shape[0], kh.shape[1], D)
    kh = kh - km.unsqueeze(-2)
    out = {"kmean": km}
    for name, t in (("q", qh), ("k", kh), ("v", v.to(f32).transpose(1, 2)),
                    ("do", None if do is None else do.to(f32).transpose(1, 2))):
        if t is None:
            continue
        c, s = quant_tokens(t)
        out[name + "_codes"], out[name + "_scales"], out[name] = c, s, dequant_tokens(c, s)
    return out


def dm_oracle(q, k, v, do, causal=True, mode="matched", k_mean=None, o_for_stale=None, lse_override=None, aux=False,
              q_block=1024, numerics="sm100-mx"):
    """Forward + backward of the "sm100-mx" emulation.  Returns O (bf16), LSE (B, H, N) natural log, dQ / dK / dV fp32
    in the input layout, delta (B, H, N); aux=True adds rowsum_dS and sum_absPdP (fp64 sums over keys).
    reference.py:387-523 (dm_reference) restricted to preset "sm100-mx" (:612-613): forward P per (row, 32 keys),
    l from the unquantised P, backward P^T per (key, 32 queries), dS per (128 queries x 32 keys), matched
    delta = sum P dP / sum P in fp64 (:526-535), stale delta = rowsum(dO * O) on the bf16 O (:500-501).
    numerics: another arm of NUMERICS changes the dS block to 32 x 32 (:625, 630) or drops the division (:620)."""
    if mode not in ("matched", "stale"):
        raise ValueError(mode)
    ds_rows, delta_norm = NUMERICS[numerics]
    B, N, H, D = q.shape
    Hk = k.shape[2]
    rep = H // Hk
    sm = D ** -0.5
    dev = q.device
    f32 = torch.float32
    ops = producers(q, k, v, do, k_mean)
    Q, K, V, dO = ops["q"], ops["k"], ops["v"], ops["do"]
    do_raw = do.to(f32).transpose(1, 2)
    O = torch.empty(B, H, N, D, device=dev, dtype=f32)
    LSE = torch.empty(B, H, N, device=dev, dtype=f32)
    dQ = torch.zeros(B, H, N, D, device=dev, dtype=f32)
    dK = torch.zeros(B, Hk, N, D, device=dev, dtype=f32)
    dV = torch.zeros(B, Hk, N, D, device=dev, dtype=f32)
    delta = torch.empty(B, H, N, device=dev, dtype=f32)
    rs = torch.empty(B, H, N, device=dev, dtype=torch.float64) if aux else None
    ap = torch.empty(B, H, N, device=dev, dtype=torch.float64) if aux else None
    qb = min(q_block, N)
    idx = torch.arange(N, device=dev)

    def keys_for(i1):
        return i1 if causal else N

    def logits(i0, i1, nk):
        S = Q[:, :, i0:i1] @ K[:, :, :nk].repeat_interleave(rep, 1).transpose(-1, -2)
        if causal:
            S = S.masked_fill(idx[None, :nk] > idx[i0:i1, None], float("-inf"))
        return S

    for i0 in range(0, N, qb):                       # forward, reference.py:454-471
        i1 = min(i0 + qb, N)
        nk = keys_for(i1)
        S = logits(i0, i1, nk)
        m = S.amax(-1, keepdim=True)
        P = torch.exp(S - m)
        l = P.sum(-1, keepdim=True)
        Pq = quant_p_forward(S, m)
        O[:, :, i0:i1] = (Pq @ V[:, :, :nk].repeat_interleave(rep, 1)) / l
        LSE[:, :, i0:i1] = (m + torch.log(l)).squeeze(-1)
    if lse_override is not None:
        LSE = lse_override.to(f32).reshape(B, H, N).clone()
    Ob = O.to(torch.bfloat16)
    O_stale = Ob.to(f32) if o_for_stale is None else o_for_stale.to(f32).transpose(1, 2)

    for i0 in range(0, N, qb):                       # backward, reference.py:476-518
        i1 = min(i0 + qb, N)
        nk = keys_for(i1)
        S = logits(i0, i1, nk)
        P = torch.exp(S - LSE[:, :, i0:i1, None])
        Pt = quant_rows_of_queries(P)
        dV[:, :, :nk] += (Pt.transpose(-1, -2) @ dO[:, :, i0:i1]).reshape(B, Hk, rep, nk, D).sum(2)
        dP = dO[:, :, i0:i1] @ V[:, :, :nk].repeat_interleave(rep, 1).transpose(-1, -2)
        if mode == "stale":
            dl = (do_raw[:, :, i0:i1] * O_stale[:, :, i0:i1]).sum(-1, keepdim=True)
        else:
            dl = (P.double() * dP.double()).sum(-1, keepdim=True)
            if delta_norm:
                dl = dl / P.double().sum(-1, keepdim=True)
            dl = dl.float()
        delta[:, :, i0:i1] = dl.squeeze(-1)
        dS = P * (dP - dl)
        if aux:
            rs[:, :, i0:i1] = dS.double().sum(-1)
            ap[:, :, i0:i1] = (P.double() * dP.double()).abs().sum(-1)
        dSq = quant_ds(dS, ds_rows)
        dK[:, :, :nk] += (dSq.transpose(-1, -2) @ Q[:, :, i0:i1]).reshape(B, Hk, rep, nk, D).sum(2)
        dQ[:, :, i0:i1] = (dSq @ K[:, :, :nk].repeat_interleave(rep, 1)) * sm
    out = {"O": Ob.transpose(1, 2), "LSE": LSE, "dQ": dQ.transpose(1, 2), "dK": dK.transpose(1, 2),
           "dV": dV.transpose(1, 2), "delta": delta, "kmean": ops["kmean"]}
    if aux:
        out["rowsum_dS"], out["sum_absPdP"] = rs, ap
    return out


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    """|a - b| / |b| in fp64 (the reference tests' `rel`, tests/test_sm100.py:45-47)."""
    a, b = a.double(), b.double()
    return ((a - b).norm() / b.norm().clamp_min(1e-300)).item()


def make_inputs(B, N, H, Hk, D, seed=0, device="cpu", qk_scale=1.0, unit_rms=False):
    """Seeded bf16 q, k, v, dO drawn i.i.d. N(0, 1) in that order on a CPU generator (tests/test_sm100.py:50-52);
    qk_scale multiplies q and k before the bf16 cast; unit_rms divides q and k rows by their RMS over D."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    out = []
    for i, h in enumerate((H, Hk, Hk, H)):
        t = torch.randn(B, N, h, D, generator=g)
        if i < 2:
            if unit_rms:
                t = t / t.pow(2).mean(-1, keepdim=True).sqrt()
            t = t * qk_scale
        out.append(t.to(torch.bfloat16).to(device))
    return out
