"""The autograd route and the input contract.

`dm_attn_func_bhnd(q, k, v, causal, softmax_scale, delta_mode)` on (B, H, N, D) inputs returns (B, N, H, D), as
delta_matching/attn.py:121-127 does.  Forward: producers (codes, scales, K mean) then the forward kernel.  Backward: the
dO producer (with the stale delta rowsum(dO * O) when delta_mode == "stale"), the matched delta from pass 0 of the
backward when delta_mode == "matched", then the backward kernels; dK / dV come back already reduced over the GQA group.
Saved for the backward: the fp8 codes, their scales, O and the LSE (delta_matching/attn.py:68 without the transposed
"twin" copies, which tcgen05's MN-major operands make unnecessary).
"""
from __future__ import annotations

import torch

from . import ops
from . import torch_ops as _torch_ops  # noqa: F401  (registers torch.ops.delta_matching_b200.*)

_OPS = torch.ops.delta_matching_b200


def _calls():
    """The registered ops while a compiler is tracing (it records them as opaque nodes), the plain functions otherwise."""
    return _OPS if torch.compiler.is_compiling() else _torch_ops.DIRECT


def blocks(D: int):
    """Tokens per quantisation scale as (Q / dO rows, K / V keys): one power-of-two scale per 32 tokens over all of
    head_dim at both head dims (the reference's Blackwell contract, delta_matching/sm100/quant.py:1-12; its Hopper
    kernels use (128, 64) / (64, 32), delta_matching/core.py:26-29)."""
    return (32, 32)


def _check_inputs(q, k, v, causal, softmax_scale, mode):
    """The input contract on (B, H, N, D) views: ValueError / TypeError / NotImplementedError naming the violated
    constraint, in the order and wording of delta_matching/core.py:112-154 (the device check asks for sm_100)."""
    if not all(isinstance(t, torch.Tensor) for t in (q, k, v)):
        raise TypeError("delta_matching: q, k, v must be torch tensors")
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError(f"delta_matching: q, k, v must be 4-D (got {q.dim()}-D, {k.dim()}-D, {v.dim()}-D)")
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise ValueError(f"delta_matching: q, k, v must be CUDA tensors (got {q.device}, {k.device}, {v.device})")
    if not (q.device == k.device == v.device):
        raise ValueError(f"delta_matching: q, k, v must be on one device (got {q.device}, {k.device}, {v.device})")
    if not (q.dtype == k.dtype == v.dtype == torch.bfloat16):
        raise TypeError(f"delta_matching: q, k, v must be torch.bfloat16 (got {q.dtype}, {k.dtype}, {v.dtype})")
    if mode not in ("matched", "stale"):
        raise ValueError(f"delta_matching: mode must be 'matched' or 'stale' (got {mode!r})")
    if mode == "matched" and not causal:
        raise ValueError("delta_matching: mode='matched' needs causal=True (the matched delta is built for causal "
                         "attention); use mode='stale' for non-causal attention")
    B, H, N, D = q.shape
    if k.shape != v.shape:
        raise ValueError(f"delta_matching: k and v must have the same shape (got {tuple(k.shape)} and {tuple(v.shape)})")
    Bk, Hk, Nk, Dk = k.shape
    if Bk != B or Dk != D:
        raise ValueError("delta_matching: k and v must match q's batch size and head_dim "
                         f"(q {tuple(q.shape)}, k {tuple(k.shape)})")
    if Nk != N:
        raise ValueError(f"delta_matching: q, k, v must have the same seqlen (self-attention only; got {N} and {Nk})")
    if Hk == 0 or H % Hk:
        raise ValueError(f"delta_matching: nheads ({H}) must be a positive multiple of nheads_k ({Hk})")
    if D not in (128, 256):
        raise ValueError(f"delta_matching: head_dim must be 128 or 256 (got {D})")
    mult = 256 if D == 128 else 128
    if N == 0 or N % mult:
        raise ValueError(f"delta_matching: seqlen must be a positive multiple of {mult} at head_dim {D} (got {N})")
    if B == 0:
        raise ValueError("delta_matching: empty batch")
    if B * H > 65535:
        raise ValueError(f"delta_matching: batch * nheads must be at most 65535 (got {B * H})")
    if softmax_scale is not None and abs(softmax_scale - D ** -0.5) > 1e-12:
        raise NotImplementedError(f"delta_matching: softmax_scale is fixed at head_dim ** -0.5 = {D ** -0.5!r} (it is "
                                  f"baked into the Q codes); got {softmax_scale!r}")
    if not _is_sm100(q.device.index if q.device.index is not None else torch.cuda.current_device()):
        major, minor = torch.cuda.get_device_capability(q.device)
        raise ValueError(f"delta_matching: needs a Blackwell GPU (sm_100); {q.device} is sm{major}{minor}")


@torch.compiler.assume_constant_result
def _is_sm100(index: int) -> bool:
    """A fact about the machine, not about the tensors: a tracing compiler may bake the answer into its graph."""
    return torch.cuda.get_device_capability(index)[0] == 10


class _DMAttn(torch.autograd.Function):
    """Forward and backward as calls of the registered ops (delta_matching_b200/torch_ops.py), the way the reference's
    autograd function calls torch.ops.delta_matching (delta_matching/attn.py:37-118): a tracing compiler records five
    opaque ops instead of breaking its graph here; eager calls skip the dispatcher and run the same functions directly."""

    @staticmethod
    def forward(ctx, q, k, v, causal, delta_mode, ds32, norm):
        K = _calls()
        q8, qs, k8, ks, v8, vs, _ = K.quant_qkv(q, k, v)
        o, lse = K.fwd_fp8(q8, k8, v8, qs, ks, vs, causal)
        ctx.save_for_backward(q8, qs, k8, ks, v8, vs, o, lse)
        ctx.causal = causal
        ctx.delta_mode = delta_mode
        ctx.ds32, ctx.norm = ds32, norm
        return o

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dO):
        q8, qs, k8, ks, v8, vs, o, lse = ctx.saved_tensors
        K = _calls()
        if dO.stride(-1) != 1:          # e.g. the expanded gradient of o.sum()
            dO = dO.contiguous()
        do_bhnd = dO.permute(0, 2, 1, 3)                   # (B, N, H, D) -> (B, H, N, D) view, read in place
        if ctx.delta_mode == "matched":
            do8, dos, _ = K.quant_do(do_bhnd, do_bhnd, False)       # the matched mode never reads O
            delta = K.delta_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, ctx.causal, ctx.norm)
        else:
            do8, dos, delta = K.quant_do(do_bhnd, o.permute(0, 2, 1, 3), True)
        dq, dk, dv = K.bwd_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, delta, ctx.causal, ctx.ds32)
        return dq.permute(0, 2, 1, 3), dk.permute(0, 2, 1, 3), dv.permute(0, 2, 1, 3), None, None, None, None


def _numerics(name, D):
    """(ds32, norm) of a numerics arm (ops.NUMERICS); the head_dim-256 names are accepted at head_dim 256 only."""
    if name not in ops.NUMERICS:
        raise ValueError(f"delta_matching: numerics must be one of {sorted(ops.NUMERICS)} (got {name!r})")
    if "-d256" in name and D != 256:
        raise ValueError(f"delta_matching: numerics {name!r} is the head_dim-256 name of its scheme (head_dim is {D})")
    return ops.NUMERICS[name]


def dm_attn_func_bhnd(q, k, v, causal=True, softmax_scale=None, delta_mode="stale", numerics="sm100-mx"):
    """Attention on (B, H, N, D) inputs: q (B, H, N, D), k / v (B, Hk, N, D) bf16 on CUDA (any strides; H % Hk == 0) ->
    O (B, N, H, D) bf16 contiguous.  delta_mode: "stale" (delta = rowsum(dO * O)) or "matched" (the Delta-Matching
    backward; needs causal=True).  Input errors raise ValueError / TypeError / NotImplementedError.  Works under
    torch.compile without a graph break (the kernels are registered ops with fake implementations) and under CUDA-graph
    capture after a warm-up call.  numerics: the reference's Blackwell contract "sm100-mx" or one of the arms of
    ops.NUMERICS (the same forward; the backward's dS block or the matched delta's normalisation differ)."""
    _check_inputs(q, k, v, causal, softmax_scale, delta_mode)
    ds32, norm = _numerics(numerics, q.shape[-1])
    return _DMAttn.apply(q, k, v, causal, delta_mode, ds32, norm)


@torch.no_grad()
def dm_attn_debug(q, k, v, do, causal=True, mode="matched", identity=False, numerics="sm100-mx"):
    """The delta the backward consumes and the LSE it recomputes P from ("delta", "lse", (B, H, N) fp32), from the same
    producers, forward and delta path as dm_attn_func on (B, N, H, D) inputs; identity=True (matched mode) also returns
    "rowsum_dS" = sum_j dS_ij and "sum_abs_PdP" = sum_j |P_ij dP_ij| accumulated inside the backward before dS is
    quantised.  Mirrors delta_matching/sm100/attention.py:36-52."""
    qh, kh, vh, doh = (t.transpose(1, 2) for t in (q, k, v, do))
    _check_inputs(qh, kh, vh, causal, None, mode)
    ds32, norm = _numerics(numerics, q.shape[-1])
    q8, qs, k8, ks, v8, vs, km = ops.quant_qkv(qh, kh, vh)
    o, lse = ops.fwd_fp8(q8, k8, v8, qs, ks, vs, causal)
    if mode == "matched":
        do8, dos, _ = ops.quant_do(doh, None)
        delta = ops.delta_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, causal, norm)
    else:
        do8, dos, delta = ops.quant_do(doh, o.permute(0, 2, 1, 3))
    out = {"delta": delta, "lse": lse, "o": o, "kmean": km}
    if identity:
        _, _, _, rs, ap = ops.bwd_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, delta, causal, identity=True, ds32=ds32)
        out["rowsum_dS"], out["sum_abs_PdP"] = rs, ap
    return out
