"""The op layer registered with torch.library, so that a tracing compiler sees five opaque ops with known output shapes
instead of ctypes calls it cannot look into.

    torch.ops.delta_matching_b200.quant_qkv(q, k, v)                     -> q8, qs, k8, ks, v8, vs, kmean
    torch.ops.delta_matching_b200.fwd_fp8(q8, k8, v8, qs, ks, vs, causal) -> O, LSE
    torch.ops.delta_matching_b200.quant_do(do, o, with_o)                -> do8, dos, delta
    torch.ops.delta_matching_b200.delta_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, causal, norm) -> delta
    torch.ops.delta_matching_b200.bwd_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, delta, causal, ds32) -> dq, dk, dv

The reference registers the same roles as real ops (csrc/delta_matching_api.cpp:683-715: fwd_fp8, delta_fp8, bwd_fp8_t)
and its autograd function calls them through torch.ops (delta_matching/attn.py:37-118), which is what lets its API run
under torch.compile without a graph break (tests/test_api.py:304-317).  The implementations are the functions of
delta_matching_b200.ops (CUDA only; there is no CPU implementation to fall back to); the fake implementations only
state shapes, dtypes and devices.  Tensors are in the op layer's layout: inputs (B, H, N, D) views, codes (B, H, N, D)
e4m3, scales (B, H, N // 32) fp32, O / dQ (B, N, H, D), dK / dV (B, N, Hk, D) bf16.
"""
from __future__ import annotations

from typing import Tuple

import torch
from torch import Tensor

from . import ops

NS = "delta_matching_b200"
E4M3 = torch.float8_e4m3fn
F32 = torch.float32
BF16 = torch.bfloat16


def _quant_qkv(q: Tensor, k: Tensor, v: Tensor) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    return ops.quant_qkv(q, k, v)


quant_qkv = torch.library.custom_op(f"{NS}::quant_qkv", _quant_qkv, mutates_args=(), device_types="cuda")


@quant_qkv.register_fake
def _(q, k, v):
    B, H, N, D = q.shape
    Hk = k.shape[1]
    code = lambda h: q.new_empty((B, h, N, D), dtype=E4M3)
    scale = lambda h: q.new_empty((B, h, N // ops.BLK), dtype=F32)
    return code(H), scale(H), code(Hk), scale(Hk), code(Hk), scale(Hk), q.new_empty((B, Hk, D), dtype=F32)


def _fwd_fp8(q8: Tensor, k8: Tensor, v8: Tensor, qs: Tensor, ks: Tensor, vs: Tensor, causal: bool) -> Tuple[Tensor, Tensor]:
    return ops.fwd_fp8(q8, k8, v8, qs, ks, vs, causal)


fwd_fp8 = torch.library.custom_op(f"{NS}::fwd_fp8", _fwd_fp8, mutates_args=(), device_types="cuda")


@fwd_fp8.register_fake
def _(q8, k8, v8, qs, ks, vs, causal):
    B, H, N, D = q8.shape
    return q8.new_empty((B, N, H, D), dtype=BF16), q8.new_empty((B, H, N), dtype=F32)


def _quant_do(do: Tensor, o: Tensor, with_o: bool) -> Tuple[Tensor, Tensor, Tensor]:
    """with_o: also return the stale delta rowsum(dO * O); otherwise `o` is not read and delta comes back empty."""
    do8, dos, delta = ops.quant_do(do, o if with_o else None)
    if delta is None:
        delta = do.new_empty((0,), dtype=F32)
    return do8, dos, delta


quant_do = torch.library.custom_op(f"{NS}::quant_do", _quant_do, mutates_args=(), device_types="cuda")


@quant_do.register_fake
def _(do, o, with_o):
    B, H, N, D = do.shape
    delta = do.new_empty((B, H, N) if with_o else (0,), dtype=F32)
    return do.new_empty((B, H, N, D), dtype=E4M3), do.new_empty((B, H, N // ops.BLK), dtype=F32), delta


def _delta_fp8(q8: Tensor, k8: Tensor, v8: Tensor, do8: Tensor, qs: Tensor, ks: Tensor, vs: Tensor, dos: Tensor,
               lse: Tensor, causal: bool, norm: bool) -> Tensor:
    return ops.delta_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, causal, norm)


delta_fp8 = torch.library.custom_op(f"{NS}::delta_fp8", _delta_fp8, mutates_args=(), device_types="cuda")


@delta_fp8.register_fake
def _(q8, k8, v8, do8, qs, ks, vs, dos, lse, causal, norm):
    return torch.empty_like(lse)


def _bwd_fp8(q8: Tensor, k8: Tensor, v8: Tensor, do8: Tensor, qs: Tensor, ks: Tensor, vs: Tensor, dos: Tensor,
             lse: Tensor, delta: Tensor, causal: bool, ds32: bool) -> Tuple[Tensor, Tensor, Tensor]:
    return ops.bwd_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, delta, causal, ds32=ds32)


bwd_fp8 = torch.library.custom_op(f"{NS}::bwd_fp8", _bwd_fp8, mutates_args=(), device_types="cuda")


@bwd_fp8.register_fake
def _(q8, k8, v8, do8, qs, ks, vs, dos, lse, delta, causal, ds32):
    B, H, N, D = q8.shape
    Hk = k8.shape[1]
    return (q8.new_empty((B, N, H, D), dtype=BF16), q8.new_empty((B, N, Hk, D), dtype=BF16),
            q8.new_empty((B, N, Hk, D), dtype=BF16))


class _Direct:
    """The same five calls without the dispatcher in between: what the eager path uses (a registered op costs tens of
    microseconds of host time per call, which shows once the kernels of a step take about two milliseconds)."""
    quant_qkv = staticmethod(_quant_qkv)
    fwd_fp8 = staticmethod(_fwd_fp8)
    quant_do = staticmethod(_quant_do)
    delta_fp8 = staticmethod(_delta_fp8)
    bwd_fp8 = staticmethod(_bwd_fp8)


DIRECT = _Direct
