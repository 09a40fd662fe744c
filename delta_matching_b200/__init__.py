"""delta_matching_b200: the fp8 attention forward and backward of delta-matching, built for NVIDIA B200 (sm_100a).

The same Python surface as the reference package (delta_matching/__init__.py:44-77):

    from delta_matching_b200 import dm_attn_func
    o = dm_attn_func(q, k, v, causal=True, mode="matched")     # q (B, N, H, D), k / v (B, N, Hk, D), bf16, CUDA
    o = dm_attn_func(q, k, v, causal=True, mode="stale")

Constraints: self-attention; head_dim 128 (seqlen % 256 == 0) or 256 (seqlen % 128 == 0); bf16; softmax_scale =
head_dim ** -0.5; mode "matched" needs causal=True.  Violations raise ValueError / TypeError / NotImplementedError.
`dm_attn_func_bhnd` takes (B, H, N, D) and returns (B, N, H, D).  `flash_attn_func` has flash-attention 2's signature
and refuses the arguments the kernels do not implement.  All work runs in hand-written CUDA for sm_100a behind the C
ABI of include/dm_b200.h; there is no fallback path.
"""
from __future__ import annotations

import os as _os

import torch

from .attn import blocks, dm_attn_func_bhnd, dm_attn_debug

__version__ = "0.1.0"
# the quantisation contract the kernels implement, by head dim: the reference's Blackwell presets
# (delta_matching/reference.py:612-613, 629)
KERNEL_NUMERICS = {"128": "sm100-mx", "256": "sm100-mx-d256"}
# every numerics arm the kernels implement (values of dm_attn_func's `numerics`; reference.py:613-630)
NUMERICS_ARMS = ("sm100-mx", "sm100-mx-d256", "sm100-mx-ds32", "sm100-mx-d256-ds32", "sm100-mx-nonorm")
FA_SRC_COMMIT = "none (from-scratch sm_100a build)"
CUTLASS_COMMIT = "none (from-scratch sm_100a build)"
__all__ = ["dm_attn_func", "dm_attn_func_bhnd", "dm_attn_func_plain", "flash_attn_func", "blocks", "kernel_version",
           "__version__", "KERNEL_NUMERICS", "NUMERICS_ARMS"]

# The reference keeps a second "plain" route as a cross-check of its Triton producers (delta_matching/core.py:178-271);
# there is one producer implementation here, so the name is an alias.
dm_attn_func_plain = dm_attn_func_bhnd


def dm_attn_func(q, k, v, softmax_scale=None, causal=False, mode="matched", numerics="sm100-mx"):
    """Attention in the flash-attention layout: q (B, N, H, D), k / v (B, N, Hk, D) bf16 on CUDA -> o (B, N, H, D) bf16.
    mode: "matched" (the Delta-Matching backward; needs causal=True) or "stale" (delta = rowsum(dO * O)).
    numerics: "sm100-mx" (the contract; "sm100-mx-d256" names it at head_dim 256) or another arm of the reference
    emulation's preset table that the kernels implement: "sm100-mx-ds32" / "sm100-mx-d256-ds32" (dS scaled per
    32 x 32 block) and "sm100-mx-nonorm" (matched delta without the division by sum P); see NUMERICS_ARMS."""
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not isinstance(t, torch.Tensor) or t.dim() != 4:
            raise ValueError(f"delta_matching: {name} must be a 4-D tensor (batch, seqlen, nheads, headdim)")
    return dm_attn_func_bhnd(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), causal=causal,
                             softmax_scale=softmax_scale, delta_mode=mode, numerics=numerics)


def flash_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1), softcap=0.0,
                    alibi_slopes=None, deterministic=False, return_attn_probs=False, mode="matched"):
    """flash_attn.flash_attn_func's signature for one-line ports; the arguments the kernels do not implement must be at
    their defaults.  `deterministic` is accepted and ignored: every output is deterministic."""
    if dropout_p != 0.0:
        raise NotImplementedError("delta_matching: dropout is not implemented (dropout_p must be 0)")
    if tuple(window_size) != (-1, -1):
        raise NotImplementedError("delta_matching: sliding windows are not implemented (window_size must be (-1, -1))")
    if softcap != 0.0:
        raise NotImplementedError("delta_matching: softcap is not implemented")
    if alibi_slopes is not None:
        raise NotImplementedError("delta_matching: alibi_slopes are not implemented")
    if return_attn_probs:
        raise NotImplementedError("delta_matching: return_attn_probs is not implemented")
    return dm_attn_func(q, k, v, softmax_scale=softmax_scale, causal=causal, mode=mode)


def kernel_version():
    """A stamp for training logs: package version, a content hash of the kernel sources, the numerics contract and,
    once the library is loaded, its path (keys as delta_matching/__init__.py:80-104)."""
    from . import _lib, build
    info = {"version": __version__, "code_sha": build.code_sha(), "fa_src_commit": FA_SRC_COMMIT,
            "numerics": dict(KERNEL_NUMERICS), "numerics_arms": list(NUMERICS_ARMS), "bf16_dp": False}
    if _lib.loaded_library() is not None:
        info["library"] = _lib.loaded_library()
    return info
