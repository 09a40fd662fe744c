"""The op layer: torch tensors in, torch tensors out, the work done by the C ABI (include/dm_b200.h).

These functions take the place of `torch.ops.delta_matching.{fwd_fp8, delta_fp8, bwd_fp8_t}` (schemas at
csrc/delta_matching_api.cpp:683-715) and of the producers `quant_qkv2` / `quant_do_delta`
(delta_matching/sm100/quant.py:278-341).  Conventions kept from the reference: outputs are allocated by the op with
torch's allocator and returned, the call runs on the tensors' device and that device's current stream, and misuse
raises RuntimeError before any launch.  Layout here: codes (B, H, N, D) float8_e4m3fn, scales (B, H, N // 32) fp32.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib

E4M3 = torch.float8_e4m3fn
BLK = 32                                  # tokens per quantisation scale
DS_BLOCK32 = 4                            # DM_DS_BLOCK32 of include/dm_b200.h: flag bit beside the parts of the backward
# Numerics arms: name of the reference emulation's preset (delta_matching/reference.py:613-630) -> (dS scale per
# 32 x 32 block instead of 128 x 32, matched delta divided by sum P).  The first is the reference's Blackwell contract and
# the default; the head_dim-256 presets name the same schemes.
NUMERICS = {
    "sm100-mx": (False, True),
    "sm100-mx-d256": (False, True),
    "sm100-mx-ds32": (True, True),
    "sm100-mx-d256-ds32": (True, True),
    "sm100-mx-nonorm": (False, False),
}
_STATUS = {}                              # device index -> int32 status word (pinned host memory the kernels write)
_DEBUG = os.environ.get("DM_DEBUG", "0") not in ("", "0")

STATUS_TEXT = {1: "TMA producer gave up waiting for a free stage", 2: "MMA issuer gave up waiting",
               3: "compute warps gave up waiting for an accumulator", 4: "probe kernel gave up waiting"}


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _stream(t):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _require(cond, msg):
    if not cond:
        raise RuntimeError("delta_matching: " + msg)


def _cuda(*ts):
    dev = None
    for t in ts:
        if t is None:
            continue
        _require(isinstance(t, torch.Tensor) and t.is_cuda, "every tensor must be a CUDA tensor")
        _require(t.numel() > 0, "empty tensor")
        dev = dev or t.device
        _require(t.device == dev, "every tensor must be on the same device")
    return dev


def _dev_index(device) -> int:
    idx = torch.device(device).index
    return torch.cuda.current_device() if idx is None else idx


def status_word(device) -> torch.Tensor:
    """The per-device int32 word the kernels set when a bounded wait runs out (0 = no problem).  It lives in pinned host
    memory, which the GPU writes directly (pinned allocations are mapped into the device's address space under unified
    addressing), so the host reads it without a copy and without a synchronisation."""
    idx = _dev_index(device)
    w = _STATUS.get(idx)
    if w is None:
        with torch.cuda.device(idx):
            w = _STATUS[idx] = torch.zeros(1, dtype=torch.int32).pin_memory()
    return w


def _raise_if_set(idx: int) -> None:
    w = _STATUS.get(idx)
    if w is None:
        return
    v = int(w[0])
    if v != 0:
        w[0] = 0
        raise RuntimeError(f"delta_matching: a kernel on cuda:{idx} reported status {v} "
                           f"({STATUS_TEXT.get(v, 'unknown')}); its outputs are invalid")


def check_status(device=None) -> None:
    """Synchronise `device` (every device used so far when None) and raise RuntimeError if one of its kernels reported a
    timed-out wait since the last check."""
    devs = [_dev_index(device)] if device is not None else list(_STATUS)
    for idx in devs:
        if idx in _STATUS:
            torch.cuda.synchronize(idx)
            _raise_if_set(idx)


def _enter(device):
    """At the entry of every op: a plain read of the pinned status word, no synchronisation.  A kernel that gave up
    earlier on this device makes the next op raise instead of consuming its output."""
    _raise_if_set(_dev_index(device))


def _after(device):
    if _DEBUG and not torch.cuda.is_current_stream_capturing():
        check_status(device)


def launch_count() -> int:
    """Kernel launches the library has made in this process (counted by the library's launchers)."""
    return int(_lib.lib().dm_launch_count())


def _rows(x):
    """(B, H, N, D) bf16 view with a unit stride on D and 16-byte aligned rows (copied otherwise)."""
    if x.stride(-1) != 1 or any(s % 8 for s in x.stride()[:-1]) or x.data_ptr() % 16:
        x = x.contiguous()
    return x


# ------------------------------------------------------------------------------------------------------------ producers
def kmean(k: torch.Tensor) -> torch.Tensor:
    """k (B, Hk, N, D) bf16 -> (B, Hk, D) fp32 mean over tokens (fixed summation order)."""
    dev = _cuda(k)
    _enter(dev)
    _require(k.dim() == 4 and k.dtype == torch.bfloat16, "k must be a 4-D bfloat16 tensor")
    k = _rows(k)
    B, Hk, N, D = k.shape
    L = _lib.lib()
    with torch.cuda.device(dev):
        mean = torch.empty(B, Hk, D, device=dev, dtype=torch.float32)
        ws = torch.empty(max(1, L.dm_quant_qkv_workspace_bytes(B, N, Hk, D)), device=dev, dtype=torch.uint8)
        _lib.check(L.dm_kmean(_ptr(k), k.stride(0), k.stride(1), k.stride(2), B, N, Hk, D, _ptr(mean), _ptr(ws), _stream(k)))
    return mean


def quant_rows(x: torch.Tensor, prescale: float = 1.0, mean: torch.Tensor | None = None, o: torch.Tensor | None = None):
    """x (B, H, N, D) bf16 -> (codes (B, H, N, D) e4m3, scales (B, H, N // 32) fp32[, delta (B, H, N) fp32 if o given]).
    y = (x - mean[b, h]) * prescale is quantised; delta = sum_d x * o on the raw values."""
    dev = _cuda(x, mean, o)
    _enter(dev)
    _require(x.dim() == 4 and x.dtype == torch.bfloat16, "input must be a 4-D bfloat16 tensor")
    x = _rows(x)
    B, H, N, D = x.shape
    L = _lib.lib()
    with torch.cuda.device(dev):
        codes = torch.empty(B, H, N, D, device=dev, dtype=E4M3)
        scales = torch.empty(B, H, N // BLK, device=dev, dtype=torch.float32)
        delta = None
        os_ = (0, 0, 0)
        if o is not None:
            _require(o.shape == x.shape and o.dtype == torch.bfloat16, "o must match dO (bfloat16, same shape)")
            o = _rows(o)
            os_ = (o.stride(0), o.stride(1), o.stride(2))
            delta = torch.empty(B, H, N, device=dev, dtype=torch.float32)
        if mean is not None:
            _require(mean.dtype == torch.float32 and tuple(mean.shape) == (B, H, D), "mean must be fp32 (B, H, D)")
            mean = mean.contiguous()
        _lib.check(L.dm_quant_rows(_ptr(x), x.stride(0), x.stride(1), x.stride(2), _ptr(mean), float(prescale),
                                   _ptr(o), *os_, B, N, H, D, _ptr(codes), _ptr(scales), _ptr(delta), _stream(x)))
    return (codes, scales, delta) if o is not None else (codes, scales)


def quant_qkv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor):
    """q (B, H, N, D), k / v (B, Hk, N, D) bf16 -> (q8, qs, k8, ks, v8, vs, kmean).  q is scaled by D^-0.5, k is centred
    by its per-(batch, kv head) mean over tokens (returned as kmean (B, Hk, D) fp32)."""
    dev = _cuda(q, k, v)
    _enter(dev)
    for t in (q, k, v):
        _require(t.dim() == 4 and t.dtype == torch.bfloat16, "q, k, v must be 4-D bfloat16 tensors")
    q, k, v = _rows(q), _rows(k), _rows(v)
    B, H, N, D = q.shape
    Hk = k.shape[1]
    L = _lib.lib()
    with torch.cuda.device(dev):
        e = lambda h: torch.empty(B, h, N, D, device=dev, dtype=E4M3)
        s = lambda h: torch.empty(B, h, N // BLK, device=dev, dtype=torch.float32)
        q8, k8, v8, qs, ks, vs = e(H), e(Hk), e(Hk), s(H), s(Hk), s(Hk)
        km = torch.empty(B, Hk, D, device=dev, dtype=torch.float32)
        ws = torch.empty(max(1, L.dm_quant_qkv_workspace_bytes(B, N, Hk, D)), device=dev, dtype=torch.uint8)
        _lib.check(L.dm_quant_qkv(_ptr(q), q.stride(0), q.stride(1), q.stride(2),
                                  _ptr(k), k.stride(0), k.stride(1), k.stride(2),
                                  _ptr(v), v.stride(0), v.stride(1), v.stride(2),
                                  B, N, H, Hk, D, _ptr(q8), _ptr(k8), _ptr(v8), _ptr(qs), _ptr(ks), _ptr(vs), _ptr(km),
                                  _ptr(ws), _stream(q)))
    return q8, qs, k8, ks, v8, vs, km


def quant_do(do: torch.Tensor, o: torch.Tensor | None = None):
    """dO (B, H, N, D) bf16 [+ O, same logical shape] -> (dO8, dOs, delta | None); delta = rowsum(dO * O) (stale mode)."""
    if o is None:
        c, s = quant_rows(do)
        return c, s, None
    return quant_rows(do, 1.0, None, o)


# ------------------------------------------------------------------------------------------------------------ kernels
def _check_codes(B, H, Hk, N, D, q8, k8, v8, qs, ks, vs, do8=None, dos=None):
    for name, t, h in (("q8", q8, H), ("k8", k8, Hk), ("v8", v8, Hk), ("do8", do8, H)):
        if t is None:
            continue
        _require(t.dtype == E4M3, f"{name} must be float8_e4m3fn (e4m3 codes)")
        _require(tuple(t.shape) == (B, h, N, D) and t.is_contiguous(), f"{name} must be contiguous (B, H, N, D)")
    for name, t, h in (("q scales", qs, H), ("k scales", ks, Hk), ("v scales", vs, Hk), ("dO scales", dos, H)):
        if t is None:
            continue
        _require(t.dtype == torch.float32, f"{name} must be fp32")
        _require(tuple(t.shape) == (B, h, N // BLK) and t.is_contiguous(), f"{name} must be contiguous (B, H, N // 32)")


def fwd_fp8(q8, k8, v8, qs, ks, vs, causal: bool, unordered: bool = False):
    """-> (O (B, N, H, D) bf16 contiguous, LSE (B, H, N) fp32 natural log).  Replaces the fwd_fp8 op.  unordered=True is
    the test hook dm_dbg_fwd_unordered (same results, one ordering wait per key tile fewer)."""
    dev = _cuda(q8, k8, v8, qs, ks, vs)
    _enter(dev)
    _require(q8.dim() == 4 and k8.dim() == 4, "codes must be 4-D")
    B, H, N, D = q8.shape
    Hk = k8.shape[1]
    _check_codes(B, H, Hk, N, D, q8, k8, v8, qs, ks, vs)
    L = _lib.lib()
    with torch.cuda.device(dev):
        o = torch.empty(B, N, H, D, device=dev, dtype=torch.bfloat16)
        lse = torch.empty(B, H, N, device=dev, dtype=torch.float32)
        fn = L.dm_dbg_fwd_unordered if unordered else L.dm_fwd
        _lib.check(fn(_ptr(q8), _ptr(k8), _ptr(v8), _ptr(qs), _ptr(ks), _ptr(vs), B, N, H, Hk, D, int(bool(causal)),
                      _ptr(o), o.stride(0), o.stride(1), o.stride(2), _ptr(lse), _ptr(status_word(dev)), _stream(q8)))
        _after(dev)
    return o, lse


def delta_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, causal: bool, norm: bool = True):
    """-> matched delta (B, H, N) fp32 from pass 0 of the backward.  Replaces the delta_fp8 op.
    norm=False leaves out the division by sum_j P_ij (numerics arm "sm100-mx-nonorm", see NUMERICS)."""
    dev = _cuda(q8, k8, v8, do8, qs, ks, vs, dos, lse)
    _enter(dev)
    B, H, N, D = q8.shape
    Hk = k8.shape[1]
    _check_codes(B, H, Hk, N, D, q8, k8, v8, qs, ks, vs, do8, dos)
    _require(lse.dtype == torch.float32 and tuple(lse.shape) == (B, H, N) and lse.is_contiguous(), "lse must be fp32 (B, H, N)")
    L = _lib.lib()
    with torch.cuda.device(dev):
        delta = torch.empty(B, H, N, device=dev, dtype=torch.float32)
        fn = L.dm_delta if norm else L.dm_delta_sum
        _lib.check(fn(_ptr(q8), _ptr(k8), _ptr(v8), _ptr(do8), _ptr(qs), _ptr(ks), _ptr(vs), _ptr(dos), _ptr(lse),
                      B, N, H, Hk, D, int(bool(causal)), _ptr(delta), _ptr(status_word(dev)), _stream(q8)))
        _after(dev)
    return delta


def bwd_workspace_bytes(B: int, N: int, H: int, D: int) -> int:
    """Bytes of the dS workspace of the two-pass backward (0: the shape is not one the kernels take)."""
    return int(_lib.lib().dm_bwd_workspace_bytes(int(B), int(N), int(H), int(D)))


_SMALL_WS = 4 << 30


def _workspace_cap_bytes(device=None, need: int = 0) -> int:
    """Bound of the dS workspace of one backward call: DM_BWD_WORKSPACE_MB (MiB; 0 selects the backward that recomputes
    instead of storing), else the reference's own knob DM_BWD_WS_LIMIT_GB (delta_matching/split.py:37-97 bounds the same
    buffer by splitting the call per head group), else 4 GiB when the whole call needs no more than that (no query of the
    device: the common training shapes stay on this path), else 60 % of the device memory that is free or held idle by
    torch's caching allocator, so that on a 180 GB GPU many (batch, kv-group) units of a long context share one launch."""
    try:
        if "DM_BWD_WORKSPACE_MB" in os.environ:
            return int(os.environ["DM_BWD_WORKSPACE_MB"]) << 20
        if "DM_BWD_WS_LIMIT_GB" in os.environ:
            return int(float(os.environ["DM_BWD_WS_LIMIT_GB"]) * (1 << 30))
    except ValueError:
        pass
    if need <= _SMALL_WS:
        return _SMALL_WS
    if device is None or torch.cuda.is_current_stream_capturing():
        return 16384 << 20
    free, _ = torch.cuda.mem_get_info(device)
    idle = torch.cuda.memory_reserved(device) - torch.cuda.memory_allocated(device)
    return max(_SMALL_WS, int(0.6 * (free + idle)))


_MAX_WS_TILES = (1 << 24) - 1


def plan_workspace_ranges(B: int, Hk: int, rep: int, n_t: int, group_bytes: int, cap: int):
    """(batch start, batch end, kv-group start, kv-group end) ranges of one two-pass backward call each, such that the
    dS workspace of a range (group_bytes per (batch, kv group)) stays within `cap` bytes and its tile count within the
    limit of one call: whole batches when a batch fits, else kv-group ranges of one batch (at least one group)."""
    def even(total, fit):
        """`total` items in the fewest ranges of at most `fit`, the ranges as equal as possible (a last range with a
        single unit would leave most SMs idle for its whole launch)."""
        n = -(-total // fit)
        return [(total * i // n, total * (i + 1) // n) for i in range(n)]

    groups_fit = max(1, min(Hk, cap // group_bytes, _MAX_WS_TILES // (rep * n_t * n_t)))
    if groups_fit >= Hk:
        bs = max(1, min(B, cap // (group_bytes * Hk), _MAX_WS_TILES // (rep * Hk * n_t * n_t)))
        return [(b0, b1, 0, Hk) for b0, b1 in even(B, bs)]
    return [(b, b + 1, g0, g1) for b in range(B) for g0, g1 in even(Hk, groups_fit)]


def bwd_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, delta, causal: bool, identity: bool = False, parts: int = 3,
            workspace=None, ds32: bool = False):
    """-> (dq (B, N, H, D), dk (B, N, Hk, D), dv (B, N, Hk, D)) bf16; dk / dv are already reduced over the GQA group.
    identity=True also returns (rowsum_dS, sum_abs_PdP), fp32 (B, H, N), accumulated in the kernel before dS is
    quantised.  parts: 1 = only the dK / dV kernel, 2 = only the dQ kernel, 3 = both (the outputs of a kernel that did
    not run are uninitialised).  Replaces the bwd_fp8_t op and the group fold of delta_matching/attn.py:114-117.
    ds32=True scales dS per (32 queries x 32 keys) instead of (128 x 32) (numerics arm "sm100-mx-ds32", see NUMERICS).

    Without the identity probe the two-pass form runs: the dK / dV kernel leaves the dS codes in a workspace and dQ
    streams them (bit-identical to the recomputing kernel).  The workspace is allocated here unless
    `workspace` (uint8, at least bwd_workspace_bytes) is given; when it would exceed DM_BWD_WORKSPACE_MB the call is
    split over (batch, kv-head group) ranges, and when a single group exceeds it the recomputing kernel runs."""
    dev = _cuda(q8, k8, v8, do8, qs, ks, vs, dos, lse, delta)
    _enter(dev)
    B, H, N, D = q8.shape
    Hk = k8.shape[1]
    _check_codes(B, H, Hk, N, D, q8, k8, v8, qs, ks, vs, do8, dos)
    for name, t in (("lse", lse), ("delta", delta)):
        _require(t.dtype == torch.float32 and tuple(t.shape) == (B, H, N) and t.is_contiguous(), f"{name} must be fp32 (B, H, N)")
    L = _lib.lib()
    _require(parts in (1, 2, 3), "parts must be 1 (dK/dV), 2 (dQ) or 3")
    flags = int(parts) | (DS_BLOCK32 if ds32 else 0)
    rep = H // Hk
    n_t = N // 128
    group_bytes = bwd_workspace_bytes(1, N, rep, D)
    cap = _workspace_cap_bytes(dev, group_bytes * B * Hk)
    two_pass = (not identity and group_bytes > 0 and (workspace is not None or group_bytes <= cap)
                and rep * n_t * n_t <= _MAX_WS_TILES)
    with torch.cuda.device(dev):
        dq = torch.empty(B, N, H, D, device=dev, dtype=torch.bfloat16)
        dk = torch.empty(B, N, Hk, D, device=dev, dtype=torch.bfloat16)
        dv = torch.empty(B, N, Hk, D, device=dev, dtype=torch.bfloat16)
        rs = torch.empty(B, H, N, device=dev, dtype=torch.float32) if identity else None
        ap = torch.empty(B, H, N, device=dev, dtype=torch.float32) if identity else None
        st = _ptr(status_word(dev))
        if not two_pass:
            _lib.check(L.dm_bwd_parts(_ptr(q8), _ptr(k8), _ptr(v8), _ptr(do8), _ptr(qs), _ptr(ks), _ptr(vs), _ptr(dos),
                                      _ptr(lse), _ptr(delta), B, N, H, Hk, D, int(bool(causal)),
                                      _ptr(dq), dq.stride(0), dq.stride(1), dq.stride(2),
                                      _ptr(dk), dk.stride(0), dk.stride(1), dk.stride(2),
                                      _ptr(dv), dv.stride(0), dv.stride(1), dv.stride(2),
                                      _ptr(rs), _ptr(ap), flags, st, _stream(q8)))
        else:
            if workspace is not None:
                _require(workspace.dtype == torch.uint8 and workspace.is_contiguous() and workspace.device == dev,
                         "workspace must be a contiguous uint8 CUDA tensor on the inputs' device")
                cap = workspace.numel()
            ranges = plan_workspace_ranges(B, Hk, rep, n_t, group_bytes, cap)
            need = max(bwd_workspace_bytes(b1 - b0, N, (g1 - g0) * rep, D) for b0, b1, g0, g1 in ranges)
            if workspace is None:
                workspace = torch.empty(need, device=dev, dtype=torch.uint8)
            _require(workspace.numel() >= need, f"workspace of {workspace.numel()} bytes given, {need} needed")
            for b0, b1, g0, g1 in ranges:
                hs = slice(g0 * rep, g1 * rep)
                gsl = slice(g0, g1)
                v_q8, v_do8, v_qs, v_dos = q8[b0:b1, hs], do8[b0:b1, hs], qs[b0:b1, hs], dos[b0:b1, hs]
                v_k8, v_v8, v_ks, v_vs = k8[b0:b1, gsl], v8[b0:b1, gsl], ks[b0:b1, gsl], vs[b0:b1, gsl]
                v_lse, v_delta = lse[b0:b1, hs], delta[b0:b1, hs]
                # either whole batches (all heads) or head ranges of one batch: every view is dense
                v_dq, v_dk, v_dv = dq[b0:b1, :, hs], dk[b0:b1, :, gsl], dv[b0:b1, :, gsl]
                _lib.check(L.dm_bwd_ws(_ptr(v_q8), _ptr(v_k8), _ptr(v_v8), _ptr(v_do8), _ptr(v_qs), _ptr(v_ks), _ptr(v_vs),
                                       _ptr(v_dos), _ptr(v_lse), _ptr(v_delta), b1 - b0, N, (g1 - g0) * rep, g1 - g0, D,
                                       int(bool(causal)),
                                       _ptr(v_dq), dq.stride(0), dq.stride(1), dq.stride(2),
                                       _ptr(v_dk), dk.stride(0), dk.stride(1), dk.stride(2),
                                       _ptr(v_dv), dv.stride(0), dv.stride(1), dv.stride(2),
                                       _ptr(workspace), workspace.numel(), flags, st, _stream(q8)))
        _after(dev)
    return (dq, dk, dv, rs, ap) if identity else (dq, dk, dv)


def mma_tile(a, b, sfa=None, sfb=None, a_tmem=False, a_mn=False, b_mn=False, nk=4):
    """One 128 x 128 x (32 nk) tile product through the kernels' operand paths (see dm_dbg_mma_tile); a, b uint8 /
    e4m3 (128, 128); sfa / sfb int32 (128, 4) scale words select the block-scaled instruction."""
    dev = _cuda(a, b, sfa, sfb)
    _enter(dev)
    L = _lib.lib()
    with torch.cuda.device(dev):
        out = torch.empty(128, 128, device=dev, dtype=torch.float32)
        _lib.check(L.dm_dbg_mma_tile(_ptr(a), _ptr(b), _ptr(sfa), _ptr(sfb), int(a_tmem), int(a_mn), int(b_mn),
                                     int(sfa is not None), int(nk), _ptr(out), _ptr(status_word(dev)), _stream(a)))
    return out


def wait_expiry_probe(a, b, limit_us: int = 100):
    """Launch the one-tile kernel with the arrival its threads wait for left out and `limit_us` as the limit of that wait
    (dm_dbg_wait_expiry): the kernel returns by itself and leaves status 4 in the device's status word.  -> the (unwritten)
    output tensor.  Used by the tests to show the give-up path end to end."""
    dev = _cuda(a, b)
    L = _lib.lib()
    with torch.cuda.device(dev):
        out = torch.zeros(128, 128, device=dev, dtype=torch.float32)
        _lib.check(L.dm_dbg_wait_expiry(_ptr(a), _ptr(b), _ptr(out), int(limit_us) * 1000, _ptr(status_word(dev)), _stream(a)))
    return out
