"""A training step of the attention fed from host memory: forward + backward with the copies pipelined.

`attn_step_host` takes pinned CPU tensors, splits them into (batch, kv-head group) chunks (these problems are independent, so
the results are bit-identical to one un-chunked call) and runs three streams: host->device copies of chunk c + 1,
kernels of chunk c and device->host copies of chunk c - 1 overlap, which hides the compute and one direction of the
PCIe traffic behind the other.  The device work is the op sequence of `dm_attn_func` and its backward
(delta_matching_b200/attn.py; reference surface: delta_matching/__init__.py:52-77), with the same input checks.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_STREAMS = {}


def _side_streams(device):
    key = torch.device(device).index
    if key not in _STREAMS:
        _STREAMS[key] = (torch.cuda.Stream(device=device), torch.cuda.Stream(device=device))
    return _STREAMS[key]


def _check_host(name, t, pinned=True):
    if not isinstance(t, torch.Tensor) or t.dim() != 4:
        raise ValueError(f"delta_matching: {name} must be a 4-D tensor (batch, seqlen, nheads, headdim)")
    if t.device.type != "cpu":
        raise ValueError(f"delta_matching: {name} must be a CPU tensor (use dm_attn_func for CUDA tensors)")
    if t.dtype != torch.bfloat16:
        raise TypeError(f"delta_matching: {name} must be bfloat16")
    if not t.is_contiguous():
        raise ValueError(f"delta_matching: {name} must be contiguous")
    if pinned and not t.is_pinned():
        raise ValueError(f"delta_matching: {name} must be in pinned memory (tensor.pin_memory())")


def attn_step_host(q, k, v, do, *, causal=True, mode="matched", softmax_scale=None, chunks=None, out=None, device=None):
    """Forward and backward for host tensors.

    q, do: (B, N, H, D); k, v: (B, N, Hk, D); bf16, contiguous, pinned.  Returns (o, dq, dk, dv) as pinned CPU tensors
    (or fills `out`, a tuple of four such tensors).  The copies are asynchronous: the results are complete once the
    current CUDA stream of `device` has been synchronised.  `chunks` is how many slices are pipelined: up to the batch
    size they are batch ranges, beyond it (batch size times a divisor of nheads_k) ranges of kv-head groups of one batch,
    moved with strided copies; the default aims at eight.  Argument errors are those of `dm_attn_func`.

    Per chunk: q, k, v are copied in and the forward starts while dO is still on its way; O is copied out while the
    backward runs; dQ, dK, dV follow.  The kernels are the ones `dm_attn_func` and its backward launch, in the same
    order (the op layer is called directly, there is no autograd graph)."""
    from . import ops
    from .attn import _check_inputs
    for name, t in (("q", q), ("k", k), ("v", v), ("do", do)):
        _check_host(name, t)
    if do.shape != q.shape:
        raise ValueError("delta_matching: do must have the shape of q")
    if k.shape != v.shape or k.shape[0] != q.shape[0]:
        raise ValueError("delta_matching: k and v must have equal shapes and the batch size of q")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    B, N, H, D = q.shape
    Hk = k.shape[2]
    if Hk == 0 or H % Hk:
        raise ValueError(f"delta_matching: nheads ({H}) must be a positive multiple of nheads_k ({Hk})")
    rep = H // Hk
    if chunks is None:
        # about eight slices keep the pipeline's fill and drain short: whole batches if there are enough, else kv-group ranges
        split = 1
        while B * split < 8 and split * 2 <= Hk and Hk % (split * 2) == 0:
            split *= 2
        n_chunks = B * split if split > 1 else B
    else:
        n_chunks = int(chunks)
    if n_chunks < 1 or n_chunks > B * Hk or (n_chunks > B and (n_chunks % B or Hk % (n_chunks // B))):
        raise ValueError("delta_matching: chunks must be between 1 and the batch size, or the batch size times a divisor "
                         "of nheads_k")
    if out is None:
        out = tuple(torch.empty(t.shape, dtype=torch.bfloat16).pin_memory() for t in (q, q, k, v))
    else:
        for name, t, like in zip(("o", "dq", "dk", "dv"), out, (q, q, k, v)):
            _check_host(name, t)
            if t.shape != like.shape:
                raise ValueError(f"delta_matching: out tensor {name} has the wrong shape")
    # a chunk is (batch range, kv-group range): whole batches, or a range of kv-head groups of one batch
    if n_chunks <= B:
        units = [((B * c) // n_chunks, (B * (c + 1)) // n_chunks, 0, Hk) for c in range(n_chunks)]
    else:
        gs = Hk // (n_chunks // B)
        units = [(b, b + 1, g0, g0 + gs) for b in range(B) for g0 in range(0, Hk, gs)]
    nb = max(u[1] - u[0] for u in units)
    ng = max(u[3] - u[2] for u in units)
    L = _lib.lib()

    def copy(dev_t, host_t, b0, b1, h0, h1, to_device, stream):
        """host_t[b0:b1, :, h0:h1, :] <-> the leading (b1 - b0) batches of the dense device tensor dev_t."""
        heads, esz = host_t.shape[2], 2 * D
        if h0 == 0 and h1 == heads:
            rows, width, hpitch = (b1 - b0) * N, heads * esz, heads * esz
        else:
            rows, width, hpitch = N, (h1 - h0) * esz, heads * esz
        hptr = host_t.data_ptr() + (b0 * N * heads + h0) * esz
        if to_device:
            rc = L.dm_copy_2d_async(ctypes.c_void_p(dev_t.data_ptr()), width, ctypes.c_void_p(hptr), hpitch, width, rows, 1,
                                    ctypes.c_void_p(stream.cuda_stream))
        else:
            rc = L.dm_copy_2d_async(ctypes.c_void_p(hptr), hpitch, ctypes.c_void_p(dev_t.data_ptr()), width, width, rows, 0,
                                    ctypes.c_void_p(stream.cuda_stream))
        _lib.check(rc)

    with torch.cuda.device(dev), torch.no_grad():
        main = torch.cuda.current_stream(dev)
        s_in, s_out = _side_streams(dev)
        # two sets of device input buffers, allocated on the main stream; a chunk uses a dense leading part of each
        sizes = (nb * N * ng * rep * D, nb * N * ng * D, nb * N * ng * D, nb * N * ng * rep * D)
        bufs = [[torch.empty(n, dtype=torch.bfloat16, device=dev) for n in sizes] for _ in range(min(2, len(units)))]
        probe = torch.empty(1, dtype=torch.bfloat16, device=dev)       # shape-only views for the input contract
        _check_inputs(*(probe.expand(1, h, N, D) for h in (H, Hk, Hk)), causal, softmax_scale, mode)
        start = torch.cuda.Event()
        start.record(main)
        s_in.wait_event(start)
        s_out.wait_event(start)
        ev_done = []
        last_out = None
        for c, (b0, b1, g0, g1) in enumerate(units):
            n, hq, hg = b1 - b0, (g1 - g0) * rep, g1 - g0
            buf = bufs[c % len(bufs)]
            dq_, dk_, dv_, ddo_ = (t[: n * N * h * D].view(n, N, h, D) for t, h in zip(buf, (hq, hg, hg, hq)))
            if c >= len(bufs):
                s_in.wait_event(ev_done[c - len(bufs)])               # the kernels that read this buffer set are done
            copy(dq_, q, b0, b1, g0 * rep, g1 * rep, True, s_in)
            copy(dk_, k, b0, b1, g0, g1, True, s_in)
            copy(dv_, v, b0, b1, g0, g1, True, s_in)
            ev_qkv = torch.cuda.Event()
            ev_qkv.record(s_in)
            copy(ddo_, do, b0, b1, g0 * rep, g1 * rep, True, s_in)
            ev_do = torch.cuda.Event()
            ev_do.record(s_in)
            # forward as soon as q, k, v are on the device
            main.wait_event(ev_qkv)
            qh, kh, vh, doh = (t.transpose(1, 2) for t in (dq_, dk_, dv_, ddo_))
            q8, qs, k8, ks, v8, vs, _ = ops.quant_qkv(qh, kh, vh)
            o, lse = ops.fwd_fp8(q8, k8, v8, qs, ks, vs, causal)
            ev_fwd = torch.cuda.Event()
            ev_fwd.record(main)
            s_out.wait_event(ev_fwd)
            o.record_stream(s_out)
            copy(o, out[0], b0, b1, g0 * rep, g1 * rep, False, s_out)
            # backward once dO has arrived; O goes out meanwhile
            main.wait_event(ev_do)
            if mode == "matched":
                do8, dos, _ = ops.quant_do(doh, None)
                delta = ops.delta_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, causal)
            else:
                do8, dos, delta = ops.quant_do(doh, o.permute(0, 2, 1, 3))
            gq, gk, gv = ops.bwd_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, delta, causal)
            done = torch.cuda.Event()
            done.record(main)
            ev_done.append(done)
            s_out.wait_event(done)
            for t in (gq, gk, gv):
                t.record_stream(s_out)
            copy(gq, out[1], b0, b1, g0 * rep, g1 * rep, False, s_out)
            copy(gk, out[2], b0, b1, g0, g1, False, s_out)
            copy(gv, out[3], b0, b1, g0, g1, False, s_out)
            last_out = torch.cuda.Event()
            last_out.record(s_out)
        main.wait_event(last_out)
        for buf in bufs:
            for t in buf:
                t.record_stream(s_in)
    return out
