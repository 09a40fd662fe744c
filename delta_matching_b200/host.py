"""A training step of the attention fed from host memory: forward + backward with the copies pipelined.

`attn_step_host` takes pinned CPU tensors, splits the batch into chunks (the (batch, head) problems are independent, so
the results are bit-identical to one un-chunked call) and runs three streams: host->device copies of chunk c + 1,
kernels of chunk c and device->host copies of chunk c - 1 overlap, which hides the compute and one direction of the
PCIe traffic behind the other.  The device work is the op sequence of `dm_attn_func` and its backward
(delta_matching_b200/attn.py; reference surface: delta_matching/__init__.py:52-77), with the same input checks.
"""
from __future__ import annotations

import torch

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
    current CUDA stream of `device` has been synchronised.  `chunks` (default: the batch size) is how many slices of
    the batch are pipelined; argument errors are those of `dm_attn_func`.

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
    B = q.shape[0]
    n_chunks = B if chunks is None else int(chunks)
    if n_chunks < 1 or n_chunks > B:
        raise ValueError("delta_matching: chunks must be between 1 and the batch size")
    if out is None:
        out = tuple(torch.empty(t.shape, dtype=torch.bfloat16).pin_memory() for t in (q, q, k, v))
    else:
        for name, t, like in zip(("o", "dq", "dk", "dv"), out, (q, q, k, v)):
            _check_host(name, t)
            if t.shape != like.shape:
                raise ValueError(f"delta_matching: out tensor {name} has the wrong shape")
    bounds = [(B * c) // n_chunks for c in range(n_chunks + 1)]
    per = max(bounds[c + 1] - bounds[c] for c in range(n_chunks))

    with torch.cuda.device(dev), torch.no_grad():
        main = torch.cuda.current_stream(dev)
        s_in, s_out = _side_streams(dev)
        # two sets of device input buffers, allocated on the main stream
        bufs = [[torch.empty((per,) + tuple(t.shape[1:]), dtype=torch.bfloat16, device=dev) for t in (q, k, v, do)]
                for _ in range(min(2, n_chunks))]
        _check_inputs(*(t[:1].transpose(1, 2) for t in bufs[0][:3]), causal, softmax_scale, mode)
        start = torch.cuda.Event()
        start.record(main)
        s_in.wait_event(start)
        s_out.wait_event(start)
        ev_done = []
        last_out = None
        for c in range(n_chunks):
            lo, hi = bounds[c], bounds[c + 1]
            n = hi - lo
            buf = bufs[c % len(bufs)]
            with torch.cuda.stream(s_in):
                if c >= len(bufs):
                    s_in.wait_event(ev_done[c - len(bufs)])           # the kernels that read this buffer set are done
                for d_, h_ in zip(buf[:3], (q, k, v)):
                    d_[:n].copy_(h_[lo:hi], non_blocking=True)
                ev_qkv = torch.cuda.Event()
                ev_qkv.record(s_in)
                buf[3][:n].copy_(do[lo:hi], non_blocking=True)
                ev_do = torch.cuda.Event()
                ev_do.record(s_in)
            # forward as soon as q, k, v are on the device
            main.wait_event(ev_qkv)
            qh, kh, vh, doh = (t[:n].transpose(1, 2) for t in buf)
            q8, qs, k8, ks, v8, vs, _ = ops.quant_qkv(qh, kh, vh)
            o, lse = ops.fwd_fp8(q8, k8, v8, qs, ks, vs, causal)
            ev_fwd = torch.cuda.Event()
            ev_fwd.record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_fwd)
                o.record_stream(s_out)
                out[0][lo:hi].copy_(o, non_blocking=True)
            # backward once dO has arrived; O goes out meanwhile
            main.wait_event(ev_do)
            if mode == "matched":
                do8, dos, _ = ops.quant_do(doh, None)
                delta = ops.delta_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, causal)
            else:
                do8, dos, delta = ops.quant_do(doh, o.permute(0, 2, 1, 3))
            grads = ops.bwd_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, delta, causal)
            done = torch.cuda.Event()
            done.record(main)
            ev_done.append(done)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                for h_, d_ in zip(out[1:], grads):
                    d_.record_stream(s_out)
                    h_[lo:hi].copy_(d_, non_blocking=True)
                last_out = torch.cuda.Event()
                last_out.record(s_out)
        main.wait_event(last_out)
        for buf in bufs:
            for t in buf:
                t.record_stream(s_in)
    return out
