"""A training step of the attention fed from host memory: forward + backward with the copies pipelined.

`attn_step_host` takes pinned CPU tensors, splits the batch into chunks (the (batch, head) problems are independent, so
the results are bit-identical to one un-chunked call) and runs three streams: host->device copies of chunk c + 1,
kernels of chunk c and device->host copies of chunk c - 1 overlap, which hides the compute and one direction of the
PCIe traffic behind the other.  Everything on the device goes through `dm_attn_func` and autograd, i.e. the same path
as a call with CUDA tensors (reference surface: delta_matching/__init__.py:52-77).
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
    the batch are pipelined; argument errors are those of `dm_attn_func`."""
    from . import dm_attn_func
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

    with torch.cuda.device(dev):
        main = torch.cuda.current_stream(dev)
        s_in, s_out = _side_streams(dev)
        # two sets of device input buffers, allocated on the main stream
        bufs = [[torch.empty((per,) + tuple(t.shape[1:]), dtype=torch.bfloat16, device=dev) for t in (q, k, v, do)]
                for _ in range(min(2, n_chunks))]
        start = torch.cuda.Event()
        start.record(main)
        s_in.wait_event(start)
        s_out.wait_event(start)
        ev_done = []
        last_out = None
        for c in range(n_chunks):
            lo, hi = bounds[c], bounds[c + 1]
            buf = bufs[c % len(bufs)]
            with torch.cuda.stream(s_in):
                if c >= len(bufs):
                    s_in.wait_event(ev_done[c - len(bufs)])           # the kernels that read this buffer set are done
                for d_, h_ in zip(buf, (q, k, v, do)):
                    d_[: hi - lo].copy_(h_[lo:hi], non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(s_in)
            main.wait_event(ev_in)
            leaves = [t[: hi - lo].detach().requires_grad_() for t in buf[:3]]
            o = dm_attn_func(*leaves, softmax_scale=softmax_scale, causal=causal, mode=mode)
            o.backward(buf[3][: hi - lo])
            results = (o.detach(), leaves[0].grad, leaves[1].grad, leaves[2].grad)
            done = torch.cuda.Event()
            done.record(main)
            ev_done.append(done)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                for h_, d_ in zip(out, results):
                    d_.record_stream(s_out)
                    h_[lo:hi].copy_(d_, non_blocking=True)
                last_out = torch.cuda.Event()
                last_out.record(s_out)
        main.wait_event(last_out)
        for buf in bufs:
            for t in buf:
                t.record_stream(s_in)
    return out
