"""Benchmark of the fp8 attention forward + backward (matched mode) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c2_small]

One step = one pass of the whole composition through the public API (producers, forward, dO producer, matched-delta
pass 0, backward) over one batch of synthetic input.  Workload (per GPU): the GQA causal matched Llama-3-8B-layer shape
B=4, N=4096, H=32, Hk=8, D=128, bf16 q / k / v / dO drawn i.i.d. N(0, 1) from a seed.  With N > 1 GPUs every rank runs
the same-sized shard of (batch, kv-group) units on its own seed, with no collective on the data path (weak scaling).

Counted FLOPs per step (the metric's convention): 4 B H N^2 D forward + 2.5 x that backward, halved for causal; the
matched-delta pass 0 (one more forward's worth of matmuls) and the producers are not counted.

Prints ONE JSON line (rank 0).  `value` is timed with CUDA events on the launching stream with inputs resident in HBM;
`e2e` is the same step fed from pinned host memory with every result copied back.  `--impl reference` times the CPU
restatement of the reference's emulation (oracle/) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "fp8 attn fwd+bwd TFLOPS/GPU & % of fp8 tensor peak, hd128 causal matched"
WORKLOADS = {
    "c2": dict(B=4, N=4096, H=32, Hk=8, D=128),
    "c2_small": dict(B=2, N=4096, H=8, Hk=2, D=128),       # for profiler captures only; never a bench value
}
FP8_NOMINAL_TFLOPS = 4500.0


def counted_flops(B, N, H, D, causal=True):
    f = 14.0 * B * H * N * N * D
    return f / 2 if causal else f


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        return json.load(open(p)), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """SM clock, power and clock-event reasons of one GPU, read through NVML from a thread every few milliseconds while
    the timed region runs (read-only queries; nothing on the GPU is set).  CUDA_VISIBLE_DEVICES is honoured."""
    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))

    def __init__(self, index, period_s=0.005):
        self.index, self.period = index, period_s
        self.samples, self.thread, self.stop, self.max_mhz = [], None, False, None

    def _physical_index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [x.strip() for x in vis.split(",") if x.strip()]
            if self.index < len(ids) and ids[self.index].isdigit():
                return int(ids[self.index])
        return self.index

    def _run(self, nv, handle):
        while not self.stop:
            try:
                self.samples.append((nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM),
                                     nv.nvmlDeviceGetPowerUsage(handle) / 1000.0,
                                     nv.nvmlDeviceGetCurrentClocksEventReasons(handle)))
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            handle = nv.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._run, args=(nv, handle), daemon=True)
            self.thread.start()
        except Exception:
            self.thread = None
        return self

    def __exit__(self, *a):
        self.stop = True
        if self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self):
        out = {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": len(self.samples)}
        if self.samples:
            sm = [float(s[0]) for s in self.samples]
            busy = [x for x in sm if x > 0.5 * max(sm)] or sm
            out["sm_mhz"] = statistics.median(busy)
            out["power_w_median"] = statistics.median(s[1] for s in self.samples)
            mask = 0
            for s in self.samples:
                mask |= int(s[2])
            out["reasons"] = sorted(name for name, bit in self.REASONS if mask & bit)
        return out


def make_inputs(w, device, seed):
    g = torch.Generator(device=device).manual_seed(seed)
    B, N, H, Hk, D = w["B"], w["N"], w["H"], w["Hk"], w["D"]
    return [torch.randn(B, N, h, D, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
            for h in (H, Hk, Hk, H)]


def timed(fn, steps, stream):
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(steps):
        fn()
    end.record(stream)
    end.synchronize()
    return start.elapsed_time(end) / steps          # ms per step


def fp8_matmul_tflops(device):
    """A cuBLASLt e4m3 8192^3 matmul, best of 5 (context for the fp8 peak; never a denominator of `value`)."""
    try:
        n = 8192
        a = torch.randn(n, n, device=device).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=device).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=device)
        f = lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        for _ in range(3):
            f()
        best = min(timed(f, 1, torch.cuda.current_stream()) for _ in range(5))
        return 2.0 * n ** 3 / (best * 1e-3) / 1e12
    except Exception:
        return None


def cpu_sample(w, steps=1, warmup=0):
    """The oracle (the reference's emulation restated) on ONE (batch, kv-group) unit of the workload, all host threads."""
    from oracle import dm_oracle as orc
    torch.set_num_threads(os.cpu_count() or 1)
    rep = w["H"] // w["Hk"]
    q, k, v, do = orc.make_inputs(1, w["N"], rep, 1, w["D"], seed=0)
    flops = counted_flops(1, w["N"], rep, w["D"])
    for _ in range(warmup):
        orc.dm_oracle(q, k, v, do, True, "matched")
    ts = []
    for _ in range(steps):
        t0 = time.perf_counter()
        orc.dm_oracle(q, k, v, do, True, "matched")
        ts.append(time.perf_counter() - t0)
    dt = statistics.median(ts)
    sample = f"1 of {w['B'] * w['Hk']} (batch, kv-group) units: B=1 N={w['N']} H={rep} Hk=1 D={w['D']} causal matched"
    return flops / dt / 1e12, dt * 1e3, torch.get_num_threads(), sample


def run_reference(args, w, rank):
    if rank != 0:
        return
    tf, ms, cores, sample = cpu_sample(w, steps=args.steps, warmup=min(args.warmup, 1))
    line = {"impl": "reference", "metric": METRIC, "value": tf, "unit": "TFLOPS", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp8_e4m3 (emulated in fp32)", "data": "synthetic",
            "config": {"workload": args.workload + " " + json.dumps(w), "sample": sample},
            "cpu_baseline": {"value": tf, "unit": "TFLOPS", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": tf, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    emit(line)


_RESULT_FD = None


def own_stdout():
    """Libraries (NCCL's version banner, build tools) write to file descriptor 1; the contract is one JSON line there.  Keep
    a private duplicate of the real stdout for that line and point descriptor 1 at stderr for everything else."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(line):
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def main():
    own_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return run_reference(args, w, rank)

    import torch.distributed as dist
    import delta_matching_b200 as dm
    from delta_matching_b200 import build, ops
    build.build()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    warmup = max(args.warmup, 3)
    q, k, v, do = make_inputs(w, dev, seed=1234 + rank)
    leaves = [t.detach().requires_grad_() for t in (q, k, v)]
    stream = torch.cuda.current_stream()

    def step():
        for t in leaves:
            t.grad = None
        o = dm.dm_attn_func(*leaves, causal=True, mode="matched")
        o.backward(do)
        return o

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step()
    barrier()
    ops.check_status(dev)
    with ClockSampler(local) as clk:
        barrier()
        ms = timed(step, args.steps, stream)
        barrier()
    t = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    ops.check_status(dev)
    flops = counted_flops(w["B"], w["N"], w["H"], w["D"])
    value = world * flops / (ms * 1e-3) / 1e12
    launches_per_step = 10        # k-mean partial + fold, 3 quantisers, forward, dO quantiser, pass 0, dK/dV, dQ

    # ------------------------------------------------------------------ per-kernel times (same stream, CUDA events)
    qh, kh, vh, doh = (x.transpose(1, 2) for x in (q, k, v, do))
    q8, qs, k8, ks, v8, vs, _ = ops.quant_qkv(qh, kh, vh)
    o, lse = ops.fwd_fp8(q8, k8, v8, qs, ks, vs, True)
    do8, dos, _ = ops.quant_do(doh, None)
    delta = ops.delta_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, True)
    # the two backward kernels share the dS workspace: pass 1 (dK / dV) writes it, pass 2 (dQ) streams it
    ws_bytes = ops.bwd_workspace_bytes(w["B"], w["N"], w["H"], w["D"])
    ws = torch.empty(ws_bytes, device=dev, dtype=torch.uint8) if ws_bytes > 0 else None
    parts = {
        "producers_qkv": lambda: ops.quant_qkv(qh, kh, vh),
        "forward": lambda: ops.fwd_fp8(q8, k8, v8, qs, ks, vs, True),
        "producer_do": lambda: ops.quant_do(doh, None),
        "pass0_delta": lambda: ops.delta_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, True),
        "bwd_dkdv": lambda: ops.bwd_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, delta, True, parts=1, workspace=ws),
        "bwd_dq": lambda: ops.bwd_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, delta, True, parts=2, workspace=ws),
    }
    kernel_ms = {}
    for name, fn in parts.items():
        fn()
        torch.cuda.synchronize()
        kernel_ms[name] = timed(fn, max(3, args.steps), stream)
    ops.check_status(dev)
    unit = 2.0 * w["B"] * w["H"] * w["N"] * w["N"] * w["D"] / 2      # one N x N x D matmul over all heads, causal
    kernel_flops = {"forward": 2 * unit, "pass0_delta": 2 * unit, "bwd_dkdv": 4 * unit,
                    "bwd_dq": (1 if ws is not None else 3) * unit}     # pass 2 executes one matmul per tile
    dominant = max(kernel_flops, key=lambda n: kernel_ms[n])
    peaks, peak_src = measured_peaks()
    fp8_peak = 2.0 * peaks["bf16_tflops_sustained"]
    ach = kernel_flops[dominant] / (kernel_ms[dominant] * 1e-3) / 1e12
    roofline = {"bound": "tensor", "kernel": dominant, "achieved": ach, "peak": fp8_peak, "unit": "TFLOP/s",
                "frac": ach / fp8_peak, "traffic": None,
                "peak_source": f"2 x bf16_tflops_sustained of MEASURED_PEAKS.json ({peak_src}); fp8 issues at twice the bf16 rate",
                "flops_per_launch": kernel_flops[dominant], "ms_per_launch": kernel_ms[dominant],
                "frac_of_nominal_4500": ach / FP8_NOMINAL_TFLOPS}

    # ------------------------------------------------------------------ end to end from pinned host memory
    e2e = None
    if not args.no_e2e:
        host_in = [x.detach().cpu().pin_memory() for x in (q, k, v, do)]
        dev_in = [torch.empty_like(x) for x in (q, k, v, do)]
        host_out = [torch.empty(x.shape, dtype=torch.bfloat16).pin_memory() for x in (q, q, k, v)]   # o, dq, dk, dv

        from delta_matching_b200.host import attn_step_host

        def step_serial():                       # copy in, compute, copy out on one stream: nothing overlaps
            for d_, h_ in zip(dev_in, host_in):
                d_.copy_(h_, non_blocking=True)
            lv = [t.detach().requires_grad_() for t in dev_in[:3]]
            o_ = dm.dm_attn_func(*lv, causal=True, mode="matched")
            o_.backward(dev_in[3])
            for h_, d_ in zip(host_out, (o_.detach(), lv[0].grad, lv[1].grad, lv[2].grad)):
                h_.copy_(d_, non_blocking=True)

        def step_e2e():                          # the host-memory API: batch chunks pipelined over three streams
            attn_step_host(*host_in, causal=True, mode="matched", out=host_out)

        for _ in range(2):
            step_serial()
            step_e2e()
        barrier()
        ms_serial = timed(step_serial, max(3, args.steps // 2), stream)
        barrier()
        ms_e = timed(step_e2e, args.steps, stream)
        barrier()
        te = torch.tensor([ms_e], device=dev)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        ms_e = float(te.item())
        e2e = {"value": world * flops / (ms_e * 1e-3) / 1e12, "unit": "TFLOPS", "ms_per_step": ms_e,
               "h2d_bytes_per_step": sum(x.numel() * 2 for x in host_in),
               "d2h_bytes_per_step": sum(x.numel() * 2 for x in host_out),
               "api": "delta_matching_b200.host.attn_step_host (pinned host tensors in and out, (batch, kv-group range) chunks pipelined)",
               "ms_per_step_unpipelined": ms_serial}
    ops.check_status(dev)

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps, "warmup": warmup,
                "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
                "config": {"workload": args.workload + " per GPU: " + json.dumps(w) + " causal matched, bf16 q/k/v/dO i.i.d. N(0,1)",
                           "parallelism": f"{world} x (batch, kv-group) shards, no collective", "l2": "inputs (320 MB) larger than L2"},
                "per_gpu_tflops": value / world, "pct_of_fp8_nominal_peak": 100.0 * value / world / FP8_NOMINAL_TFLOPS,
                "pct_of_fp8_measured_peak": 100.0 * value / world / fp8_peak,
                "kernel_ms": kernel_ms, "roofline": roofline, "clocks": clk.summary(), "e2e": e2e,
                "gpu_launches": launches_per_step * args.steps}
        fp8_mm = fp8_matmul_tflops(dev)
        if fp8_mm is not None:
            line["fp8_matmul_tflops_cublaslt_8192"] = fp8_mm
        if world == 1 and not args.no_cpu_baseline:
            tf, cms, cores, sample = cpu_sample(w)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOPS", "cores": cores, "kind": "port", "sample": sample,
                                    "ms_per_sample": cms}
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
