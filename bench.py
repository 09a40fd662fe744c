"""Benchmark of the fp8 attention forward + backward on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload auto|c2|c3|c4|c5|c2_small]

One step = one pass of the whole composition through the public API (producers, forward, dO producer, matched-delta
pass 0 or stale delta, backward) over one batch of synthetic input.  Workloads (bf16 inputs drawn from a seed):

    c2  B=4 N=4096  H=32 Hk=8  D=128 causal matched, q k v dO i.i.d. N(0,1)       the headline shape (one GPU)
    c3  B=2 N=8192  H=16 Hk=16 D=256 causal matched
    c4  B=8 N=2048  H=16 Hk=16 D=128 non-causal stale, q and k multiplied by s in {1, 3, 10, 30}
    c5  B=8 N=32768 H=64 Hk=8  D=128 causal matched, q k rows at unit RMS; the 64 (batch, kv-group) units are split
        over the ranks (strong scaling), unit u drawn from seed + u on the rank that owns it

`--workload auto` (default) is c2 on one GPU and c5 on several.  With one GPU the line also carries short runs of c3, c4
and c5 under "configs" and of c2 under the other numerics arms under "numerics_arms" (drop them with --no-extra).  There is no collective on the data path; after the timed region
the ranks all_gather one 64-bit hash and one fp64 sum per unit of (O, dQ, dK, dV) for validation.

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
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "fp8 attn fwd+bwd TFLOPS/GPU & % of fp8 tensor peak, hd128 causal matched"
WORKLOADS = {
    "c2": dict(B=4, N=4096, H=32, Hk=8, D=128, causal=True, mode="matched"),
    "c2_small": dict(B=2, N=4096, H=8, Hk=2, D=128, causal=True, mode="matched"),   # profiler captures only
    "c3": dict(B=2, N=8192, H=16, Hk=16, D=256, causal=True, mode="matched"),
    "c4": dict(B=8, N=2048, H=16, Hk=16, D=128, causal=False, mode="stale", sweep=(1.0, 3.0, 10.0, 30.0)),
    "c5": dict(B=8, N=32768, H=64, Hk=8, D=128, causal=True, mode="matched", unit_rms=True, sharded=True),
}
FP8_NOMINAL_TFLOPS = 4500.0
SEED = 1234
# DRAM bytes (read + written) per live 128 x 128 tile position of the dK/dV kernel: one ncu capture of one launch on
# c2_small (dram__bytes_read.sum 21.79 MB + dram__bytes_write.sum 89.94 MB over 8448 tile positions; the summary is in
# profiles/), scaled to a launch by its tile count (traffic grows with the tile count: per position one 16 KiB dS tile
# is written for pass 2, of which about a third was still in L2 when the captured kernel ended, and the Q / dO / K / V
# tiles are read mostly from L2).
DKDV_DRAM_BYTES_PER_TILE = 13148.0


def counted_flops(B, N, H, D, causal=True):
    f = 14.0 * B * H * N * N * D
    return f / 2 if causal else f


def live_tiles(w):
    n_t = w["N"] // 128
    per_head = n_t * (n_t + 1) // 2 if w["causal"] else n_t * n_t
    return w["B"] * w["H"] * per_head


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


def make_inputs(w, device, seed, qk_scale=1.0):
    """q, k, v, dO in (B, N, H | Hk, D) layout, drawn in that order from one generator (the reference's benchmark inputs,
    benchmarks/bench.py:28-32); q and k are multiplied by qk_scale before the bf16 cast."""
    g = torch.Generator(device=device).manual_seed(seed)
    B, N, H, Hk, D = w["B"], w["N"], w["H"], w["Hk"], w["D"]
    out = []
    for h, s in ((H, qk_scale), (Hk, qk_scale), (Hk, 1.0), (H, 1.0)):
        x = torch.randn(B, N, h, D, generator=g, device=device, dtype=torch.float32)
        out.append((x * s if s != 1.0 else x).to(torch.bfloat16))
    return out


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


# ---------------------------------------------------------------------------------------------------- CPU baseline
def _cpu_time(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(steps):
        t0 = time.perf_counter()
        fn()
        ts.append(time.perf_counter() - t0)
    return statistics.median(ts)


def cpu_sample(w, steps=1, warmup=0):
    """The oracle (the reference's emulation restated) on ONE (batch, kv-group) unit of the workload, all host threads.
    The sequence is capped at 4096 tokens (the emulation is O(N^2) on CPU), which the sample text says."""
    from oracle import dm_oracle as orc
    torch.set_num_threads(os.cpu_count() or 1)
    rep = w["H"] // w["Hk"]
    n = min(w["N"], 4096)
    q, k, v, do = orc.make_inputs(1, n, rep, 1, w["D"], seed=0, unit_rms=bool(w.get("unit_rms")))
    flops = counted_flops(1, n, rep, w["D"], w["causal"])
    dt = _cpu_time(lambda: orc.dm_oracle(q, k, v, do, w["causal"], w["mode"]), steps, warmup)
    sample = (f"1 of {w['B'] * w['Hk']} (batch, kv-group) units: B=1 N={n} H={rep} Hk=1 D={w['D']} "
              f"{'causal' if w['causal'] else 'non-causal'} {w['mode']}" + ("" if n == w["N"] else f" (N cut from {w['N']})"))
    return flops / dt / 1e12, dt * 1e3, torch.get_num_threads(), sample


def cpu_config1():
    """The reference's own CPU-runnable case (B=1 N=256 H=Hk=2 D=128 causal, seed 0) in both delta modes: one warm-up
    call, median of 5."""
    from oracle import dm_oracle as orc
    torch.set_num_threads(os.cpu_count() or 1)
    q, k, v, do = orc.make_inputs(1, 256, 2, 2, 128, seed=0)
    flops = counted_flops(1, 256, 2, 128)
    out = {}
    for mode in ("matched", "stale"):
        dt = _cpu_time(lambda: orc.dm_oracle(q, k, v, do, True, mode), 5, 1)
        out[mode] = {"ms": dt * 1e3, "gflops": flops / dt / 1e9}
    return out


def run_reference(args, name, w, rank):
    if rank != 0:
        return
    tf, ms, cores, sample = cpu_sample(w, steps=args.steps, warmup=min(args.warmup, 1))
    line = {"impl": "reference", "metric": METRIC, "value": tf, "unit": "TFLOPS", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong" if w.get("sharded") else "weak", "vs_baseline": None,
            "dtype": "fp8_e4m3 (emulated in fp32)", "data": "synthetic",
            "config": {"workload": name + " " + json.dumps(w), "sample": sample},
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


# ---------------------------------------------------------------------------------------------------- GPU arms
class Job:
    """One workload on this rank: inputs, the step through the public API, counted FLOPs of the whole job."""

    def __init__(self, name, w, dev, rank, world, qk_scale=1.0, numerics="sm100-mx"):
        import delta_matching_b200 as dm
        self.numerics = numerics
        from delta_matching_b200 import shard
        self.name, self.w, self.dev, self.world = name, w, dev, world
        self.dm = dm
        self.sharded = bool(w.get("sharded"))
        if self.sharded:
            self.units = shard.unit_range(w["B"], w["Hk"], world, rank)
            self.rep = w["H"] // w["Hk"]
            self.q, self.k, self.v, self.do = shard.make_unit_inputs(self.units, w["N"], self.rep, w["D"], SEED, dev,
                                                                     unit_rms=bool(w.get("unit_rms")))
            self.job_flops = counted_flops(w["B"], w["N"], w["H"], w["D"], w["causal"])          # all ranks together
        else:
            self.q, self.k, self.v, self.do = make_inputs(w, dev, SEED + rank, qk_scale)
            self.job_flops = world * counted_flops(w["B"], w["N"], w["H"], w["D"], w["causal"])  # one replica per rank
        self.leaves = [t.detach().requires_grad_() for t in (self.q, self.k, self.v)]
        self.o = None

    def step(self):
        for t in self.leaves:
            t.grad = None
        self.o = self.dm.dm_attn_func(*self.leaves, causal=self.w["causal"], mode=self.w["mode"], numerics=self.numerics)
        self.o.backward(self.do)

    def outputs(self):
        return self.o.detach(), self.leaves[0].grad, self.leaves[1].grad, self.leaves[2].grad

    def input_bytes(self):
        return sum(t.numel() * 2 for t in (self.q, self.k, self.v, self.do))


def run_timed(job, steps, warmup, barrier, allmax, clock_index=None):
    """warm-up, then `steps` steps between two barriers, CUDA events on the launching stream, max over ranks."""
    from delta_matching_b200 import ops
    stream = torch.cuda.current_stream()
    for _ in range(warmup):
        job.step()
    barrier()
    ops.check_status(job.dev)
    if clock_index is None:
        barrier()
        ms = timed(job.step, steps, stream)
        barrier()
        clocks = None
    else:
        with ClockSampler(clock_index) as clk:
            barrier()
            ms = timed(job.step, steps, stream)
            barrier()
        clocks = clk.summary()
    ms = allmax(ms)
    ops.check_status(job.dev)
    return ms, clocks


def validate_units(job, world, rank):
    """Per-unit hashes of (O, dQ, dK, dV) gathered over the ranks (NCCL all_gather, after the timed region), plus one
    cross-check: rank 0 recomputes the LAST unit of the job (owned by the last rank when there are several) alone, as a
    batch of one, and compares its hash with the gathered one: the same unit gives the same bits on another GPU, in
    another shard size."""
    from delta_matching_b200 import shard
    w = job.w
    h, s = shard.unit_hashes(*job.outputs())
    H, S = shard.gather_unit_hashes(h, s, world)
    out = None
    if rank == 0:
        last = w["B"] * w["Hk"] - 1
        q, k, v, do = shard.make_unit_inputs([last], w["N"], job.rep, w["D"], SEED, job.dev, unit_rms=bool(w.get("unit_rms")))
        lv = [t.requires_grad_() for t in (q, k, v)]
        o = job.dm.dm_attn_func(*lv, causal=w["causal"], mode=w["mode"])
        o.backward(do)
        h1, _ = shard.unit_hashes(o.detach(), lv[0].grad, lv[1].grad, lv[2].grad)
        out = {"unit_hashes": [f"{int(x) & 0xFFFFFFFFFFFFFFFF:016x}" for x in H.tolist()],
               "unit_sums": [float(x) for x in S.tolist()],
               "recomputed_unit": last, "recomputed_unit_matches": bool(int(h1[0]) == int(H[last])),
               "all_finite": bool(torch.isfinite(S).all().item())}
    return out


def kernel_breakdown(job, steps, first_units=None):
    """Each kernel of the step timed alone (CUDA events, same stream), and its roofline: tensor kernels by executed
    matmul FLOPs against 2 x the measured bf16 burst rate, HBM kernels by algorithmic bytes against the measured copy
    bandwidth.  first_units: take only that many leading batch entries of the rank's inputs (long-context shards)."""
    from delta_matching_b200 import ops
    w, dev = job.w, job.dev
    stream = torch.cuda.current_stream()
    causal, matched = w["causal"], w["mode"] == "matched"
    src = (job.q, job.k, job.v, job.do) if first_units is None else tuple(t[:first_units] for t in (job.q, job.k, job.v, job.do))
    qh, kh, vh, doh = (x.transpose(1, 2) for x in src)
    q8, qs, k8, ks, v8, vs, _ = ops.quant_qkv(qh, kh, vh)
    o, lse = ops.fwd_fp8(q8, k8, v8, qs, ks, vs, causal)
    if matched:
        do8, dos, _ = ops.quant_do(doh, None)
        delta = ops.delta_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, causal)
    else:
        do8, dos, delta = ops.quant_do(doh, o.permute(0, 2, 1, 3))
    B, H, N, D = q8.shape
    ws_bytes = ops.bwd_workspace_bytes(B, N, H, D)
    ws = torch.empty(ws_bytes, device=dev, dtype=torch.uint8) if 0 < ws_bytes <= (48 << 30) else None
    parts = {
        "producers_qkv": lambda: ops.quant_qkv(qh, kh, vh),
        "forward": lambda: ops.fwd_fp8(q8, k8, v8, qs, ks, vs, causal),
        # the same kernel without the wait that orders S(i + 1) behind the scale-word reads of PV(i): what the ordering costs
        "forward_unordered_hook": lambda: ops.fwd_fp8(q8, k8, v8, qs, ks, vs, causal, unordered=True),
        "producer_do": (lambda: ops.quant_do(doh, None)) if matched else (lambda: ops.quant_do(doh, o.permute(0, 2, 1, 3))),
        "bwd_dkdv": lambda: ops.bwd_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, delta, causal, parts=1, workspace=ws),
        "bwd_dq": lambda: ops.bwd_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, delta, causal, parts=2, workspace=ws),
    }
    if matched:
        parts["pass0_delta"] = lambda: ops.delta_fp8(q8, k8, v8, do8, qs, ks, vs, dos, lse, causal)
    kernel_ms = {}
    for name, fn in parts.items():
        fn()
        torch.cuda.synchronize()
        kernel_ms[name] = timed(fn, max(3, steps), stream)
    ops.check_status(dev)
    tiles = live_tiles(dict(w, B=B, H=H))
    unit = 2.0 * 128 * 128 * D * tiles               # one matmul over every live tile
    two_pass = ws is not None
    hd256 = D == 256
    # matmuls executed per tile: dK/dV 4 (head_dim 256: a dV launch with S^T, dV and a dK launch with S^T, dP^T, dK = 5),
    # dQ 1 streaming / 3 recomputing
    kernel_flops = {"forward": 2 * unit, "bwd_dkdv": (5 if hd256 else 4) * unit,
                    "bwd_dq": (1 if two_pass else 3) * unit}
    if matched:
        kernel_flops["pass0_delta"] = 2 * unit
    peaks, peak_src = measured_peaks()
    burst, sustained = 2.0 * peaks["bf16_tflops"], 2.0 * peaks["bf16_tflops_sustained"]
    hbm = peaks["hbm_gbs"]
    rooflines = []
    for name, fl in kernel_flops.items():
        ach = fl / (kernel_ms[name] * 1e-3) / 1e12
        rooflines.append({"kernel": name, "bound": "tensor", "achieved": ach, "peak": burst, "unit": "TFLOP/s",
                          "frac": ach / burst, "flops_per_launch": fl, "ms_per_launch": kernel_ms[name]})
    eq, ek = B * H * N * D, B * k8.shape[1] * N * D
    hbm_bytes = {"producers_qkv": 3.0 * eq + 5.0 * ek + 3.0 * ek,          # q: 2 in + 1 out; k: read twice (mean) + 1 out
                 "producer_do": (3.0 if matched else 5.0) * eq}
    if two_pass:
        hbm_bytes["bwd_dq"] = tiles * (16384.0 + 4.0) + 2.0 * eq            # dS tiles streamed once + dQ written
    for name, by in hbm_bytes.items():
        ach = by / (kernel_ms[name] * 1e-3) / 1e9
        rooflines.append({"kernel": name, "bound": "hbm", "achieved": ach, "peak": hbm, "unit": "GB/s", "frac": ach / hbm,
                          "bytes_per_launch": by, "ms_per_launch": kernel_ms[name]})
    dominant = max(kernel_flops, key=lambda n: kernel_ms[n])
    dom = next(r for r in rooflines if r["kernel"] == dominant and r["bound"] == "tensor")
    roofline = {"bound": "tensor", "kernel": dominant, "achieved": dom["achieved"], "peak": burst, "unit": "TFLOP/s",
                "frac": dom["frac"],
                "traffic": (DKDV_DRAM_BYTES_PER_TILE * tiles if (dominant == "bwd_dkdv" and DKDV_DRAM_BYTES_PER_TILE) else None),
                "peak_source": f"2 x bf16_tflops of MEASURED_PEAKS.json ({peak_src}): the burst figure, because kernel_ms times "
                               "a kernel alone in a short loop; fp8 issues at twice the bf16 rate",
                "peak_sustained": sustained,
                "flops_per_launch": kernel_flops[dominant], "ms_per_launch": kernel_ms[dominant],
                "frac_of_nominal_4500": dom["achieved"] / FP8_NOMINAL_TFLOPS}
    executed = sum(kernel_flops.values())
    return kernel_ms, roofline, rooflines, executed


def sustained_leg(job, seconds, ms_hint, clock_index, executed_flops):
    """The same step looped for at least `seconds` (the power state a training run lives in), with the clocks sampled."""
    stream = torch.cuda.current_stream()
    n = max(10, int(seconds * 1e3 / max(ms_hint, 1e-3)) + 1)
    with ClockSampler(clock_index, period_s=0.02) as clk:
        torch.cuda.synchronize()
        ms = timed(job.step, n, stream)
        torch.cuda.synchronize()
    c = clk.summary()
    peaks, _ = measured_peaks()
    sus = 2.0 * peaks["bf16_tflops_sustained"]
    tf_exec = executed_flops / (ms * 1e-3) / 1e12
    return {"steps": n, "seconds": n * ms * 1e-3, "ms_per_step": ms, "value": job.job_flops / job.world / (ms * 1e-3) / 1e12,
            "unit": "TFLOPS counted per GPU", "executed_tflops": tf_exec, "frac_sustained": tf_exec / sus,
            "peak_sustained": sus, "sm_mhz_median": c.get("sm_mhz"), "power_w_median": c.get("power_w_median"),
            "reasons": c.get("reasons"), "ms_x_mhz": (ms * c["sm_mhz"]) if c.get("sm_mhz") else None}


def e2e_leg(job, steps, barrier, allmax):
    """The step through delta_matching_b200.host.attn_step_host: pinned host tensors in and out, copies inside the timed
    region; next to it the un-pipelined form (copy in, compute, copy out on one stream)."""
    from delta_matching_b200.host import attn_step_host
    w = job.w
    stream = torch.cuda.current_stream()
    host_in = [x.detach().cpu().pin_memory() for x in (job.q, job.k, job.v, job.do)]
    host_out = [torch.empty(x.shape, dtype=torch.bfloat16).pin_memory() for x in (job.q, job.q, job.k, job.v)]

    def step_e2e():
        attn_step_host(*host_in, causal=w["causal"], mode=w["mode"], out=host_out)

    for _ in range(2):
        step_e2e()
    barrier()
    ms_e = allmax(timed(step_e2e, steps, stream))
    barrier()
    out = {"value": job.job_flops / (ms_e * 1e-3) / 1e12, "unit": "TFLOPS", "ms_per_step": ms_e,
           "h2d_bytes_per_step": sum(x.numel() * 2 for x in host_in),
           "d2h_bytes_per_step": sum(x.numel() * 2 for x in host_out),
           "api": "delta_matching_b200.host.attn_step_host (pinned host tensors in and out, (batch, kv-group range) "
                  "chunks pipelined over three streams)"}
    if job.input_bytes() <= (2 << 30):
        dev_in = [torch.empty_like(x) for x in (job.q, job.k, job.v, job.do)]
        dev_out = [torch.empty_like(x) for x in (job.q, job.q, job.k, job.v)]
        side = torch.cuda.Stream()

        def copies_only():
            # the step's PCIe traffic alone: inputs in on one stream while the outputs of the previous step go out on
            # another (dense copies, no kernels): the floor of the end-to-end figure on this host
            side.wait_stream(stream)
            with torch.cuda.stream(side):
                for h_, d_ in zip(host_out, dev_out):
                    h_.copy_(d_, non_blocking=True)
            for d_, h_ in zip(dev_in, host_in):
                d_.copy_(h_, non_blocking=True)
            stream.wait_stream(side)

        copies_only()
        barrier()
        out["ms_per_step_copies_only"] = allmax(timed(copies_only, max(3, steps // 2), stream))
        barrier()

        def step_serial():
            for d_, h_ in zip(dev_in, host_in):
                d_.copy_(h_, non_blocking=True)
            lv = [t.detach().requires_grad_() for t in dev_in[:3]]
            o_ = job.dm.dm_attn_func(*lv, causal=w["causal"], mode=w["mode"])
            o_.backward(dev_in[3])
            for h_, d_ in zip(host_out, (o_.detach(), lv[0].grad, lv[1].grad, lv[2].grad)):
                h_.copy_(d_, non_blocking=True)

        step_serial()
        barrier()
        out["ms_per_step_unpipelined"] = timed(step_serial, max(3, steps // 2), stream)
        barrier()
    return out


def short_run(name, dev, steps=5, warmup=3):
    """A short single-GPU run of another configuration for the "configs" record of the one-GPU line."""
    from delta_matching_b200 import ops
    w = WORKLOADS[name]
    ident = lambda x: x
    nobar = torch.cuda.synchronize
    res = {"workload": {k: v for k, v in w.items() if k != "sweep"}}
    if "sweep" in w:
        res["sweep"] = {}
        for s in w["sweep"]:
            job = Job(name, w, dev, 0, 1, qk_scale=s)
            ms, _ = run_timed(job, steps, warmup, nobar, ident)
            res["sweep"][f"s={s:g}"] = {"ms_per_step": ms, "value": job.job_flops / (ms * 1e-3) / 1e12}
            del job
        res["value"] = statistics.mean(v["value"] for v in res["sweep"].values())
    else:
        job = Job(name, w, dev, 0, 1)
        ms, _ = run_timed(job, steps, warmup, nobar, ident)
        res.update(ms_per_step=ms, value=job.job_flops / (ms * 1e-3) / 1e12)
        if job.sharded:
            res["validation"] = validate_units(job, 1, 0)
        elif job.input_bytes() <= (2 << 30):
            km, roof, _, _ = kernel_breakdown(job, steps)
            res["kernel_ms"] = km
            res["roofline"] = {k: roof[k] for k in ("kernel", "achieved", "peak", "frac", "unit")}
        del job
    res["unit"] = "TFLOPS"
    res["pct_of_fp8_nominal_peak"] = 100.0 * res["value"] / FP8_NOMINAL_TFLOPS
    res["steps"], res["warmup"] = steps, warmup
    ops.check_status(dev)
    torch.cuda.empty_cache()
    return res


def main():
    own_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="auto", choices=["auto"] + sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the short runs of the other configurations and the sustained leg")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    name = args.workload if args.workload != "auto" else ("c2" if max(world, args.gpus) == 1 else "c5")
    w = WORKLOADS[name]
    if args.impl == "reference":
        return run_reference(args, name, w, rank)

    import torch.distributed as dist
    from delta_matching_b200 import build, ops
    build.build()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    warmup = max(args.warmup, 3)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def allmax(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sweep = w.get("sweep")
    job = Job(name, w, dev, rank, world, qk_scale=(sweep[0] if sweep else 1.0))
    launches0 = ops.launch_count()
    ms, clocks = run_timed(job, args.steps, warmup, barrier, allmax, clock_index=local)
    launches = (ops.launch_count() - launches0) * args.steps // (args.steps + warmup)
    value = job.job_flops / (ms * 1e-3) / 1e12
    validation = validate_units(job, world, rank) if job.sharded else None

    small = job.input_bytes() <= (2 << 30)
    # per-kernel times: on the whole workload when it is small, else on the rank's first (batch, kv-group) unit
    kernel_ms, roofline, rooflines, executed = kernel_breakdown(job, min(args.steps, 10) if not small else args.steps,
                                                                 first_units=None if small else 1)
    if not small:
        roofline["scope"] = "one (batch, kv-group) unit of the shard, timed alone"
    sustained = None
    if small and world == 1 and not args.no_extra:
        sustained = sustained_leg(job, 2.5, ms, local, executed)
        roofline["frac_sustained"] = sustained["frac_sustained"]
    e2e = None if args.no_e2e else e2e_leg(job, args.steps, barrier, allmax)
    ops.check_status(dev)

    if rank == 0:
        peaks, _ = measured_peaks()
        shape = {k: v for k, v in w.items() if k not in ("sweep", "sharded")}
        if job.sharded:
            par = (f"{world} rank(s) x {len(job.units)} of {w['B'] * w['Hk']} (batch, kv-group) units of ONE problem, no collective "
                   "on the data path; NCCL all_gather of per-unit hashes after the timed region")
        elif world > 1:
            par = f"{world} independent replicas of the workload (one per GPU, own seed), no collective"
        else:
            par = "1 GPU"
        line = {"metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps, "warmup": warmup,
                "ms_per_step": ms, "higher_is_better": True, "scaling": "strong" if job.sharded else "weak",
                "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
                "config": {"workload": name + ": " + json.dumps(shape) + (f" qk_scale={sweep[0]:g}" if sweep else "")
                           + ", bf16 q/k/v/dO from seed " + str(SEED), "parallelism": par,
                           "l2": f"inputs of a step ({job.input_bytes() >> 20} MiB per GPU) larger than L2"},
                "per_gpu_tflops": value / world, "pct_of_fp8_nominal_peak": 100.0 * value / world / FP8_NOMINAL_TFLOPS,
                "pct_of_fp8_measured_burst_peak": 100.0 * value / world / (2.0 * peaks["bf16_tflops"]),
                "kernel_ms": kernel_ms, "roofline": roofline, "rooflines": rooflines, "sustained": sustained,
                "clocks": clocks, "e2e": e2e, "gpu_launches": launches,
                "gpu_launches_note": "kernel launches of this library inside the timed region, counted by the library itself"}
        if validation is not None:
            line["validation"] = validation
        fp8_mm = fp8_matmul_tflops(dev)
        if fp8_mm is not None:
            line["fp8_matmul_tflops_cublaslt_8192"] = fp8_mm
        if world == 1 and not args.no_extra and name == "c2":
            del job
            torch.cuda.empty_cache()
            line["configs"] = {n: short_run(n, dev) for n in ("c3", "c4", "c5")}
            # the headline workload under the other numerics arms the kernels implement (not the metric's numerics)
            line["numerics_arms"] = {}
            for arm in ("sm100-mx-ds32", "sm100-mx-nonorm"):
                aj = Job(name, w, dev, 0, 1, numerics=arm)
                ams, _ = run_timed(aj, 5, 3, torch.cuda.synchronize, lambda x: x)
                line["numerics_arms"][arm] = {"ms_per_step": ams, "value": aj.job_flops / (ams * 1e-3) / 1e12, "unit": "TFLOPS"}
                del aj
            torch.cuda.empty_cache()
        if world == 1 and not args.no_cpu_baseline:
            tf, cms, cores, sample = cpu_sample(w)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOPS", "cores": cores, "kind": "port", "sample": sample,
                                    "ms_per_sample": cms, "config1_B1_N256_H2_D128_causal": cpu_config1()}
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
