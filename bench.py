#!/usr/bin/env python
"""Benchmark of the FFT spatial-convolution path (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--layer C2] [--impl ours|reference]

A step is the three nn passes (updateOutput, updateGradInput, accGradParameters) of one
layer over one seeded synthetic batch; `value` is direct-convolution-equivalent TFLOP/s
(3 * 2*B*P*F*kH*kW*oH*oW flops per step) with the operands resident in HBM.  With N > 1
ranks the global batch of 128 is split across ranks (strong scaling) and the weight
gradient's spectrum is all-reduced inside accGradParameters.  `e2e` is the same step
through the host-buffer entry points of the C ABI (pinned host memory, copies timed).
The last stdout line is the short result object; the per-kernel and per-layer tables go
to --detail-file.  Outside the timed region every timed layer is checked on sampled
planes against the fp64 direct convolution (`parity_checked`).
`--impl reference` times the reference's own CPU convolution (compiled from its source
under oracle/_ref) on a bounded batch slice with every host thread.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# name: (B, P, F, iH, iW, kH, kW, padH, padW, bias?)   -- the reference's benchmark list
LAYERS = {
    "C1": (16, 16, 16, 32, 32, 5, 5, 0, 0, False),
    "C2": (128, 3, 96, 128, 128, 11, 11, 0, 0, True),
    "C3": (128, 64, 128, 64, 64, 9, 9, 0, 0, False),
    "C4a": (128, 128, 128, 32, 32, 9, 9, 0, 0, False),
    "C4b": (128, 128, 128, 16, 16, 7, 7, 0, 0, False),
    "C5": (128, 384, 384, 13, 13, 3, 3, 1, 1, False),
}
PASSES = ("updateOutput", "updateGradInput", "accGradParameters")
STAGES = ("fft_a", "fft_b", "contract", "allreduce", "ifft", "bias")
METRIC = "direct-conv-equivalent TFLOP/s, 3 passes (fwd+bwd+accGrad)"
PARITY_TOL = 1e-4  # max|x - ref| <= PARITY_TOL * max|ref| against the fp64 direct convolution


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def conv_flops(L, batch=None):
    B, P, F, iH, iW, kH, kW, pH, pW, _ = L
    B = batch if batch is not None else B
    oH, oW = iH + 2 * pH - kH + 1, iW + 2 * pW - kW + 1
    return 2.0 * B * P * F * kH * kW * oH * oW


def fft_size(L):
    _, _, _, iH, iW, kH, kW, pH, pW, _ = L
    n, need = 8, max(iH + 2 * pH, iW + 2 * pW, kH, kW)
    while n < need:
        n *= 2
    return n


def stage_algorithmic(L, B, pass_idx, stage):
    """Algorithmic (bytes, flops) of one launch of a stage:
    a transform of D planes of h x w reads or writes 4*D*h*w real bytes and 8*D*bins
    spectrum bytes; the contraction reads two spectra, writes one and does 8*M*N*K*bins flops."""
    _, P, F, iH, iW, kH, kW, pH, pW, _ = L
    oH, oW = iH + 2 * pH - kH + 1, iW + 2 * pW - kW + 1
    n = fft_size(L)
    bins = (n // 2 + 1) * n
    real = {"in": (B * P, iH * iW), "out": (B * F, oH * oW), "w": (F * P, kH * kW)}
    plan = {  # pass -> (fft_a, fft_b, ifft) operands
        0: ("in", "w", "out"), 1: ("out", "w", "in"), 2: ("out", "in", "w")}[pass_idx]
    def tr(which):
        d, hw = real[which]
        return 4.0 * d * hw + 8.0 * d * bins
    if stage == "fft_a":
        return tr(plan[0]), 0.0
    if stage == "fft_b":
        return tr(plan[1]), 0.0
    if stage == "ifft":
        return tr(plan[2]), 0.0
    if stage == "contract":
        spectra = 8.0 * bins * (B * P + B * F + F * P)
        return spectra, 8.0 * B * P * F * bins
    if stage == "allreduce":
        return 8.0 * bins * F * P, 0.0
    if stage == "bias":
        return 8.0 * B * F, 0.0
    raise KeyError(stage)


# ---------------------------------------------------------------------------
# reference arm / CPU baseline
# ---------------------------------------------------------------------------
def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_reference_step(L, threads, items, filters, seed=0):
    """One bounded sample: the three reference CPU functions on `items` batch elements and
    the first `filters` output planes of the layer, batch slices spread over `threads`
    threads.  Work is linear in both, so throughput carries over to the full layer.
    Returns (seconds, kind)."""
    import numpy as np
    import oracle
    _, P, _, iH, iW, kH, kW, pH, pW, _ = L
    s = oracle.Shape(items, P, filters, iH, iW, kH, kW, pH, pW)
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((items, P, iH, iW)).astype(np.float32)
    w = rng.uniform(-1, 1, (filters, P, kH, kW)).astype(np.float32) / np.float32(np.sqrt(kH * kW * P))
    go = rng.standard_normal((items, filters, s.oH, s.oW)).astype(np.float32)
    use_ref = oracle.reference_available()
    t0 = time.perf_counter()
    if use_ref:
        oracle.reference_update_output(s, x, w, threads=threads)
        oracle.reference_update_grad_input(s, go, w, threads=threads)
        oracle.reference_acc_grad_weight(s, x, go, 1.0, threads=threads)
    else:  # the fp64 restatement (OpenMP over planes)
        oracle.update_output(s, x, w)
        oracle.update_grad_input(s, go, w)
        oracle.acc_grad_weight(s, x, go, 1.0)
    return time.perf_counter() - t0, ("reference" if use_ref else "port")


def sample_flops(L, items, filters):
    return 3.0 * conv_flops(L, items) * filters / L[2]


def cpu_sample(L, threads, target_s):
    """Sizes a sample (batch items, filters) that takes about target_s seconds: one batch
    element per thread, then as many filters as fit, calibrated by a small probe."""
    items = int(min(L[0], threads))
    probe_f = max(1, L[2] // 32)
    dt, _ = cpu_reference_step(L, threads, items, probe_f)
    rate = sample_flops(L, items, probe_f) / max(dt, 1e-6)
    filters = int(max(1, min(L[2], round(rate * target_s / sample_flops(L, items, 1)))))
    return items, filters


def sample_text(name, L, items, filters, threads):
    return (f"{items} of {L[0]} batch elements x {filters} of {L[2]} filters of layer {name}, all three passes, "
            f"{threads} threads (one batch slice each); throughput is linear in both")


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    L = LAYERS[args.layer]
    threads = host_threads()
    target = max(0.5, min(8.0, 120.0 / max(1, args.steps + args.warmup)))
    items, filters = cpu_sample(L, threads, target)
    kind = "reference"
    for _ in range(args.warmup):
        _, kind = cpu_reference_step(L, threads, items, filters)
    times = []
    for i in range(args.steps):
        dt, kind = cpu_reference_step(L, threads, items, filters, seed=i + 1)
        times.append(dt)
    total = sum(times)
    value = sample_flops(L, items, filters) * args.steps / total / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(args.layer, L, args.gpus),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": min(threads, items), "kind": kind,
                         "sample": sample_text(args.layer, L, items, filters, threads)},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


def step_bytes(L):
    """Bytes of the real tensors one step touches (input, output / gradOutput, weight)."""
    B, P, F, iH, iW, kH, kW, pH, pW, _ = L
    oH, oW = iH + 2 * pH - kH + 1, iW + 2 * pW - kW + 1
    return 4 * (B * P * iH * iW + B * F * oH * oW + F * P * kH * kW)


def workload_config(name, L, gpus, allreduce="spectrum", reuse="none", exchange="NCCL"):
    B, P, F, iH, iW, kH, kW, pH, pW, _ = L
    return {
        "workload": f"{name}: {B}x{P}x{iH}x{iW} input, {F} filters {kH}x{kW}, pad {pH}, FFT {fft_size(L)}; step = 3 passes",
        "global_batch": B,
        "parallelism": (f"batch/{gpus} ranks, gradWeight " + ("spectrum" if allreduce == "spectrum" else "(spatial)")
                        + f" summed over {exchange}") if gpus > 1 else "single GPU",
        "l2": "inputs > L2" if step_bytes(L) > (126 << 20) else "inputs fit L2 (warm); layers_step_ms after flush",
        "memory_reuse": reuse,
    }


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            with open(self.path) as f:
                for line in f:
                    c = [x.strip() for x in line.split(",")]
                    if len(c) < 9:
                        continue
                    try:
                        sm.append(float(c[1]))
                        mx.append(float(c[2]))
                    except ValueError:
                        continue
                    for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                        if v.lower().startswith("active"):
                            reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            busy = [v for v in sm if v >= 0.5 * max(sm)] or sm
            out.update(sm_mhz=statistics.median(busy), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


def gen(torch, shape, seed, kind="normal", bound=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    t = torch.empty(shape, device="cuda", dtype=torch.float32)
    return t.normal_(generator=g) if kind == "normal" else t.uniform_(-bound, bound, generator=g)


class LayerRun:
    """Device tensors and a native handle for one layer at a local batch."""

    def __init__(self, torch, name, L, local_batch, rank, comm=None, allreduce="spectrum", reuse="none"):
        from fbcunn_b200 import SpatialConvolutionFBFFT
        self.torch, self.name, self.L, self.B = torch, name, L, local_batch
        _, P, F, iH, iW, kH, kW, pH, pW, has_bias = L
        cfg = list(LAYERS).index(name) + 1
        oH, oW = iH + 2 * pH - kH + 1, iW + 2 * pW - kW + 1
        bound = 1.0 / (kH * kW * P) ** 0.5
        self.x = gen(torch, (local_batch, P, iH, iW), 1000 * cfg + 10 * rank)
        self.go = gen(torch, (local_batch, F, oH, oW), 1000 * cfg + 10 * rank + 1)
        self.m = SpatialConvolutionFBFFT(P, F, kW, kH, 1, 1, pW, pH, reuse, allreduce=allreduce)
        self.m.weight.copy_(gen(torch, (F, P, kH, kW), 1000 * cfg + 2, "uniform", bound))
        if has_bias:
            self.m.bias.copy_(gen(torch, (F,), 1000 * cfg + 3, "uniform", 0.01))
        else:
            self.m.bias.zero_()
        if comm is not None:
            self.m.attachCommunicator(*comm)

    def step(self):
        self.m.updateOutput(self.x)
        self.m.updateGradInput(self.x, self.go)
        self.m.accGradParameters(self.x, self.go, 1.0)

    def run_pass(self, i):
        if i == 0:
            self.m.updateOutput(self.x)
        elif i == 1:
            self.m.updateGradInput(self.x, self.go)
        else:
            self.m.accGradParameters(self.x, self.go, 1.0)

    def handle(self):
        return self.m._handle


def step_times(torch, capi, lib, run, iters):
    """ms per step of three passes launched back to back (no flush, no profiling events), and the
    same step replayed from a CUDA graph: what launch gaps cost on the small layers."""
    capi.check(lib.fbfftconv_profile_enable(run.handle(), 0))
    out = {}

    def timed(fn):
        fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(max(iters, 5)):
            fn()
        b.record()
        b.synchronize()
        return a.elapsed_time(b) / max(iters, 5)

    out["eager"] = timed(run.step)
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            run.step()
        out["cuda_graph"] = timed(graph.replay)
    except Exception as e:  # a capture the runtime refuses is reported, not fatal
        out["cuda_graph"] = None
        out["cuda_graph_error"] = str(e).splitlines()[0][:200]
        torch.cuda.synchronize()
    return out


def read_profile(handle):
    from fbcunn_b200 import capi
    out = {}
    for pi, pname in enumerate(PASSES):
        for si, sname in enumerate(STAGES):
            ms, n = ctypes.c_double(), ctypes.c_int()
            capi.check(capi.lib().fbfftconv_profile_read(handle, pi, si, ctypes.byref(ms), ctypes.byref(n)))
            if n.value:
                out[(pi, sname)] = (ms.value, n.value, int(capi.lib().fbfftconv_profile_overlapped(handle, pi, si)) == 1)
    return out


def kernel_table(L, B, prof, pk):
    rows = []
    for (pi, sname), (ms, n, overlapped) in sorted(prof.items()):
        by, fl = stage_algorithmic(L, B, pi, sname)
        avg_s = ms / n / 1e3
        row = {"pass": PASSES[pi], "kernel": sname, "launches": n, "avg_us": 1e6 * avg_s, "total_ms": ms,
               "gbs": by / avg_s / 1e9 if avg_s > 0 else None}
        if overlapped:
            # ran next to the pass's other forward transform on the library's second stream: the time
            # is wall time shared with that kernel, not this kernel's cost, so no rate is derived from it
            row["overlapped"] = True
            row["gbs"] = None
        if row["gbs"] is not None:
            row["frac_hbm"] = row["gbs"] / pk["hbm_gbs"]
        if fl:
            row["tflops"] = fl / avg_s / 1e12 if avg_s > 0 else None
            if row["tflops"] is not None:
                row["frac_tensor_3xtf32"] = row["tflops"] / tensor_peak_3xtf32(pk)
        rows.append(row)
    return rows


def captured_traffic(layer, top, L, local_b):
    """DRAM bytes per launch of the dominant kernel from the committed ncu capture
    (profiles/dram_traffic.json), scaled by the planes this launch processes; None where no
    capture of that kernel on that layer exists."""
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
            table = json.load(f)
        entry = table[layer][f'{top["kernel"]}:{top["pass"]}']
    except (OSError, KeyError, ValueError):
        return None
    if entry["unit"] == "launch":
        return float(entry["bytes_per_unit"]) if local_b == L[0] else None
    return float(entry["bytes_per_unit"]) * local_b * L[2]  # planes (b, f) in this launch


def sig(v, digits=4):
    """Rounds to `digits` significant digits (keeps the result line short)."""
    if v is None or isinstance(v, (bool, int, str)):
        return v
    return float(f"{float(v):.{digits}g}")


def compact(d, keys):
    return {k: sig(d[k], 5) if isinstance(d.get(k), float) else d.get(k) for k in keys if k in d}


def tensor_peak_3xtf32(pk):
    """Algorithmic TFLOP/s the 3xTF32 contraction can reach: dense TF32 is taken as half the
    measured bf16 rate and every product costs three MMAs."""
    return pk["bf16_tflops"] / 2.0 / 3.0


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    from fbcunn_b200 import build as fb_build
    from fbcunn_b200 import capi

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    fb_build.build()
    capi.lib()
    comm = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        from fbcunn_b200 import SpatialConvolutionFBFFT
        from fbcunn_b200.sharding import share_unique_id
        comm = (share_unique_id(dist, SpatialConvolutionFBFFT.makeUniqueId), rank, world)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    pk = peaks()
    name, L = args.layer, LAYERS[args.layer]
    assert L[0] % world == 0, "global batch must divide over the ranks"
    local_b = L[0] // world
    run = LayerRun(torch, name, L, local_b, rank, comm, args.allreduce, args.reuse)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # before the warm-up so that short timed regions still get samples
    for _ in range(max(args.warmup, 3)):
        run.step()
    barrier()

    # ---- timed region: K steps, device time, max over ranks --------------------
    lib = capi.lib()
    capi.check(lib.fbfftconv_profile_enable(run.handle(), 1))
    capi.check(lib.fbfftconv_profile_reset(run.handle()))
    launches0 = capi.kernel_launches()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        run.step()
    ev1.record()
    barrier()
    elapsed_ms = max_over_ranks(ev0.elapsed_time(ev1))
    launches = capi.kernel_launches() - launches0
    prof = read_profile(run.handle())
    capi.check(lib.fbfftconv_profile_enable(run.handle(), 0))
    device_status = int(lib.fbfftconv_tensor_core_status(0))
    if device_status != 0:
        raise SystemExit(f"tensor-core contraction reported device status {device_status}")
    ms_per_step = elapsed_ms / args.steps
    value = 3.0 * conv_flops(L) / (ms_per_step / 1e3) / 1e12
    # who carried the weight-gradient sum: the library's kernels over peer memory (NVLink loads / stores), or NCCL
    exchange = "peer memory" if world > 1 and run.m.peerExchangeStatus() == 1 else "NCCL"
    if world > 1 and run.m.peerExchangeStatus() >= 100:
        raise SystemExit(f"a bounded wait of the peer exchange gave up: status {run.m.peerExchangeStatus()}")

    kernels = kernel_table(L, local_b, prof, pk)
    top = max((k for k in kernels if k["kernel"] != "allreduce" and not k.get("overlapped")),
              key=lambda k: k["total_ms"])
    by, fl = stage_algorithmic(L, local_b, PASSES.index(top["pass"]), top["kernel"])
    secs = top["avg_us"] / 1e6
    # the contraction is held against the tensor roofline where its intensity is above the
    # ridge of (3xTF32 peak) / (HBM peak), otherwise against HBM like the transforms
    ridge = tensor_peak_3xtf32(pk) * 1e12 / (pk["hbm_gbs"] * 1e9)
    if fl and fl / by > ridge:
        achieved = fl / secs / 1e12
        roofline = {"bound": "tensor", "kernel": f'{top["kernel"]} of {top["pass"]}', "achieved": achieved,
                    "peak": tensor_peak_3xtf32(pk), "peak_source": pk["source"] + " bf16/6 (3xTF32)",
                    "unit": "TFLOP/s", "frac": achieved / tensor_peak_3xtf32(pk), "traffic": None,
                    "algorithmic_flops_per_launch": fl}
    else:
        achieved = by / secs / 1e9
        roofline = {"bound": "hbm", "kernel": f'{top["kernel"]} of {top["pass"]}', "achieved": achieved,
                    "peak": pk["hbm_gbs"], "peak_source": pk["source"], "unit": "GB/s",
                    "frac": achieved / pk["hbm_gbs"], "traffic": None, "algorithmic_bytes_per_launch": by}
    roofline["traffic"] = captured_traffic(name, top, L, local_b)
    roofline["avg_launch_us"] = top["avg_us"]
    roofline["share_of_step"] = top["total_ms"] / elapsed_ms

    # ---- e2e: host buffers through the *_host entry points ----------------------
    e2e = measure_e2e(torch, lib, run, L, local_b, world, barrier, max_over_ranks,
                      steps=max(1, min(args.steps, 5)))

    clocks = sampler.stop() if rank == 0 else None  # sampled from the warm-up to the end of the e2e leg

    # ---- parity of what was timed, on sampled planes (not timed) -------------------
    parity = None
    if not args.no_parity:
        parity = parity_check(torch, dist, run, L, local_b, world, max_over_ranks)
        if not parity["ok"]:
            raise SystemExit(f"parity check failed: {parity}")

    # ---- per layer, per pass (cold L2) ------------------------------------------
    layers = {}
    if not args.no_layers:
        del run
        torch.cuda.empty_cache()
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        for lname, LL in LAYERS.items():
            if LL[0] % world:
                continue
            lb = LL[0] // world
            r = LayerRun(torch, lname, LL, lb, rank, comm, args.allreduce)
            for _ in range(3):
                r.step()
            capi.check(lib.fbfftconv_profile_enable(r.handle(), 1))
            capi.check(lib.fbfftconv_profile_reset(r.handle()))
            per_pass = []
            for pi in range(3):
                ts = []
                for _ in range(args.layer_iters):
                    flush.zero_()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    barrier()
                    a.record()
                    r.run_pass(pi)
                    b.record()
                    barrier()
                    ts.append(max_over_ranks(a.elapsed_time(b)))
                ms = statistics.median(ts)
                per_pass.append({"pass": PASSES[pi], "ms": ms, "tflops": conv_flops(LL) / (ms / 1e3) / 1e12})
            prof_l = read_profile(r.handle())
            layers[lname] = {"fft_size": fft_size(LL), "local_batch": lb, "passes": per_pass,
                             "kernels": kernel_table(LL, lb, prof_l, pk)}
            if world == 1:
                layers[lname]["step_ms"] = step_times(torch, capi, lib, r, args.layer_iters)
            if parity is not None and lname != name:
                pc = parity_check(torch, dist, r, LL, lb, world, max_over_ranks)
                layers[lname]["parity"] = pc
                if not pc["ok"]:
                    raise SystemExit(f"parity check failed on {lname}: {pc}")
                parity["max_rel_err"] = max(parity["max_rel_err"], pc["max_rel_err"])
                parity.setdefault("layers", [name]).append(lname)
            del r
            torch.cuda.empty_cache()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        # the reference's CPU convolution is single-threaded: one thread on one batch element is the
        # reference as it stands; the threaded figure (one batch slice per host thread) is what the
        # host can do with it and is the one carried as `value`
        threads = host_threads()
        items1, filters1 = cpu_sample(L, 1, 4.0)
        dt1, kind = cpu_reference_step(L, 1, items1, filters1)
        items, filters = cpu_sample(L, threads, 6.0)
        dt, kind = cpu_reference_step(L, threads, items, filters)
        dt2, kind = cpu_reference_step(L, threads, items, filters, seed=1)
        dt = min(dt, dt2)
        cpu = {"value": sig(sample_flops(L, items, filters) / dt / 1e12), "unit": "TFLOP/s",
               "cores": min(threads, items), "kind": kind,
               "one_thread_value": sig(sample_flops(L, items1, filters1) / dt1 / 1e12),
               "sample": f"{items}/{L[0]} batch x {filters}/{L[2]} filters, {dt:.1f} s; 1 thread: {items1} x {filters1}, "
                         f"{dt1:.1f} s; linear"}

    if rank == 0:
        detail = {"kernels": kernels, "layers": layers, "roofline": roofline, "e2e": e2e, "parity": parity,
                  "config": workload_config(name, L, world, args.allreduce, args.reuse, exchange)}
        try:
            with open(args.detail_file, "w") as f:
                json.dump(detail, f, indent=1)
        except OSError as e:
            sys.stderr.write(f"bench detail not written: {e}\n")
        # per layer: sum of the three per-pass medians (ms), each timed after an L2 flush
        layers_step_ms = {k: sig(sum(p["ms"] for p in v["passes"])) for k, v in layers.items()}
        line = {
            "metric": METRIC, "value": sig(value, 5), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": sig(ms_per_step, 5), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(name, L, world, args.allreduce, args.reuse, exchange),
            "roofline": compact(roofline, ("bound", "kernel", "achieved", "peak", "unit", "frac", "traffic",
                                           "avg_launch_us", "peak_source")),
            "cpu_baseline": cpu,
            "e2e": compact(e2e, ("value", "unit", "ms_per_step", "h2d_bytes_per_step", "d2h_bytes_per_step")),
            "gpu_launches": int(launches), "clocks": clocks, "layers_step_ms": layers_step_ms,
            "parity_checked": bool(parity and parity["checked"]),
            "parity_max_rel_err": sig(parity["max_rel_err"], 3) if parity else None,
        }
        print(json.dumps(line, separators=(",", ":")), flush=True)
    if world > 1:
        import gc
        gc.collect()  # handles detach from the communicator before it is shut down
        lib.fbfftconv_comm_shutdown()
        dist.destroy_process_group()
    return 0


def parity_check(torch, dist, run, L, local_b, world, max_over_ranks, planes=8):
    """Outside the timed region: the three passes of the timed layer, on the tensors that were
    timed, against the fp64 direct convolution (the CPU oracle, here only as the checker) on
    `planes` sampled planes per pass.  With several ranks every rank computes the oracle planes of
    the weight gradient for its own batch shard and the partial results are summed over ranks
    (what the reference's data-parallel test asserts about replicas, test/test_DataParallel.lua:73-159)."""
    import numpy as np
    import oracle
    _, P, F, iH, iW, kH, kW, pH, pW, has_bias = L
    s = oracle.Shape(local_b, P, F, iH, iW, kH, kW, pH, pW)
    m = run.m
    x, go = run.x.cpu().numpy(), run.go.cpu().numpy()
    w = m.weight.cpu().numpy()
    b = m.bias.cpu().numpy() if has_bias else None
    rng = np.random.default_rng(20240229)  # the same planes on every rank
    bi, fi, pi = rng.integers(0, local_b, planes), rng.integers(0, F, planes), rng.integers(0, P, planes)
    out = m.updateOutput(run.x)
    got_out = out[torch.as_tensor(bi), torch.as_tensor(fi)].cpu().numpy()
    gi = m.updateGradInput(run.x, run.go)
    got_gi = gi[torch.as_tensor(bi), torch.as_tensor(pi)].cpu().numpy()
    m.accGradParameters(run.x, run.go, 1.0)
    torch.cuda.synchronize()
    got_gw = m.gradWeight[torch.as_tensor(fi), torch.as_tensor(pi)].cpu().numpy()
    got_gb = m.gradBias.cpu().numpy()
    ref_gw = oracle.acc_grad_weight_planes(s, x, go, 1.0, fi, pi)
    ref_gb = oracle.acc_grad_bias(s, go, 1.0)
    if world > 1:
        t = torch.from_numpy(np.concatenate([ref_gw.ravel(), ref_gb.ravel()])).cuda()
        dist.all_reduce(t)
        t = t.cpu().numpy()
        ref_gw, ref_gb = t[:ref_gw.size].reshape(ref_gw.shape), t[ref_gw.size:]

    def rel(a, ref):
        return float(np.abs(a.astype(np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))

    errs = {"updateOutput": rel(got_out, oracle.update_output_planes(s, x, w, b, bi, fi)),
            "updateGradInput": rel(got_gi, oracle.update_grad_input_planes(s, go, w, bi, pi)),
            "gradWeight": rel(got_gw, ref_gw), "gradBias": rel(got_gb, ref_gb)}
    errs = {k: max_over_ranks(v) for k, v in errs.items()}
    worst = max(errs.values())
    return {"checked": True, "planes_per_pass": planes, "tol": PARITY_TOL, "max_rel_err": worst,
            "per_pass": errs, "ok": worst <= PARITY_TOL}


def measure_e2e(torch, lib, run, L, local_b, world, barrier, max_over_ranks, steps):
    from fbcunn_b200 import capi
    m = run.m
    _, P, F, iH, iW, kH, kW, pH, pW, has_bias = L
    oH, oW = iH + 2 * pH - kH + 1, iW + 2 * pW - kW + 1
    pin = lambda t: t.detach().cpu().pin_memory()
    hx, hgo, hw, hb = pin(run.x), pin(run.go), pin(m.weight), pin(m.bias)
    hout = torch.empty((local_b, F, oH, oW)).pin_memory()
    hgi = torch.empty((local_b, P, iH, iW)).pin_memory()
    hgw = torch.empty((F, P, kH, kW)).pin_memory()
    hgb = torch.empty((F,)).pin_memory()
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    h = run.handle()

    def step_sync():
        capi.check(lib.fbfftconv_update_output_host(h, p(hx), p(hw), p(hb) if has_bias else None, p(hout), st))
        capi.check(lib.fbfftconv_update_grad_input_host(h, p(hgo), p(hw), p(hgi), st))
        capi.check(lib.fbfftconv_acc_grad_parameters_host(h, p(hx), p(hgo), p(hgw), p(hgb), ctypes.c_float(1.0), st))

    def step_async():
        # forward, then nn.Module:backward (updateGradInput + accGradParameters with gradOutput uploaded
        # once): uploads, kernels and downloads are enqueued on three streams and the step's results are
        # read (waited for) once per step
        capi.check(lib.fbfftconv_update_output_host_async(h, p(hx), p(hw), p(hb) if has_bias else None, p(hout), st))
        capi.check(lib.fbfftconv_backward_host_async(h, p(hx), p(hgo), p(hw), p(hgi), p(hgw), p(hgb),
                                                     ctypes.c_float(1.0), st))
        capi.check(lib.fbfftconv_host_sync(h))

    def timed(step):
        step()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            step()  # ends with a host-side wait for the step's downloads
        b.record()
        barrier()
        return max_over_ranks(a.elapsed_time(b)) / steps

    ms_sync = timed(step_sync)
    ms = timed(step_async)
    h2d = 4 * (2 * hx.numel() + hgo.numel() + 2 * hw.numel() + (hb.numel() if has_bias else 0))
    h2d_sync = 4 * (2 * hx.numel() + 2 * hgo.numel() + 2 * hw.numel() + (hb.numel() if has_bias else 0))
    d2h = 4 * (hout.numel() + hgi.numel() + hgw.numel() + hgb.numel())
    return {"value": 3.0 * conv_flops(L) / (ms / 1e3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms,
            "h2d_bytes_per_step": int(h2d) * world, "d2h_bytes_per_step": int(d2h) * world,
            "api": "fbfftconv_update_output_host_async + fbfftconv_backward_host_async (updateGradInput and "
                   "accGradParameters, gradOutput uploaded once) + fbfftconv_host_sync once per step, pinned host "
                   "buffers",
            "call_by_call_ms_per_step": ms_sync, "call_by_call_h2d_bytes_per_step": int(h2d_sync) * world,
            "call_by_call_api": "fbfftconv_*_host, three calls, each uploads its operands and waits for its download"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--layer", default="C2", choices=list(LAYERS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=0,
                    help="override the layer's global batch (small cases for profiler captures)")
    ap.add_argument("--layer-iters", type=int, default=5)
    ap.add_argument("--allreduce", default="spectrum", choices=["spectrum", "spatial"],
                    help="N > 1: sum the gradWeight spectrum before the inverse FFT (default, as the reference "
                         "data-parallel path is specified) or gradWeight after it")
    ap.add_argument("--reuse", default="none", choices=["none", "all"],
                    help="memoryReusePolicy of the timed module: 'all' lets the backward passes take over spectra "
                         "of the earlier passes of the step (not the default, which recomputes everything)")
    ap.add_argument("--no-layers", action="store_true", help="skip the per-layer / per-pass table")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-parity", action="store_true", help="skip the sampled-plane check against the CPU oracle")
    ap.add_argument("--detail-file", default=os.path.join(ROOT, "bench_detail.json"),
                    help="per-kernel and per-layer tables (the result line on stdout stays short)")
    args = ap.parse_args()
    if args.batch > 0:
        for k, v in list(LAYERS.items()):
            LAYERS[k] = (args.batch,) + v[1:]
    if args.impl == "reference":
        return run_reference_arm(args)
    return run_gpu_arm(args)


if __name__ == "__main__":
    sys.exit(main())
