#!/usr/bin/env python
"""Benchmark of the sig / sig_backprop path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config C5] [--impl ours|reference]

One "step" is one pass of the hot path over the configured synthetic batch: forward
(sig) plus backward (sig_backprop) for the fwd+bwd configs, forward only otherwise.
The default workload is BASELINE.json's configs[4] (C5: float32, B=4096, L=4096, d=16,
degree 4, Brownian-like paths, forward + backward), the configuration the headline metric
(paths/s fwd+bwd at 1/2/4/8 B200) is quoted on; the batch is split evenly over the ranks
(strong scaling) and no collective is on the data path.

Rank 0 prints ONE JSON line.  `value` is measured with inputs resident in HBM, with CUDA
events on the launching stream; `e2e` goes through the reference-named C-ABI symbols with
pinned HOST buffers (copies inside the timed region); `roofline` describes the dominant
kernel against the FMA-pipe peak measured in the same run; `parity` compares the results of
the timed kernels, on the whole shard, with the reference's own CUDA kernels and, on a
64-path subset, with the float64 CPU oracle; `configs` (default run on one GPU) holds the
other four BASELINE.json configurations in short; `cpu_baseline` times the CPU oracle (a port
of the reference's cpsig arithmetic, release-style build) on this box's host cores.
`--impl reference` times that CPU port alone, as the reference arm.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # name: B, L, d, N, dtype, input law, what a step runs
    "C1": dict(B=32, L=1000, d=10, N=5, dtype="float64", law="iid_points", mode="fwd"),
    "C2": dict(B=1024, L=256, d=2, N=12, dtype="float64", law="brownian", mode="fwd"),
    "C3": dict(B=128, L=1024, d=5, N=7, dtype="float32", law="brownian", mode="fwd"),
    "C4": dict(B=256, L=2048, d=8, N=4, dtype="float32", law="brownian", mode="fwdbwd"),
    "C5": dict(B=4096, L=4096, d=16, N=4, dtype="float32", law="brownian", mode="fwdbwd"),
    # shapes beyond the five: deep degrees the reference serves with its register "Tree" kernels
    # (siglib/cusig/cu_signature_horner.cuh:267-307, 389-438) and C1 with time augmentation
    "X1": dict(B=64, L=128, d=6, N=8, dtype="float32", law="brownian", mode="fwdbwd"),
    "X2": dict(B=8, L=64, d=16, N=6, dtype="float64", law="brownian", mode="fwdbwd"),
    "X3": dict(B=64, L=256, d=24, N=4, dtype="float64", law="brownian", mode="fwdbwd"),
    "X4": dict(B=32, L=1000, d=10, N=5, dtype="float64", law="iid_points", mode="fwd", time_aug=True),
}


# ---- algorithmic work (FMA-pipe instructions per path and step, non-redundant form) ----

def instr_forward(d, N):
    """One Horner step in the level-tensor form with increments pre-scaled by 1/j:
    FMAs into levels 2..N, MULs building the work levels, ADDs (work + signature, level 1),
    and the scaling of dx (reference op-count form: siglib/cpsig/cp_signature.h:670-701)."""
    fma = sum(d ** k for k in range(2, N + 1))
    mul = sum(d ** (l + 1) for k in range(2, N + 1) for l in range(1, k - 1))
    add = sum(sum(d ** l for l in range(1, k - 1)) + d ** (k - 1) for k in range(2, N + 1)) + d
    return fma + mul + add + d * (N - 1), fma


def instr_backward(d, N):
    """Rewind (= one forward step) plus the pull-back of siglib/cpsig/cp_signature.h:1147-1187:
    per target level T and level l < T two FMA streams over d^(l+1) entries (gradient and
    adjoint contraction), four ops per level-l word (value add+mul, scale, adjoint add), the
    rebuild of the work levels, and the O(d) bookkeeping."""
    fwd, fwd_fma = instr_forward(d, N)
    pull, pull_fma = d, 0
    for T in range(2, N + 1):
        for l in range(1, T):
            pull += 2 * d ** (l + 1) + 4 * d ** l
            pull_fma += 2 * d ** (l + 1)
        pull += sum(d ** (l + 1) for l in range(1, T - 1)) + 2 * d
    return fwd + pull, fwd_fma + pull_fma


def instr_backward_executed(d, N):
    """What the register-tile reverse sweep really issues, in the same counting: the pull-back is
    the same, but the rewind stops below level N (the reverse sweep never reads the level-N state,
    so it is neither loaded nor rewound): one forward step of degree N-1 instead of degree N."""
    fwd, fwd_fma = instr_forward(d, N)
    total, total_fma = instr_backward(d, N)
    low, low_fma = instr_forward(d, N - 1) if N >= 2 else (0, 0)
    return total - fwd + low, total_fma - fwd_fma + low_fma


# DRAM traffic of the two dominant kernels as ncu measured it on a small case of the C5 shape
# (B=512, L=257, d=16, degree 4: dram__bytes_read.sum + dram__bytes_write.sum per launch; see
# profiles/).  Not scaled to the full launch: part of the small case's reads hit the L2 left warm
# by the kernel before it, which a 4096-path launch cannot repeat.
NCU_SMALL_CASE_TRAFFIC = {
    "backward": {"bytes": 176.5e6, "algorithmic_bytes": 303.0e6, "case": "C5 shape at B=512, L=257 (ncu, one launch)"},
    "forward": {"bytes": 97.9e6, "algorithmic_bytes": 151.6e6, "case": "C5 shape at B=512, L=257 (ncu, one launch)"},
}


def bind_to_local_cpus(local_rank):
    """Pins this process to the CPUs next to its GPU before any pinned host buffer is allocated, so
    that the buffers are placed in that socket's memory (first touch) and the copies of the ranks
    do not all cross one socket's memory controller.  Best effort: silently does nothing where the
    topology files are missing or the cpuset of the container forbids it."""
    try:
        import torch
        bus = torch.cuda.get_device_properties(local_rank).pci_bus_id
        dom = torch.cuda.get_device_properties(local_rank).pci_domain_id
        dev = torch.cuda.get_device_properties(local_rank).pci_device_id
        name = "%04x:%02x:%02x.0" % (dom, bus, dev)
        with open("/sys/bus/pci/devices/%s/local_cpulist" % name) as f:
            text = f.read().strip()
        cpus = set()
        for part in text.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0) & cpus
        if allowed and allowed != os.sched_getaffinity(0):
            os.sched_setaffinity(0, allowed)
            return "cpus %s (local to GPU %s)" % (text, name)
        return "unchanged (%d cpus allowed)" % len(os.sched_getaffinity(0))
    except Exception as exc:
        return "unchanged (%s)" % type(exc).__name__


def make_paths(cfg, batch, seed, torch):
    """Seeded synthetic input with the law BASELINE.json states for the config."""
    gen = torch.Generator().manual_seed(seed)
    L, d = cfg["L"], cfg["d"]
    dt = torch.float32 if cfg["dtype"] == "float32" else torch.float64
    if cfg["law"] == "iid_points":
        return torch.randn((batch, L, d), generator=gen, dtype=dt)
    inc = torch.randn((batch, L - 1, d), generator=gen, dtype=dt) * (1.0 / L) ** 0.5
    path = torch.zeros((batch, L, d), dtype=dt)
    torch.cumsum(inc, dim=1, out=path[:, 1:])
    return path


class ClockSampler:
    """Polls nvidia-smi for one GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self._stop, self._thread = index, [], threading.Event(), None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
                parts = [p.strip() for p in out.stdout.strip().split(",")]
                if len(parts) >= 6:
                    self.samples.append(parts)
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        mhz = sorted(float(s[0]) for s in self.samples)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": float(self.samples[0][1]), "reasons": reasons,
                "samples": len(self.samples)}


def cpu_baseline(cfg, cores, paths_per_core=None, target_seconds=10.0):
    """Times the CPU port (oracle/timing.py: the oracle's sources built -O3 -march=native on this
    machine, threaded over static contiguous chunks, and for narrow paths the SIMD-across-paths
    forward the reference's dispatcher would take) on a bounded sample: one path per thread is
    timed first, then as many paths per thread as fit about `target_seconds`.
    Returns (paths/s, sample size, seconds, forward variant)."""
    import torch
    from oracle import timing

    def run(sample):
        path = make_paths(cfg, sample, 99, torch).numpy()
        t0 = time.perf_counter()
        sig, variant = timing.sig(path, cfg["N"], n_threads=cores)
        if cfg["mode"] == "fwdbwd":
            rng = np.random.default_rng(5)
            seeds = rng.normal(size=sig.shape).astype(path.dtype)
            timing.sig_backprop(path, sig, seeds, cfg["N"], n_threads=cores)
        return time.perf_counter() - t0, variant

    lanes = 8 if cfg["dtype"] == "float32" else 4
    if paths_per_core is None:
        probe = max(run(cores * lanes)[0] / lanes, 1e-4)
        paths_per_core = int(max(lanes, min(4096, target_seconds / probe)))
    sample = max(1, cores * paths_per_core)
    dt, variant = run(sample)
    return sample / dt, sample, dt, variant


def run_reference_arm(args, cfg, rank):
    """The reference's CPU implementation of the path (its cpsig library cannot be built
    offline, so the port in oracle/ stands in), all host threads, bounded sample per step."""
    if rank != 0:
        return
    cores = len(os.sched_getaffinity(0)) or 1
    lanes = 8 if cfg["dtype"] == "float32" else 4
    # size one step to about 4 s of wall time on this box, then time exactly `steps` of them
    probe = max(cpu_baseline(cfg, cores, lanes)[2] / lanes, 1e-4)
    per_core = int(max(lanes, min(4096, 4.0 / probe)))
    for _ in range(min(args.warmup, 1)):
        cpu_baseline(cfg, cores, per_core)
    total_paths, total_t, variant = 0, 0.0, ""
    for _ in range(args.steps):
        _, n, dt, variant = cpu_baseline(cfg, cores, per_core)
        total_paths += n
        total_t += dt
    value = total_paths / total_t
    sample = "%d paths of %s per step (%s), %d host threads, %s forward, gcc -O3 -march=native" % (
        per_core * cores, args.config, cfg["mode"], cores, variant)
    print(json.dumps({
        "impl": "reference", "metric": "paths_per_second_" + cfg["mode"], "value": value, "unit": "paths/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total_t / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32" if cfg["dtype"] == "float32" else "f64",
        "data": "synthetic", "config": workload_config(args, cfg, args.gpus),
        "cpu_baseline": {"value": value, "unit": "paths/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "paths/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def workload_config(args, cfg, world):
    return {"workload": "%s: sig %s, %s, B=%d, L=%d, d=%d, degree=%d, %s paths" % (
                args.config, "forward+backward" if cfg["mode"] == "fwdbwd" else "forward", cfg["dtype"], cfg["B"],
                cfg["L"], cfg["d"], cfg["N"], "Brownian-like" if cfg["law"] == "brownian" else "iid N(0,1)"),
            "global_batch": cfg["B"], "per_gpu_batch": cfg["B"] // world, "parallelism": "batch-sharded x%d" % world,
            "l2": "inputs larger than L2" if cfg["B"] // world * (cfg["L"] * cfg["d"] + sum((cfg["d"] + (1 if cfg.get("time_aug") else 0)) ** k for k in range(1, cfg["N"] + 1))) * (4 if cfg["dtype"] == "float32" else 8) > 126e6
                  else "L2 flushed (256 MB written) before every timed call"}


def run_fma_patterns(args):
    """--op fma_patterns: SM cycles per 128 lane-FMAs of one warp instruction stream, per operand
    pattern of the packed / scalar FP32 FMA (pysiglib_b200/csrc/bench/fma_patterns.cu), with one and
    with two warps per SM scheduler.  128 cycles is the nominal pipe rate."""
    import torch
    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    lib = ctypes.CDLL(os.path.join(ROOT, "pysiglib_b200", "lib", "libsigb200_bench.so"))
    lib.sigb200_bench_fma_pattern.argtypes = (ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                              ctypes.c_void_p)
    lib.sigb200_bench_fma_pattern.restype = ctypes.c_int
    dev = torch.device("cuda", 0)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    sink = torch.zeros(2, dtype=torch.float32, device=dev)
    names = ["packed, one fresh operand", "packed, row by row (the kernels' pattern)", "packed, column by column",
             "packed, no operand reuse", "scalar, row by row"]
    iters, out = 20000, {}
    for mode, name in enumerate(names):
        for warps in (1, 2):
            cycles = torch.zeros(sms * warps, dtype=torch.int64, device=dev)
            for it in (200, iters):   # a short warm-up launch, then the measured one
                rc = lib.sigb200_bench_fma_pattern(mode, ctypes.c_void_p(sink.data_ptr()), sms * warps, it,
                                                   ctypes.c_void_p(cycles.data_ptr()), None)
                assert rc == 0, rc
                torch.cuda.synchronize()
            out["%s, %d warp%s per scheduler" % (name, warps, "s" if warps > 1 else "")] = float(cycles.max()) / (iters * warps)
    print(json.dumps({"op": "fma_patterns", "unit": "SM cycles per 128 lane-FMAs per scheduler (nominal 128)", "n_gpus": 1,
                      "cycles": out}))


def run_neighbour_op(args):
    """--op: times one of the operators either side of the signature (not the headline metric).
    One GPU, device-resident inputs larger than L2, CUDA events around the public Python call;
    prints one JSON line with the algorithmic bytes moved against the measured HBM bandwidth."""
    import torch
    import pysiglib_b200 as psl
    from pysiglib_b200 import load_cusig
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU fallback"
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(11)
    rnd = lambda *shape: torch.randn(shape, generator=gen, device=dev, dtype=torch.float32)
    extra = {}
    if args.op == "log_sig":
        # log_sig from the path (one native call) beside sig alone and beside the two public calls the
        # reference composes (sig, then sig_to_log_sig); FMA-bound like sig, so no HBM roofline here
        B, L, d, N = args.batch or 4096, args.length or 4096, 16, 4
        x = torch.cumsum(rnd(B, L, d) * (1.0 / L) ** 0.5, dim=1).contiguous()
        psl.prepare_log_sig(d, N, 1)
        warm, steps = max(args.warmup, 3), args.steps
        with ClockSampler(0) as clocks:
            sig_ms = _time_ms(torch, lambda: psl.sig(x, N), warm, steps)
            one_ms = _time_ms(torch, lambda: psl.log_sig(x, N, method=1), warm, steps)
            two_ms = _time_ms(torch, lambda: psl.sig_to_log_sig(psl.sig(x, N), d, N, method=1), warm, steps)
            load_cusig.set_tile_preference(1)
            try:
                fused_ms = _time_ms(torch, lambda: psl.log_sig(x, N, method=1), warm, steps)
            finally:
                load_cusig.set_tile_preference(0)
        print(json.dumps({"op": "log_sig", "config": {"workload": "log_sig method 1 from the path: float32, B=%d, L=%d, d=%d, degree %d" % (B, L, d, N)},
                          "n_gpus": 1, "steps": steps, "warmup": warm, "dtype": "f32", "data": "synthetic",
                          "sig_ms": sig_ms, "log_sig_ms": one_ms, "log_sig_over_sig": one_ms / sig_ms,
                          "two_public_calls_ms": two_ms, "fused_sweep_forced_ms": fused_ms, "clocks": clocks.summary()}))
        return
    if args.op in ("sig_combine", "sig_join"):
        B, d, N = args.batch or 4096, 16, 4
        S = sum(d ** k for k in range(1, N + 1))
        a, b, g, v = rnd(B, S) * 0.1, rnd(B, S) * 0.1, rnd(B, S), rnd(B, d) * 0.3
        if args.op == "sig_combine":
            fwd, bwd = (lambda: psl.sig_combine(a, b, d, N)), (lambda: psl.sig_combine_backprop(g, a, b, d, N))
            fwd_bytes, bwd_bytes = 3 * B * S * 4, 5 * B * S * 4
        else:
            fwd, bwd = (lambda: psl.sig_join(a, v, d, N)), (lambda: psl.sig_join_backprop(g, a, v, d, N))
            fwd_bytes, bwd_bytes = 2 * B * S * 4, 3 * B * S * 4
        workload = "%s: float32, B=%d signatures of d=%d, degree %d (S=%d)" % (args.op, B, d, N, S)
    elif args.op == "sig_to_log_sig":
        B, d, N = args.batch or 4096, 16, 4
        S = sum(d ** k for k in range(1, N + 1))
        a = rnd(B, S) * 0.1
        M = psl.log_sig_length(d, N)
        g = rnd(B, M)
        psl.prepare_log_sig(d, N, 1)
        fwd = lambda: psl.sig_to_log_sig(a, d, N, method=1)
        bwd = lambda: psl.sig_to_log_sig_backprop(a, g, d, N, method=1)
        fwd_bytes, bwd_bytes = (B * S + B * M) * 4, (2 * B * S + B * M) * 4
        workload = "sig_to_log_sig method 1: float32, B=%d signatures of d=%d, degree %d (S=%d -> %d Lyndon coordinates)" % (B, d, N, S, M)
    elif args.op == "transform_path":
        B, L, d = args.batch or 4096, args.length or 4096, 16
        x = rnd(B, L, d)
        g = rnd(B, 2 * L - 1, 2 * d + 1)
        fwd = lambda: psl.transform_path(x, time_aug=True, lead_lag=True)
        bwd = lambda: psl.transform_path_backprop(g, time_aug=True, lead_lag=True)
        fwd_bytes = bwd_bytes = (B * L * d + B * (2 * L - 1) * (2 * d + 1)) * 4
        workload = "transform_path: float32, B=%d, L=%d, d=%d, time_aug + lead_lag" % (B, L, d)
    else:  # correction
        B, L, d, N = args.batch or 2048, args.length or 256, 4, 4
        S = sum(d ** k for k in range(1, N + 1))
        x = torch.cumsum(rnd(B, L, d) * (1.0 / L) ** 0.5, dim=1).contiguous()
        c = (rnd(B, L - 1, d * d) * 0.05).contiguous()
        s0 = psl.sig(x, N, correction=c)
        g = rnd(B, S)
        fwd = lambda: psl.sig(x, N, correction=c)
        bwd = lambda: psl.sig_backprop(x, s0, g, N, correction=c)
        fwd_bytes = (B * L * d + B * (L - 1) * d * d + B * S) * 4
        bwd_bytes = (2 * B * L * d + B * (L - 1) * d * d + 2 * B * S) * 4
        workload = "sig with level-2 corrections: float32, B=%d, L=%d, d=%d, degree %d" % (B, L, d, N)
        from oracle import refcuda
        if refcuda.available() and not args.no_refcuda:
            ref_s = refcuda.sig(x, N, correction=c)
            extra["max_abs_diff_vs_reference_cuda"] = float((ref_s - s0).abs().max())
            extra["reference_cuda"] = {
                "fwd_ms": _time_ms(torch, lambda: refcuda.sig(x, N, correction=c), 1, 3),
                "bwd_ms": _time_ms(torch, lambda: refcuda.sig_backprop(x, ref_s, g, N, correction=c), 1, 3),
                "what": "reference cu_signature.cu correction kernels compiled for sm_100a, same inputs"}
    warm, steps = max(args.warmup, 3), args.steps
    before = load_cusig.launch_count()
    with ClockSampler(0) as clocks:
        fwd_ms = _time_ms(torch, fwd, warm, steps)
        bwd_ms = _time_ms(torch, bwd, warm, steps)
    launches = (load_cusig.launch_count() - before)
    hbm_peak, note = 6650.0, "fallback"
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            hbm_peak, note = float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        pass
    gbs = lambda nbytes, ms: nbytes / (ms * 1e-3) / 1e9
    line = {"op": args.op, "config": {"workload": workload, "l2": "inputs larger than L2" if fwd_bytes > 3e8 else "inputs fit L2"},
            "n_gpus": 1, "steps": steps, "warmup": warm, "dtype": "f32", "data": "synthetic",
            "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
            "roofline": {"bound": "hbm", "unit": "GB/s", "peak": hbm_peak, "peak_source": note,
                         "forward": {"achieved": gbs(fwd_bytes, fwd_ms), "frac": gbs(fwd_bytes, fwd_ms) / hbm_peak},
                         "backward": {"achieved": gbs(bwd_bytes, bwd_ms), "frac": gbs(bwd_bytes, bwd_ms) / hbm_peak}},
            "clocks": clocks.summary(), "gpu_launches_counted": launches}
    line.update(extra)
    print(json.dumps(line))


def _time_ms(torch, fn, warmup, steps):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / steps


def _level_slices(d, N):
    out, start = [], 0
    for k in range(1, N + 1):
        out.append(slice(start, start + d ** k))
        start += d ** k
    return out


def error_metrics(torch, got, want, d, N, tol, rows=512):
    """Two readings of |got - want| for signatures (batch, S), both per coefficient:
    `scaled`: relative to max(|want|, largest |want| of that level and path), the metric of the
    test-suite; `strict`: relative to |want| itself (coefficients that are exactly 0 in `want`
    are left out), reported as the maximum and as the fraction of coefficients within `tol`."""
    worst_scaled, worst_strict, inside, counted = 0.0, 0.0, 0, 0
    for b0 in range(0, got.shape[0], rows):
        a = got[b0:b0 + rows].double()
        w = want[b0:b0 + rows].double()
        diff = (a - w).abs()
        for sl in _level_slices(d, N):
            floor = w[:, sl].abs().amax(dim=1, keepdim=True).clamp_min(1e-300)
            worst_scaled = max(worst_scaled, float((diff[:, sl] / torch.maximum(w[:, sl].abs(), floor)).max()))
        nz = w != 0
        rel = diff[nz] / w[nz].abs()
        if rel.numel():
            worst_strict = max(worst_strict, float(rel.max()))
            inside += int((rel <= tol).sum())
            counted += rel.numel()
    return {"max_scaled_rel": worst_scaled, "max_strict_rel": worst_strict,
            "frac_strict_within_tol": inside / max(counted, 1), "tol": tol}


def grad_error_metrics(torch, got, want, tol, rows=512):
    """The same two readings for path gradients (batch, L, d); the scale of a path is its largest
    |gradient| entry."""
    worst_scaled, worst_strict, inside, counted = 0.0, 0.0, 0, 0
    for b0 in range(0, got.shape[0], rows):
        a = got[b0:b0 + rows].double().flatten(1)
        w = want[b0:b0 + rows].double().flatten(1)
        diff = (a - w).abs()
        floor = w.abs().amax(dim=1, keepdim=True).clamp_min(1e-300)
        worst_scaled = max(worst_scaled, float((diff / floor).max()))
        nz = w != 0
        rel = diff[nz] / w[nz].abs()
        if rel.numel():
            worst_strict = max(worst_strict, float(rel.max()))
            inside += int((rel <= tol).sum())
            counted += rel.numel()
    return {"max_scaled_rel": worst_scaled, "max_strict_rel": worst_strict,
            "frac_strict_within_tol": inside / max(counted, 1), "tol": tol}


def parity_block(torch, cfg, path, sig, grad, seeds, ref_sig, ref_grad, subset=64):
    """Parity of the results the timed kernels produced (outside the timed region):
    (1) against the reference's own CUDA kernels on the whole shard (when they are built),
    (2) against the float64 CPU oracle on the first `subset` paths, and beside it the same
    numbers for the reference's CUDA kernels, which shows how far two correct float32
    implementations are apart in the strict per-coefficient metric."""
    from oracle import oracle
    ta = bool(cfg.get("time_aug", False))
    d, N = cfg["d"] + (1 if ta else 0), cfg["N"]
    tol = 1e-5 if cfg["dtype"] == "float32" else 1e-10
    out = {"tolerance": tol, "metrics": "max_scaled_rel: |a-b| / max(|b|, largest |b| of the level (signature) or of "
           "the path (gradient)); max_strict_rel: |a-b| / |b| per coefficient; frac_strict_within_tol: share of "
           "coefficients whose strict error is within the tolerance"}
    if ref_sig is not None:
        out["vs_reference_cuda_full_shard"] = {"paths": int(sig.shape[0]),
                                               "forward": error_metrics(torch, sig, ref_sig, d, N, tol)}
        if grad is not None and ref_grad is not None:
            out["vs_reference_cuda_full_shard"]["backward"] = grad_error_metrics(torch, grad, ref_grad, tol)
    n = min(subset, sig.shape[0])
    cores = len(os.sched_getaffinity(0)) or 1
    p64 = path[:n].double().cpu().numpy()
    s64 = oracle.sig(p64, N, n_threads=cores, time_aug=ta)
    want_s = torch.tensor(s64, device=sig.device)
    sub = {"paths": n, "forward_ours": error_metrics(torch, sig[:n], want_s, d, N, tol)}
    if ref_sig is not None:
        sub["forward_reference_cuda"] = error_metrics(torch, ref_sig[:n], want_s, d, N, tol)
    if grad is not None:
        g64 = oracle.sig_backprop(p64, s64, seeds[:n].double().cpu().numpy(), N, n_threads=cores, time_aug=ta)
        want_g = torch.tensor(g64, device=sig.device)
        sub["backward_ours"] = grad_error_metrics(torch, grad[:n], want_g, tol)
        if ref_grad is not None:
            sub["backward_reference_cuda"] = grad_error_metrics(torch, ref_grad[:n], want_g, tol)
        same = oracle.sig_backprop(path[:n].cpu().numpy(), sig[:n].cpu().numpy(), seeds[:n].cpu().numpy(), N,
                                   n_threads=cores, time_aug=ta)
        sub["backward_cpu_port_same_dtype"] = grad_error_metrics(torch, torch.tensor(same, device=sig.device), want_g, tol)
    out["vs_float64_oracle_subset"] = sub
    return out


class L2Flush:
    """Writes a buffer larger than the 126 MB L2 between timed iterations of small workloads."""
    def __init__(self, torch, dev):
        self.buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def __call__(self):
        self.buf.fill_(1)


def time_small_config(torch, name, dev, steps, peak_of, flush, with_refcuda):
    """One of C1-C4 on one GPU, device-resident, L2 flushed between iterations, CUDA events around
    every call on the launching stream; returns the compact record of the `configs` dict."""
    from pysiglib_b200 import load_cusig
    cfg = CONFIGS[name]
    B, L, d, N = cfg["B"], cfg["L"], cfg["d"], cfg["N"]
    dtype = cfg["dtype"]
    real = ctypes.c_float if dtype == "float32" else ctypes.c_double
    S = sum(d ** k for k in range(1, N + 1))
    fwdbwd = cfg["mode"] == "fwdbwd"
    path = make_paths(cfg, B, 1000, torch).to(dev)
    seeds = torch.randn((B, S), generator=torch.Generator().manual_seed(5000), dtype=path.dtype).to(dev) if fwdbwd else None
    sig = torch.empty((B, S), dtype=path.dtype, device=dev)
    grad = torch.empty_like(path) if fwdbwd else None
    ptr = lambda t: ctypes.cast(t.data_ptr(), ctypes.POINTER(real))
    stream = torch.cuda.current_stream(dev)
    sptr = ctypes.c_void_p(stream.cuda_stream)
    fwd_fn, bwd_fn = load_cusig.fn("sigb200_signature", dtype), load_cusig.fn("sigb200_sig_backprop", dtype)

    def fwd():
        rc = fwd_fn(ptr(path), ptr(sig), B, d, L, N, False, False, real(1.0), False, sptr, 0, None)
        assert rc == 0, load_cusig.last_error_message()

    def bwd():
        rc = bwd_fn(ptr(path), ptr(grad), ptr(seeds), ptr(sig), B, d, L, N, False, False, real(1.0), False, sptr, 0)
        assert rc == 0, load_cusig.last_error_message()

    def timed(fn):
        total = 0.0
        for it in range(3 + steps):
            flush()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            fn()
            e1.record(stream)
            e1.synchronize()
            if it >= 3:
                total += e0.elapsed_time(e1)
        return total / steps

    fwd_ms = timed(fwd)
    bwd_ms = timed(bwd) if fwdbwd else None
    i_fwd, f_fwd = instr_forward(d, N)
    peak = peak_of(dtype)
    tf = lambda slots, ms: 2 * slots * (L - 1) * B / (ms * 1e-3) / 1e12
    rec = {"workload": "%s %s B=%d L=%d d=%d degree=%d" % (dtype, "fwd+bwd" if fwdbwd else "fwd", B, L, d, N),
           "fwd_ms": fwd_ms, "frac": tf(i_fwd, fwd_ms) / peak, "frac_fma_only": tf(f_fwd, fwd_ms) / peak,
           "plan": load_cusig.describe_plan(B, d, L, N, dtype=dtype),
           "paths_per_s": B / ((fwd_ms + (bwd_ms or 0.0)) * 1e-3)}
    if fwdbwd:
        i_bwd, _ = instr_backward(d, N)
        i_exe, _ = instr_backward_executed(d, N)
        rec.update({"bwd_ms": bwd_ms, "bwd_frac": tf(i_bwd, bwd_ms) / peak, "bwd_frac_executed": tf(i_exe, bwd_ms) / peak,
                    "bwd_plan": load_cusig.describe_plan(B, d, L, N, dtype=dtype, backward=True)})
        # the configuration as BASELINE.json states it: torch_api.sig under autograd, loss = sig(path).sum()
        from pysiglib_b200 import torch_api
        x = path.clone().requires_grad_(True)

        def autograd_step():
            x.grad = None
            torch_api.sig(x, N).sum().backward()

        rec["torch_api_autograd_ms"] = timed(autograd_step)
        rec["torch_api_paths_per_s"] = B / (rec["torch_api_autograd_ms"] * 1e-3)
    if with_refcuda:
        from oracle import refcuda
        if refcuda.available():
            try:
                ref_sig = torch.empty_like(sig)
                rec["reference_cuda_fwd_ms"] = timed(lambda: refcuda.sig(path, N, out=ref_sig))
                tol = 1e-5 if dtype == "float32" else 1e-10
                rec["parity_fwd_vs_reference_cuda"] = error_metrics(torch, sig, ref_sig, d, N, tol)
                if fwdbwd:
                    ref_grad = torch.empty_like(path)
                    rec["reference_cuda_bwd_ms"] = timed(lambda: refcuda.sig_backprop(path, ref_sig, seeds, N, out=ref_grad))
                    rec["parity_bwd_vs_reference_cuda"] = grad_error_metrics(torch, grad, ref_grad, tol)
            except Exception as exc:
                rec["reference_cuda"] = "unavailable: " + str(exc)[:120]
    return rec


def run_inproc_partitioner(args, cfg, torch):
    """--partitioner inproc: ONE process drives `--gpus` devices through the C-side batch
    partitioner (sigb200_signature_sharded_* / sigb200_sig_backprop_sharded_*: contiguous batch
    slices, one host thread and one stream set per device, no exchange between devices).  Host
    buffers in, host buffers out, so the only number is an end-to-end one."""
    from pysiglib_b200 import load_cusig
    n = args.gpus
    assert torch.cuda.device_count() >= n, "--gpus %d but %d devices visible" % (n, torch.cuda.device_count())
    B, L, d, N = cfg["B"], cfg["L"], cfg["d"], cfg["N"]
    name = cfg["dtype"]
    real = ctypes.c_float if name == "float32" else ctypes.c_double
    S = sum(d ** k for k in range(1, N + 1))
    fwdbwd = cfg["mode"] == "fwdbwd"
    host_path = make_paths(cfg, B, 1000, torch).pin_memory()
    host_sig = torch.empty((B, S), dtype=host_path.dtype).pin_memory()
    host_seeds = torch.randn((B, S), generator=torch.Generator().manual_seed(5000), dtype=host_path.dtype).pin_memory() if fwdbwd else None
    host_grad = torch.empty_like(host_path).pin_memory() if fwdbwd else None
    ptr = lambda t: ctypes.cast(t.data_ptr(), ctypes.POINTER(real))
    fwd = load_cusig.fn("sigb200_signature_sharded", name)
    bwd = load_cusig.fn("sigb200_sig_backprop_sharded", name)

    def step():
        rc = fwd(ptr(host_path), ptr(host_sig), B, d, L, N, False, False, real(1.0), False, None, n)
        assert rc == 0, load_cusig.last_error_message()
        if fwdbwd:
            rc = bwd(ptr(host_path), ptr(host_grad), ptr(host_seeds), ptr(host_sig), B, d, L, N, False, False,
                     real(1.0), False, None, n)
            assert rc == 0, load_cusig.last_error_message()

    for _ in range(max(args.warmup, 3)):
        step()
    before = load_cusig.launch_count()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    esize = 4 if name == "float32" else 8
    path_bytes, sig_bytes = B * L * d * esize, B * S * esize
    value = B * args.steps / dt
    print(json.dumps({
        "metric": "paths_per_second_" + cfg["mode"], "value": value, "unit": "paths/s", "n_gpus": n, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32" if name == "float32" else "f64", "data": "synthetic",
        "partitioner": "inproc: one process, C-side batch partitioner over %d devices, host buffers" % n,
        "config": workload_config(args, cfg, n), "gpu_launches": int(load_cusig.launch_count() - before),
        "e2e": {"value": value, "unit": "paths/s",
                "h2d_bytes_per_step": path_bytes + ((path_bytes + 2 * sig_bytes) if fwdbwd else 0),
                "d2h_bytes_per_step": sig_bytes + (path_bytes if fwdbwd else 0),
                "timer": "host clock around the synchronous sharded C-ABI calls"}}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="sig", choices=["sig", "sig_combine", "sig_join", "sig_to_log_sig", "log_sig", "transform_path", "correction", "fma_patterns"],
                    help="sig (default) is the headline path; the others time one neighbouring operator on one GPU")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", default="C5", choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-refcuda", action="store_true", help="skip timing the reference's own CUDA kernels")
    ap.add_argument("--gather", action="store_true",
                    help="with N > 1 also time one NCCL all-gather of the signatures onto every rank (not part of value)")
    ap.add_argument("--no-configs", action="store_true", help="skip the short C1-C4 records of the default run")
    ap.add_argument("--no-parity", action="store_true", help="skip the parity block")
    ap.add_argument("--partitioner", default="torchrun", choices=["torchrun", "inproc"],
                    help="inproc: ONE process drives --gpus devices through the C-side batch partitioner "
                         "(sigb200_*_sharded_*, host buffers); torchrun (default): one process per GPU")
    ap.add_argument("--batch", type=int, default=None, help="override the batch size (profiling on a small case)")
    ap.add_argument("--length", type=int, default=None, help="override the path length (profiling on a small case)")
    args = ap.parse_args()
    cfg = dict(CONFIGS[args.config])
    if args.batch:
        cfg["B"] = args.batch
    if args.length:
        cfg["L"] = args.length
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, cfg, rank)
        return
    if args.op == "fma_patterns":
        if rank == 0:
            run_fma_patterns(args)
        return
    if args.op != "sig":
        if rank == 0:
            run_neighbour_op(args)
        return

    import torch
    import torch.distributed as dist
    from pysiglib_b200 import load_cusig
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU fallback"
    if args.partitioner == "inproc":
        if rank == 0:
            run_inproc_partitioner(args, cfg, torch)
        return
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    all_cpus = os.sched_getaffinity(0)
    affinity = bind_to_local_cpus(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    warmup = max(args.warmup, 3)

    # this rank's contiguous shard of the batch (remainder to the first ranks)
    chunk, rem = divmod(cfg["B"], world)
    b_local = chunk + (1 if rank < rem else 0)
    d, L, N = cfg["d"], cfg["L"], cfg["N"]
    ta = bool(cfg.get("time_aug", False))
    D = d + (1 if ta else 0)          # dimension the signature is taken in
    name = cfg["dtype"]
    real = ctypes.c_float if name == "float32" else ctypes.c_double
    esize = 4 if name == "float32" else 8
    S = sum(D ** k for k in range(1, N + 1))
    fwdbwd = cfg["mode"] == "fwdbwd"

    host_path = make_paths(cfg, max(b_local, 1), 1000 + rank, torch)[:b_local].pin_memory()
    gen = torch.Generator().manual_seed(5000 + rank)
    host_seeds = torch.randn((b_local, S), generator=gen, dtype=host_path.dtype).pin_memory() if fwdbwd else None
    path = host_path.to(dev)
    seeds = host_seeds.to(dev) if fwdbwd else None
    sig = torch.empty((b_local, S), dtype=path.dtype, device=dev)
    grad = torch.empty_like(path) if fwdbwd else None

    fwd_fn = load_cusig.fn("sigb200_signature", name)
    bwd_fn = load_cusig.fn("sigb200_sig_backprop", name)
    ptr = lambda t: ctypes.cast(t.data_ptr(), ctypes.POINTER(real))
    stream = torch.cuda.current_stream(dev)
    sptr = ctypes.c_void_p(stream.cuda_stream)

    def step_device():
        rc = fwd_fn(ptr(path), ptr(sig), b_local, d, L, N, ta, False, real(1.0), False, sptr, 0, None)
        assert rc == 0, load_cusig.last_error_message()
        if fwdbwd:
            rc = bwd_fn(ptr(path), ptr(grad), ptr(seeds), ptr(sig), b_local, d, L, N, ta, False, real(1.0),
                        False, sptr, 0)
            assert rc == 0, load_cusig.last_error_message()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- FMA-pipe peak of this device, measured here (MEASURED_PEAKS.json has no FP32/FP64 CUDA-core figure) ----
    sink = torch.zeros(2, dtype=torch.float64, device=dev)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    blocks, iters = sms * 8, 2048
    fma_count = blocks * 256 * iters * 64

    bench_lib = ctypes.CDLL(os.path.join(ROOT, "pysiglib_b200", "lib", "libsigb200_bench.so"))
    bench_lib.sigb200_bench_fma_peak.argtypes = (ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p)
    bench_lib.sigb200_bench_fma_peak.restype = ctypes.c_int

    def fma_peak(mode):
        """mode 0: scalar float32 FMA, 1: float64 FMA, 2: packed float32 (fma.rn.f32x2)."""
        best = 0.0
        for i in range(6):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            rc = bench_lib.sigb200_bench_fma_peak(mode, ctypes.c_void_p(sink.data_ptr()), blocks,
                                                  iters // (2 if mode == 1 else 1), sptr)
            assert rc == 0, "FMA peak probe failed with CUDA error %d" % rc
            e1.record(stream)
            e1.synchronize()
            n = fma_count / (2 if mode == 1 else 1)
            if i >= 2:
                best = max(best, n / (e0.elapsed_time(e1) * 1e-3))
        return best  # FMAs per second (per lane)

    peak64 = fma_peak(1)
    peak32_scalar, peak32_packed = fma_peak(0), fma_peak(2)
    if name == "float64":
        peak_scalar = peak_packed = peak64
    else:
        peak_scalar, peak_packed = peak32_scalar, peak32_packed
    # the roofline denominator is the higher of the two float32 issue forms
    peak_fma_per_s = max(peak_scalar, peak_packed)
    peak_tflops_of = lambda dtype: 2 * (peak64 if dtype == "float64" else max(peak32_scalar, peak32_packed)) / 1e12

    # ---- device-resident timing ----
    for _ in range(warmup):
        step_device()
    barrier()
    launches0 = load_cusig.launch_count()
    # workloads smaller than the L2 get it flushed before every timed call (outside the event pairs)
    small = b_local * L * d * esize + b_local * S * esize <= 126e6
    flush = L2Flush(torch, dev) if small else None
    ev_f = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    ev_b = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    with ClockSampler(local) as clocks:
        for k in range(args.steps):
            if flush:
                flush()
            ev_f[k][0].record(stream)
            rc = fwd_fn(ptr(path), ptr(sig), b_local, d, L, N, ta, False, real(1.0), False, sptr, 0, None)
            assert rc == 0, load_cusig.last_error_message()
            ev_f[k][1].record(stream)
            if fwdbwd:
                if flush:
                    flush()
                ev_b[k][0].record(stream)
                rc = bwd_fn(ptr(path), ptr(grad), ptr(seeds), ptr(sig), b_local, d, L, N, ta, False, real(1.0),
                            False, sptr, 0)
                assert rc == 0, load_cusig.last_error_message()
                ev_b[k][1].record(stream)
        barrier()
    launches = load_cusig.launch_count() - launches0
    fwd_ms = sum(a.elapsed_time(b) for a, b in ev_f) / args.steps
    bwd_ms = sum(a.elapsed_time(b) for a, b in ev_b) / args.steps if fwdbwd else 0.0
    total_ms = (fwd_ms + bwd_ms) * args.steps
    t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms_max = float(t.item())
    value = cfg["B"] * args.steps / (total_ms_max * 1e-3)

    # ---- optional: the one collective the path can have, a gather of the per-rank results ----
    gather_ms = None
    if args.gather and world > 1 and cfg["B"] % world == 0:
        full = torch.empty((cfg["B"], S), dtype=sig.dtype, device=dev)
        dist.all_gather_into_tensor(full, sig)
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record(stream)
        for _ in range(3):
            dist.all_gather_into_tensor(full, sig)
        g1.record(stream)
        g1.synchronize()
        gt = torch.tensor([g0.elapsed_time(g1) / 3], dtype=torch.float64, device=dev)
        dist.all_reduce(gt, op=dist.ReduceOp.MAX)
        gather_ms = float(gt.item())
        assert torch.equal(full[rank * b_local:(rank + 1) * b_local], sig)
        del full

    # ---- end to end through the reference-named C-ABI symbols with pinned host buffers ----
    e2e = None
    if not args.no_e2e:
        sig_c = load_cusig.fn("signature_cuda", name)
        bwd_c = load_cusig.fn("sig_backprop_cuda", name)
        host_sig = torch.empty((b_local, S), dtype=host_path.dtype).pin_memory()
        host_grad = torch.empty_like(host_path).pin_memory() if fwdbwd else None

        def step_host():
            rc = sig_c(ptr(host_path), ptr(host_sig), b_local, d, L, N, ta, False, real(1.0), True, False,
                       None, 0, 0, 0)
            assert rc == 0, load_cusig.last_error_message()
            if fwdbwd:
                rc = bwd_c(ptr(host_path), ptr(host_grad), ptr(host_seeds), ptr(host_sig), b_local, d, L, N, ta,
                           False, real(1.0), False, None, 0, 0, 0)
                assert rc == 0, load_cusig.last_error_message()

        e2e_steps = args.steps
        for _ in range(2):
            step_host()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            step_host()
        barrier()
        dt = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        path_bytes, sig_bytes = b_local * L * d * esize, b_local * S * esize
        e2e = {"value": cfg["B"] * e2e_steps / float(dt.item()), "unit": "paths/s",
               "h2d_bytes_per_step": path_bytes + ((path_bytes + 2 * sig_bytes) if fwdbwd else 0),
               "d2h_bytes_per_step": sig_bytes + (path_bytes if fwdbwd else 0),
               "steps": e2e_steps, "warmup": 2, "host_buffers": "pinned, " + affinity,
               "timer": "host clock around synchronous C-ABI calls, device-synchronised, max over ranks"}

    # ---- the reference's own CUDA kernels on the same GPU and inputs (baseline beside ours) ----
    ref_cuda, ref_sig, ref_grad = None, None, None
    if rank == 0 and not args.no_refcuda:
        from oracle import refcuda
        if refcuda.available():
            try:
                ref_sig = torch.empty_like(sig)
                ref_grad = torch.empty_like(path) if fwdbwd else None
                times = []
                for it in range(3):
                    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
                    e0.record(stream)
                    refcuda.sig(path, N, out=ref_sig, time_aug=ta)
                    e1.record(stream)
                    if fwdbwd:
                        refcuda.sig_backprop(path, ref_sig, seeds, N, out=ref_grad, time_aug=ta)
                    e2.record(stream)
                    torch.cuda.synchronize(dev)
                    if it:
                        times.append((e0.elapsed_time(e1), e1.elapsed_time(e2)))
                rf = sum(t[0] for t in times) / len(times)
                rb = sum(t[1] for t in times) / len(times) if fwdbwd else None
                ref_cuda = {"fwd_ms": rf, "bwd_ms": rb, "value": b_local / ((rf + (rb or 0.0)) * 1e-3), "unit": "paths/s",
                            "what": "reference cu_signature.cu kernels compiled for sm_100a, this rank's shard, "
                                    "device-resident, 2 timed repetitions",
                            "max_abs_diff_fwd": float((ref_sig - sig).abs().max().item())}
            except Exception as exc:  # a failing baseline must not take the benchmark down
                ref_cuda = {"unavailable": str(exc)[:200]}
                ref_sig, ref_grad = None, None

    # ---- parity of what the timed kernels produced (outside the timed region) ----
    parity = None
    if rank == 0 and not args.no_parity:
        os.sched_setaffinity(0, all_cpus)  # the CPU checker and the CPU baseline use every host core
        try:
            parity = parity_block(torch, cfg, path, sig, grad, seeds, ref_sig, ref_grad)
        except Exception as exc:
            parity = {"unavailable": str(exc)[:200]}
    del ref_sig, ref_grad

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel ----
    i_fwd, f_fwd = instr_forward(D, N)
    i_bwd, f_bwd = instr_backward(D, N)
    steps_per_path = L - 1
    dominant_bwd = fwdbwd and bwd_ms > fwd_ms

    def roof(instr, fmas, ms, bytes_, direction):
        slots = instr * steps_per_path * b_local
        achieved = 2 * slots / (ms * 1e-3) / 1e12          # FMA-equivalent TFLOP/s: 2 flop per pipe slot
        peak = 2 * peak_fma_per_s / 1e12
        r = {"bound": "fma", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
             "frac_fma_only": (2 * fmas * steps_per_path * b_local / (ms * 1e-3) / 1e12) / peak,
             "traffic": None, "ms_per_launch": ms, "algorithmic_bytes": bytes_,
             "hbm_gbs": bytes_ / (ms * 1e-3) / 1e9, "hbm_frac": bytes_ / (ms * 1e-3) / 1e9 / hbm_peak}
        if (D, N, name) == (16, 4, "float32"):
            small = NCU_SMALL_CASE_TRAFFIC[direction]
            r["traffic"] = small["bytes"]
            r["traffic_note"] = ("ncu small-case figure, NOT this launch: dram bytes read + written by one launch of the "
                                 "same kernel on %s, whose algorithmic bytes are %.0f MB; it is below them because "
                                 "the kernel before it left part of its operands in L2" % (small["case"], small["algorithmic_bytes"] / 1e6))
        return r

    hbm_peak, peak_note = 6650.0, "fallback"
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            hbm_peak, peak_note = float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        pass
    path_bytes, sig_bytes = b_local * L * d * esize, b_local * S * esize
    roof_f = roof(i_fwd, f_fwd, fwd_ms, path_bytes + sig_bytes, "forward")
    roof_f["kernel"] = load_cusig.describe_plan(b_local, d, L, N, dtype=name, time_aug=ta)
    roofline = roof_f
    roof_b = None
    if fwdbwd:
        roof_b = roof(i_bwd, f_bwd, bwd_ms, 2 * path_bytes + 2 * sig_bytes, "backward")
        roof_b["kernel"] = load_cusig.describe_plan(b_local, d, L, N, dtype=name, backward=True, time_aug=ta)
        # the same time against the slots the reverse sweep really issues (no level-N rewind)
        i_exe, f_exe = instr_backward_executed(D, N)
        roof_b["frac_executed"] = roof(i_exe, f_exe, bwd_ms, 0, "backward")["frac"]
        roof_b["slots_per_path_step"] = {"reference_formulation": i_bwd, "executed": i_exe}
        if dominant_bwd:
            roofline = roof_b
    roofline["peak_source"] = ("FMA-pipe peak measured in this run with a register-resident FMA loop: scalar %.1f, "
                               "packed f32x2 %.1f TFLOP/s, the higher one is used; HBM peak %s"
                               % (2 * peak_scalar / 1e12, 2 * peak_packed / 1e12, peak_note))

    out = {
        "metric": "paths_per_second_" + cfg["mode"], "value": value, "unit": "paths/s", "n_gpus": world,
        "steps": args.steps, "warmup": warmup, "ms_per_step": total_ms_max / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32" if name == "float32" else "f64", "data": "synthetic",
        "config": workload_config(args, cfg, world), "clocks": clocks.summary(), "gpu_launches": int(launches),
        "roofline": roofline, "roofline_forward": roof_f, "roofline_backward": roof_b,
        "fwd_ms": fwd_ms, "bwd_ms": bwd_ms if fwdbwd else None,
    }
    if e2e is not None:
        out["e2e"] = e2e
    if parity is not None:
        out["parity"] = parity
    if ref_cuda is not None:
        out["reference_cuda"] = ref_cuda
    if world == 1 and args.config == "C5" and not args.no_configs and not args.batch and not args.length:
        # the other four BASELINE.json configurations in short (each costs milliseconds per step)
        flush = L2Flush(torch, dev)
        out["configs"] = {}
        for other in ("C1", "C2", "C3", "C4"):
            try:
                out["configs"][other] = time_small_config(torch, other, dev, 10, peak_tflops_of, flush,
                                                          not args.no_refcuda)
            except Exception as exc:
                out["configs"][other] = {"unavailable": str(exc)[:200]}
        out["configs"]["timing"] = ("device-resident, 3 warm-up + 10 timed calls each, L2 flushed (256 MB written) "
                                    "between calls, CUDA events on the launching stream")
    if gather_ms is not None:
        out["all_gather"] = {"ms": gather_ms, "bytes_per_rank": b_local * S * esize,
                             "what": "NCCL all_gather_into_tensor of the signatures onto every rank, max over ranks"}
    if not args.no_cpu and world == 1:
        os.sched_setaffinity(0, all_cpus)
        cores = len(os.sched_getaffinity(0)) or 1
        v, n, dt, variant = cpu_baseline(cfg, cores)
        out["cpu_baseline"] = {"value": v, "unit": "paths/s", "cores": cores, "kind": "port",
                               "sample": "%d paths of %s (%s) in %.1f s, %d host threads, %s forward, gcc -O3 "
                                         "-march=native" % (n, args.config, cfg["mode"], dt, cores, variant)}
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
