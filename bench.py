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
kernel against the FMA-pipe peak measured in the same run; `cpu_baseline` times the CPU
oracle (a port of the reference's cpsig arithmetic) on this box's host cores.
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
    """Times the CPU oracle (threaded, static contiguous chunks) on a bounded sample: one path
    per thread is timed first, then as many paths per thread as fit about `target_seconds`."""
    import torch
    from oracle import oracle

    def run(sample):
        path = make_paths(cfg, sample, 99, torch).numpy()
        t0 = time.perf_counter()
        sig = oracle.sig(path, cfg["N"], n_threads=cores)
        if cfg["mode"] == "fwdbwd":
            rng = np.random.default_rng(5)
            seeds = rng.normal(size=sig.shape).astype(path.dtype)
            oracle.sig_backprop(path, sig, seeds, cfg["N"], n_threads=cores)
        return time.perf_counter() - t0

    if paths_per_core is None:
        probe = max(run(cores), 1e-4)
        paths_per_core = int(max(1, min(512, target_seconds / probe)))
    sample = max(1, cores * paths_per_core)
    dt = run(sample)
    return sample / dt, sample, dt


def run_reference_arm(args, cfg, rank):
    """The reference's CPU implementation of the path (its cpsig library cannot be built
    offline, so the port in oracle/ stands in), all host threads, bounded sample per step."""
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    # size one step to about 4 s of wall time on this box, then time exactly `steps` of them
    probe = max(cpu_baseline(cfg, cores, 1)[2], 1e-4)
    per_core = int(max(1, min(512, 4.0 / probe)))
    for _ in range(min(args.warmup, 1)):
        cpu_baseline(cfg, cores, per_core)
    total_paths, total_t = 0, 0.0
    for _ in range(args.steps):
        _, n, dt = cpu_baseline(cfg, cores, per_core)
        total_paths += n
        total_t += dt
    value = total_paths / total_t
    sample = "%d paths of %s per step (%s), %d host threads" % (per_core * cores, args.config, cfg["mode"], cores)
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
            "l2": "inputs larger than L2" if cfg["B"] // world * cfg["L"] * cfg["d"] * 4 > 126e6 else "L2 flushed between steps"}


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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="sig", choices=["sig", "sig_combine", "sig_join", "sig_to_log_sig", "transform_path", "correction"],
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
    if args.op != "sig":
        if rank == 0:
            run_neighbour_op(args)
        return

    import torch
    import torch.distributed as dist
    from pysiglib_b200 import load_cusig
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU fallback"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    warmup = max(args.warmup, 3)

    # this rank's contiguous shard of the batch (remainder to the first ranks)
    chunk, rem = divmod(cfg["B"], world)
    b_local = chunk + (1 if rank < rem else 0)
    d, L, N = cfg["d"], cfg["L"], cfg["N"]
    name = cfg["dtype"]
    real = ctypes.c_float if name == "float32" else ctypes.c_double
    esize = 4 if name == "float32" else 8
    S = sum(d ** k for k in range(1, N + 1))
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
        rc = fwd_fn(ptr(path), ptr(sig), b_local, d, L, N, False, False, real(1.0), False, sptr, 0, None)
        assert rc == 0, load_cusig.last_error_message()
        if fwdbwd:
            rc = bwd_fn(ptr(path), ptr(grad), ptr(seeds), ptr(sig), b_local, d, L, N, False, False, real(1.0),
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

    def fma_peak(mode):
        """mode 0: scalar float32 FMA, 1: float64 FMA, 2: packed float32 (fma.rn.f32x2)."""
        best = 0.0
        for i in range(6):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            load_cusig.library().sigb200_fma_peak(mode, ctypes.c_void_p(sink.data_ptr()), blocks,
                                                  iters // (2 if mode == 1 else 1), sptr)
            e1.record(stream)
            e1.synchronize()
            n = fma_count / (2 if mode == 1 else 1)
            if i >= 2:
                best = max(best, n / (e0.elapsed_time(e1) * 1e-3))
        return best  # FMAs per second (per lane)

    if name == "float64":
        peak_scalar = peak_packed = fma_peak(1)
    else:
        peak_scalar, peak_packed = fma_peak(0), fma_peak(2)
    # the roofline denominator is the higher of the two float32 issue forms
    peak_fma_per_s = max(peak_scalar, peak_packed)

    # ---- device-resident timing ----
    for _ in range(warmup):
        step_device()
    barrier()
    launches0 = load_cusig.launch_count()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * args.steps + 1)]
    with ClockSampler(local) as clocks:
        ev[0].record(stream)
        for k in range(args.steps):
            rc = fwd_fn(ptr(path), ptr(sig), b_local, d, L, N, False, False, real(1.0), False, sptr, 0, None)
            assert rc == 0, load_cusig.last_error_message()
            ev[2 * k + 1].record(stream)
            if fwdbwd:
                rc = bwd_fn(ptr(path), ptr(grad), ptr(seeds), ptr(sig), b_local, d, L, N, False, False, real(1.0),
                            False, sptr, 0)
                assert rc == 0, load_cusig.last_error_message()
            ev[2 * k + 2].record(stream)
        barrier()
    launches = load_cusig.launch_count() - launches0
    total_ms = ev[0].elapsed_time(ev[-1])
    fwd_ms = sum(ev[2 * k].elapsed_time(ev[2 * k + 1]) for k in range(args.steps)) / args.steps
    bwd_ms = sum(ev[2 * k + 1].elapsed_time(ev[2 * k + 2]) for k in range(args.steps)) / args.steps
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
            rc = sig_c(ptr(host_path), ptr(host_sig), b_local, d, L, N, False, False, real(1.0), True, False,
                       None, 0, 0, 0)
            assert rc == 0, load_cusig.last_error_message()
            if fwdbwd:
                rc = bwd_c(ptr(host_path), ptr(host_grad), ptr(host_seeds), ptr(host_sig), b_local, d, L, N, False,
                           False, real(1.0), False, None, 0, 0, 0)
                assert rc == 0, load_cusig.last_error_message()

        e2e_steps = min(args.steps, 3)
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
               "steps": e2e_steps, "timer": "host clock around synchronous C-ABI calls, device-synchronised, max over ranks"}

    # ---- the reference's own CUDA kernels on the same GPU and inputs (baseline beside ours) ----
    ref_cuda = None
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
                    refcuda.sig(path, N, out=ref_sig)
                    e1.record(stream)
                    if fwdbwd:
                        refcuda.sig_backprop(path, ref_sig, seeds, N, out=ref_grad)
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
                del ref_sig, ref_grad
            except Exception as exc:  # a failing baseline must not take the benchmark down
                ref_cuda = {"unavailable": str(exc)[:200]}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel ----
    i_fwd, f_fwd = instr_forward(d, N)
    i_bwd, f_bwd = instr_backward(d, N)
    steps_per_path = L - 1
    dominant_bwd = fwdbwd and bwd_ms > fwd_ms

    def roof(instr, fmas, ms, bytes_):
        slots = instr * steps_per_path * b_local
        achieved = 2 * slots / (ms * 1e-3) / 1e12          # FMA-equivalent TFLOP/s: 2 flop per pipe slot
        peak = 2 * peak_fma_per_s / 1e12
        return {"bound": "fma", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "frac_fma_only": (2 * fmas * steps_per_path * b_local / (ms * 1e-3) / 1e12) / peak,
                "traffic": None, "ms_per_launch": ms,
                "hbm_gbs": bytes_ / (ms * 1e-3) / 1e9, "hbm_frac": bytes_ / (ms * 1e-3) / 1e9 / hbm_peak}

    hbm_peak, peak_note = 6650.0, "fallback"
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            hbm_peak, peak_note = float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        pass
    path_bytes, sig_bytes = b_local * L * d * esize, b_local * S * esize
    roof_f = roof(i_fwd, f_fwd, fwd_ms, path_bytes + sig_bytes)
    roof_f["kernel"] = load_cusig.describe_plan(b_local, d, L, N, dtype=name)
    roofline = roof_f
    roof_b = None
    if fwdbwd:
        roof_b = roof(i_bwd, f_bwd, bwd_ms, 2 * path_bytes + 2 * sig_bytes)
        roof_b["kernel"] = load_cusig.describe_plan(b_local, d, L, N, dtype=name, backward=True)
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
    if ref_cuda is not None:
        out["reference_cuda"] = ref_cuda
    if gather_ms is not None:
        out["all_gather"] = {"ms": gather_ms, "bytes_per_rank": b_local * S * esize,
                             "what": "NCCL all_gather_into_tensor of the signatures onto every rank, max over ranks"}
    if not args.no_cpu and world == 1:
        cores = os.cpu_count() or 1
        v, n, dt = cpu_baseline(cfg, cores)
        out["cpu_baseline"] = {"value": v, "unit": "paths/s", "cores": cores, "kind": "port",
                               "sample": "%d paths of %s (%s) in %.1f s, %d host threads" % (n, args.config, cfg["mode"], dt, cores)}
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
