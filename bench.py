#!/usr/bin/env python3
"""Benchmark of the batched C2C FFT hot path: the logN + logBS = 28 sweep.

One step = one pass over the reference's `--if_bench 2` shape (main.cu:117-127):
for logN = lo..hi, a forward FFT of batch = 2^(log_total - logN) signals of length 2^logN.
Metric = GFLOPS with the reference's formula 5*N*log2(N)*batch / t (main.cu:68), summed
over the sweep; HBM GB/s uses the reference's algorithmic bytes 2*N*batch*sizeof(T)
(main.cu:69).  Prints ONE JSON line.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                  [--datatype 0|1] [--ft 0|1|2] [--thread_bs B] [--lo 7] [--hi 24]
                  [--log-total 28] [--cufft] [--no-e2e] [--no-cpu] [--no-also]

Besides the headline (complex64 sweep, FT off) the line carries an "also" object measured
outside the timed region of the headline: on one GPU the complex128 sweep, the FT detect and
FT inject+correct overheads at thread_bs 8 and the cuFFT comparison; on several GPUs one
record per distributed transform (2^30 complex64 and 2^29 complex128, four-step, FT on).

N > 1 is launched with torch.distributed.run, one rank per GPU; the batch is sharded
(every rank transforms its own 2^log_total elements per point, no data-path collective).
--impl reference times the CPU port of the same sweep on the host cores (the reference
has no CPU implementation; see oracle/cpu_fft.py).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "c2c_fft_gflops_logN_plus_logBS_28_sweep"
FALLBACK_HBM_GBS = 6650.0
L2_BYTES = 126 * 1024 * 1024


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--datatype", type=int, default=0, help="0 float2 (complex64), 1 double2 (complex128)")
    ap.add_argument("--ft", type=int, default=0, help="0 off, 1 detect (--if_ft), 2 inject+correct (--if_err)")
    ap.add_argument("--thread_bs", type=int, default=0, help="tiles per block; 0 = the tuned value of each size (param/B200/thread_bs_*.csv)")
    ap.add_argument("--lo", type=int, default=7)
    ap.add_argument("--hi", type=int, default=24)
    ap.add_argument("--log-total", type=int, default=28)
    ap.add_argument("--cufft", action="store_true", help="also time cuFFT on the same buffers (comparison only)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--single-pass", type=int, default=None,
                    help="sizes with a single-pass (cluster) kernel use it, with 2^(value & 15) CTAs per cluster "
                         "(-1 = default size; +16 prefetching variant, +32 radix-8 variant); for profiling and comparison")
    ap.add_argument("--fuse-launches", type=int, default=None, metavar="LOG_CHUNK_BYTES",
                    help="two-launch sizes with a fused kernel run as ONE persistent kernel with chunks of 2^value bytes "
                         "(tfft_plan_fuse_launches, lag 1); for profiling and comparison")
    ap.add_argument("--param-csv", default=None, help="plans from this parameter file instead of the built-in tables")
    ap.add_argument("--no-also", action="store_true", help="skip the secondary measurements of the 'also' object")
    ap.add_argument("--also-steps", type=int, default=5)
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--cpu-log-sample", type=int, default=28, help="log2 elements per sweep point in the CPU sample")
    ap.add_argument("--workload", default="sweep", choices=["sweep", "fourstep", "cfg1", "cfg4"],
                    help="sweep: the logN+logBS=28 batch sweep (default); fourstep: ONE transform of 2^--logN points "
                         "distributed over the GPUs (four-step, all-to-all over NVLink)")
    ap.add_argument("--logN", type=int, default=30, help="fourstep: log2 of the transform length")
    ap.add_argument("--natural", type=int, default=0, help="fourstep: 1 = natural-order output (third exchange)")
    ap.add_argument("--exchange", default="stores", choices=["stores", "dma"],
                    help="fourstep, fused, pipelined: peer stores from the transposing kernel, or pack + copy-engine copies")
    ap.add_argument("--pipeline", type=int, default=8, help="fourstep, fused: pieces per exchange overlapped with the local transforms")
    ap.add_argument("--fused", type=int, default=1, help="fourstep: 1 = exchanges fused into peer-storing kernels, "
                                                         "0 = NCCL all-to-all between local kernels")
    return ap.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def workload_name(a):
    dt = "complex64 uniform[-1,1)" if a.datatype == 0 else "complex128 N(0,1)"
    ft = {0: "FT off", 1: "FT detect", 2: "FT inject+correct"}[a.ft]
    return (f"cfg2 sweep: logN={a.lo}..{a.hi}, batch=2^({a.log_total}-logN), {dt}, forward unnormalised, {ft}"
            if a.datatype == 0 else
            f"cfg3 sweep: logN={a.lo}..{a.hi}, batch=2^({a.log_total}-logN), {dt}, forward unnormalised, {ft}")


def flops_of_point(logn, log_total):
    return 5.0 * (1 << log_total) * logn


# ----------------------------------------------------------------------------- CPU arm


def make_host_input(n_complex, datatype, seed):
    import numpy as np

    rng = np.random.default_rng(seed)
    if datatype == 0:
        return rng.uniform(-1.0, 1.0, size=2 * n_complex).astype(np.float32).view(np.complex64)
    return rng.standard_normal(size=2 * n_complex).view(np.complex128)


def config_of(a):
    """The workload description both arms print (identical, so the two lines compare like for like)."""
    n, esize = 1 << a.log_total, 8 if a.datatype == 0 else 16
    return {"workload": workload_name(a), "thread_bs": a.thread_bs if a.thread_bs else "per size, the tuned table (1, except 8 for the SM-filling single launch of 2^14 complex64)",
            "l2": f"inputs larger than L2 ({int(n * esize) >> 20} MiB per point vs {L2_BYTES >> 20} MiB)",
            "sharding": "batch sharded, each GPU its own 2^%d elements per point, no collective" % a.log_total}


def cpu_sweep(a, x=None):
    """Times the CPU port on 2^cpu_log_sample elements per sweep point (2^28 = the whole workload)."""
    from oracle import cpu_fft

    workers = cpu_fft.host_threads()
    ls = min(a.cpu_log_sample, a.log_total)
    if x is None:
        x = make_host_input(1 << ls, a.datatype, 1)
    total_t, total_f, per = 0.0, 0.0, []
    for logn in range(a.lo, a.hi + 1):
        if logn > ls:
            continue
        xs = x.reshape(1 << (ls - logn), 1 << logn)
        t0 = time.perf_counter()
        cpu_fft.cpu_fft(xs, workers)
        dt = time.perf_counter() - t0
        total_t += dt
        total_f += 5.0 * (1 << ls) * logn
        per.append((logn, dt))
    return total_f / total_t / 1e9, total_t, workers, ls, per


def cpu_sample_text(a, ls, workers, speedup):
    part = "the whole batch" if ls >= a.log_total else f"1/{1 << (a.log_total - ls)} of the batch"
    return (f"2^{ls} elements per sweep point ({part}), scipy.fft (pocketfft) with {workers} threads "
            f"(measured {speedup:.1f}x over one thread)")


def run_reference(a):
    """Reference arm: the CPU port of the path on every host core; rank 0 alone works."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from oracle import cpu_fft

    speedup = cpu_fft.thread_speedup()
    ls = min(a.cpu_log_sample, a.log_total)
    x = make_host_input(1 << ls, a.datatype, 1)
    for _ in range(max(0, a.warmup)):
        cpu_sweep(a, x)
    t_all, f_all = 0.0, 0.0
    for _ in range(a.steps):
        gf, t, workers, ls, _ = cpu_sweep(a, x)
        t_all += t
        f_all += gf * t
    value = f_all / t_all
    sample = cpu_sample_text(a, ls, workers, speedup)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GFLOPS", "n_gpus": a.gpus,
        "steps": a.steps, "warmup": a.warmup, "ms_per_step": 1e3 * t_all / a.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32" if a.datatype == 0 else "f64", "data": "synthetic",
        "config": config_of(a),
        "cpu_baseline": {"value": value, "unit": "GFLOPS", "cores": workers, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference ships no CPU implementation of the transform; this is a CPU port (pocketfft)",
    }
    print(json.dumps(line))
    return 0


# ----------------------------------------------------------------------------- clocks


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML (read only)."""

    def __init__(self, uuid, index, period=0.01):
        super().__init__(daemon=True)
        self.period = period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml

            self.nv = pynvml
            pynvml.nvmlInit()
            try:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80): "hw_power_brake_slowdown",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop_evt.wait(self.period)

    def stop(self):
        self._stop_evt.set()
        if self.ok:
            self.join(timeout=2)
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


# ----------------------------------------------------------------------------- secondary legs


def time_sweep(torch, plans, points, x, y, stream, steps, warmup=3):
    """K sweeps back to back with per-point events; returns (ms per sweep, [ms per point])."""
    for _ in range(warmup):
        for logn in points:
            plans[logn].exec_ptr(x.data_ptr(), y.data_ptr(), stream)
    torch.cuda.synchronize()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(len(points) + 1)] for _ in range(steps)]
    for k in range(steps):
        evs[k][0].record()
        for i, logn in enumerate(points):
            plans[logn].exec_ptr(x.data_ptr(), y.data_ptr(), stream)
            evs[k][i + 1].record()
    torch.cuda.synchronize()
    per = [sum(ev[i].elapsed_time(ev[i + 1]) for ev in evs) / steps for i in range(len(points))]
    return sum(per), per


def cufft_sweep(a, torch, tf, points, log_total, datatype, x, y, stream, steps, offline_abft):
    """cuFFT on the same buffers with the same protocol (comparison only, separate library)."""
    import ctypes as C

    cmp = C.CDLL(os.path.join(os.path.dirname(tf.__file__), "libturbofft_cufft_cmp.so"))
    cmp.tfft_cmp_cufft_plan_create.argtypes = [C.c_int, C.c_longlong, C.c_int, C.c_void_p, C.POINTER(C.c_int)]
    cmp.tfft_cmp_cufft_plan_exec.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    handles = {}
    for logn in points:
        h = C.c_int(0)
        if cmp.tfft_cmp_cufft_plan_create(logn, 1 << (log_total - logn), datatype, stream, C.byref(h)) == 0:
            handles[logn] = h.value

    class _P:
        def __init__(self, h):
            self.h = h

        def exec_ptr(self, xi, yo, st):
            if self.h is not None:
                cmp.tfft_cmp_cufft_plan_exec(self.h, datatype, xi, yo)

    tot, per = time_sweep(torch, {l: _P(handles.get(l)) for l in points}, points, x, y, stream, steps)
    for h in handles.values():
        cmp.tfft_cmp_cufft_plan_destroy(h)
    out = {"ms_per_step": tot, "gflops": sum(flops_of_point(l, log_total) for l in points) / tot / 1e6,
           "per_point_ms": {str(l): (round(ms, 4) if l in handles else None) for l, ms in zip(points, per)},
           "protocol": "same as ours: warm-up sweeps, then %d sweeps back to back" % steps}
    if offline_abft:
        # cuFFT with offline (unfused) ABFT around it: the FT-without-fusion comparison point
        cmp.tfft_cmp_cufft_offline_abft.argtypes = [C.c_int, C.c_longlong, C.c_int, C.c_void_p, C.c_void_p, C.c_int,
                                                    C.POINTER(C.c_float), C.POINTER(C.c_uint), C.c_void_p]
        tot_ft, per_ft = 0.0, []
        for logn in points:
            ms, bad = C.c_float(0), C.c_uint(0)
            rc = cmp.tfft_cmp_cufft_offline_abft(logn, 1 << (log_total - logn), datatype, x.data_ptr(), y.data_ptr(), 3,
                                                 C.byref(ms), C.byref(bad), stream)
            per_ft.append({"logN": logn, "ms": round(ms.value, 4) if rc == 0 else None, "failed_checks": bad.value})
            tot_ft += ms.value if rc == 0 else float("nan")
        out["offline_abft"] = {"ms_per_step": tot_ft, "overhead_vs_cufft_pct": 100 * (tot_ft / tot - 1), "per_point": per_ft}
    return out


def also_single_gpu(a, torch, tf, dev, x, y, stream, points, ours_ms, ours_per, peak):
    """Secondary single-GPU measurements (outside the headline's timed region): cuFFT on the same
    sweep, the FT overheads at thread_bs 8 against the headline, and the complex128 sweep."""
    steps, lt = max(1, a.also_steps), a.log_total
    n = 1 << lt
    flops = sum(flops_of_point(l, lt) for l in points)
    also = {"steps": steps, "note": "measured after the headline, same process, inputs resident in HBM"}
    cu = cufft_sweep(a, torch, tf, points, lt, a.datatype, x, y, stream, steps, a.cufft)
    cu["ours_over_cufft_speed"] = cu["ms_per_step"] / ours_ms
    cu["per_point_ours_over_cufft_speed"] = {str(l): (round(cu["per_point_ms"][str(l)] / o, 3) if cu["per_point_ms"][str(l)] else None)
                                             for l, o in zip(points, ours_per)}
    also["cufft"] = cu
    ft = {"thread_bs": "per size, the tuned table (plans created with thread_bs = 0)",
          "baseline": "the headline sweep (FT off)"}
    for name, if_err in (("detect", 0), ("inject_correct", 1)):
        plans = {l: tf.Plan(l, 1 << (lt - l), a.datatype, if_ft=1, if_err=if_err, thread_bs=0, device=dev.index) for l in points}
        ms, per = time_sweep(torch, plans, points, x, y, stream, steps)
        nd, nc, loc = plans[points[-1]].ft_status()
        ft[name] = {"ms_per_step": ms, "overhead_pct": 100 * (ms / ours_ms - 1),
                    "per_point_overhead_pct": {str(l): round(100 * (m / o - 1), 1) for l, m, o in zip(points, per, ours_per)},
                    "last_point": {"logN": points[-1], "blocks": len(loc), "detected": nd, "corrected": nc}}
        for p in plans.values():
            p.destroy()
    also["ft"] = ft
    # the other datatype's sweep (config 3 when the headline is config 2)
    other = 1 - a.datatype
    rd = torch.float32 if other == 0 else torch.float64
    es = 8 if other == 0 else 16
    g = torch.Generator(device=dev).manual_seed(3)
    if other == 1:
        xo = torch.view_as_complex(torch.randn(n, 2, generator=g, device=dev, dtype=rd))
    else:
        xo = torch.view_as_complex(torch.rand(n, 2, generator=g, device=dev, dtype=rd) * 2 - 1)
    yo = torch.empty_like(xo)
    plans = {l: tf.Plan(l, 1 << (lt - l), other, thread_bs=a.thread_bs, device=dev.index) for l in points}
    ms, per = time_sweep(torch, plans, points, xo, yo, stream, steps)
    gbs = 2.0 * n * es * len(points) / (ms * 1e-3) / 1e9
    rec = {"workload": ("cfg3" if other == 1 else "cfg2") + " sweep, " + ("complex128 N(0,1)" if other == 1 else "complex64 uniform[-1,1)"),
           "ms_per_step": ms, "gflops": flops / ms / 1e6, "hbm_gbs_algorithmic": gbs, "frac_of_peak": gbs / peak,
           "per_point_ms": {str(l): round(m, 4) for l, m in zip(points, per)}}
    for p in plans.values():
        p.destroy()
    cu = cufft_sweep(a, torch, tf, points, lt, other, xo, yo, stream, steps, False)
    rec["cufft_ms_per_step"] = cu["ms_per_step"]
    rec["ours_over_cufft_speed"] = cu["ms_per_step"] / ms
    also["f64_sweep" if other == 1 else "f32_sweep"] = rec
    return also


def fourstep_record(a, torch, tf, dist, dev, world, rank, logn, datatype, ft, steps):
    """One distributed transform (BASELINE config 5): time, Parseval and sampled output bins against
    the CPU oracle's direct sum (each rank sums its own rows on the host, shares are added)."""
    import numpy as np

    from oracle import fft_oracle as orc
    from turbofft_b200 import multi_gpu as mg

    rdtype = torch.float32 if datatype == 0 else torch.float64
    esize = 8 if datatype == 0 else 16
    n = 1 << logn
    n_local = n // world
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    x = torch.view_as_complex(torch.rand(n_local, 2, generator=g, device=dev, dtype=rdtype) * 2 - 1)
    fs = mg.FusedFourStepFFT(logn, world, rank, datatype, dev.index, natural_order=False, if_ft=int(ft >= 1), if_err=int(ft == 2),
                             thread_bs=a.thread_bs, pipeline=a.pipeline, exchange="stores")
    for _ in range(3):
        y = fs(x)
    dist.barrier()
    torch.cuda.synchronize()
    fs.ft_counts()  # clears what the warm-up counted
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        y = fs(x)
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    nd, nc = fs.ft_counts() if ft else (0, 0)
    ex = (x.real.double() ** 2 + x.imag.double() ** 2).sum()
    ey = (y.real.double() ** 2 + y.imag.double() ** 2).sum()
    # sampled bins: X[k1 + N1 k2] sits at rank k1 // (N1/P), local [k1 % (N1/P)][k2]
    n1, n2 = 1 << fs.l1, 1 << fs.l2
    n1l = n1 // world
    bins = np.random.default_rng(7).integers(0, n, size=8)
    got = torch.zeros(len(bins), dtype=torch.complex128, device=dev)
    yl = y.view(n1l, n2)
    for i, k in enumerate(bins):
        k1, k2 = int(k) % n1, int(k) // n1
        if k1 // n1l == rank:
            got[i] = yl[k1 % n1l, k2].to(torch.complex128)
    inner = torch.from_numpy(orc.dft_bins_partial(x.cpu().numpy(), rank * n1l, n1, n2, bins)).to(dev)
    stats = torch.stack([torch.tensor(ms, device=dev, dtype=torch.float64), ex, ey])
    tmax = stats[:1].clone()
    dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    sums = stats[1:].clone()
    dist.all_reduce(sums, op=dist.ReduceOp.SUM)
    gr, ir = torch.view_as_real(got).contiguous(), torch.view_as_real(inner).contiguous()
    dist.all_reduce(gr, op=dist.ReduceOp.SUM)
    dist.all_reduce(ir, op=dist.ReduceOp.SUM)
    fs.close()
    ms, ex, ey = float(tmax[0]), float(sums[0]), float(sums[1])
    ref = orc.dft_bins_finish(torch.view_as_complex(ir).cpu().numpy(), n1, n2, bins)
    gotn = torch.view_as_complex(gr).cpu().numpy()
    exch = (world - 1) / world * n * esize / world
    return {"workload": f"cfg5: one 2^{logn}-point {'complex64' if datatype == 0 else 'complex128'} transform as 2^{fs.l1} x 2^{fs.l2}, "
                        f"four-step over {world} GPUs, transposed output, FT {'on' if ft else 'off'}, exchanges fused into "
                        f"peer-storing transpose kernels, {a.pipeline} pieces pipelined",
            "ms": ms, "gflops": 5.0 * n * logn / (ms * 1e-3) / 1e9, "steps": steps, "exchanges": 2,
            "nvlink_bytes_per_exchange_per_gpu": int(exch),
            "nvlink_gbs_per_gpu_if_the_exchanges_filled_the_whole_time": 2 * exch / (ms * 1e-3) / 1e9,
            "parseval_rel_err": abs(ey / (n * ex) - 1.0),
            "sampled_bins": {"count": int(len(bins)), "rel_l2_vs_cpu_direct_sum": float(np.linalg.norm(gotn - ref) / np.linalg.norm(ref)),
                             "tolerance": (1e-6 if datatype == 0 else 1e-14) * logn},
            "ft": {"detected": nd, "corrected": nc} if ft else None}


# ----------------------------------------------------------------------------- GPU arm


def run_ours(a):
    import ctypes as C

    import torch

    import turbofft_b200 as tf

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the FFT has no CPU path (use --impl reference for the CPU port)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    tf.lib()  # fails loudly if the CUDA library is missing

    tdtype = torch.complex64 if a.datatype == 0 else torch.complex128
    esize = 8 if a.datatype == 0 else 16
    n = 1 << a.log_total
    points = list(range(a.lo, a.hi + 1))
    alg_bytes_point = 2.0 * n * esize

    # seeded synthetic input, generated on the host (pinned) and copied once
    host_np = make_host_input(n, a.datatype, seed=rank)
    host_in = torch.from_numpy(host_np).pin_memory()
    x = host_in.to(dev, non_blocking=True)
    y = torch.empty_like(x)
    torch.cuda.synchronize()

    plans = {}
    for logn in points:
        if a.single_pass is not None and not a.ft:
            try:
                plans[logn] = tf.Plan(logn, 1 << (a.log_total - logn), a.datatype, thread_bs=max(1, a.thread_bs), device=local,
                                      single_pass=a.single_pass)
                continue
            except tf.TurboFFTError:
                pass  # no single-pass kernel of that size or cluster size: the launches
        plans[logn] = tf.Plan(logn, 1 << (a.log_total - logn), a.datatype, if_ft=int(a.ft >= 1), if_err=int(a.ft == 2),
                              thread_bs=a.thread_bs, device=local, param_csv=a.param_csv)
        if a.fuse_launches is not None and not a.ft:
            try:
                plans[logn].fuse_launches(max(0, a.fuse_launches - logn - (3 if a.datatype == 0 else 4)), 1)
            except tf.TurboFFTError:
                pass  # not a two-launch plan, or no fused kernel of its two launch shapes
    stream = torch.cuda.current_stream().cuda_stream

    def step(events=None):
        for i, logn in enumerate(points):
            plans[logn].exec_ptr(x.data_ptr(), y.data_ptr(), stream)
            if events is not None:
                events[i + 1].record()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # same-run STREAM-copy peak
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(3):
        tf.stream_copy(x, y)
    torch.cuda.synchronize()
    ev0.record()
    for _ in range(10):
        tf.stream_copy(x, y)
    ev1.record()
    torch.cuda.synchronize()
    copy_gbs = 2.0 * n * esize * 10 / (ev0.elapsed_time(ev1) * 1e-3) / 1e9

    for _ in range(max(a.warmup, 3)):
        step()
    barrier()

    try:
        uuid = "GPU-" + str(torch.cuda.get_device_properties(local).uuid)
    except Exception:
        uuid = None
    sampler = ClockSampler(uuid, local)
    if sampler.ok:
        sampler.start()

    # ---- timed region: K steps, device-timed, per-point events
    launches0 = tf.launch_count()
    all_events = [[torch.cuda.Event(enable_timing=True) for _ in range(len(points) + 1)] for _ in range(a.steps)]
    barrier()
    for k in range(a.steps):
        all_events[k][0].record()
        step(all_events[k])
    barrier()
    launches = tf.launch_count() - launches0
    total_ms = sum(ev[0].elapsed_time(ev[-1]) for ev in all_events)
    clocks = sampler.stop() if sampler.ok else {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}

    t_local = total_ms / a.steps
    if dist is not None:
        t = torch.tensor([t_local], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_step = float(t.item())
    else:
        t_step = t_local

    flops_step = sum(flops_of_point(l, a.log_total) for l in points)
    value = world * flops_step / (t_step * 1e-3) / 1e9
    per_point = []
    for i, logn in enumerate(points):
        ms = sum(ev[i].elapsed_time(ev[i + 1]) for ev in all_events) / a.steps
        per_point.append({"logN": logn, "ms": round(ms, 4), "gflops": round(flops_of_point(logn, a.log_total) / ms / 1e6, 1),
                          "gbs": round(alg_bytes_point / ms / 1e6, 1), "launches": len(plans[logn].info())})

    # ---- property check on the last point's output (no oracle here): Parseval
    logn_chk = points[-1]
    plans[logn_chk].exec_ptr(x.data_ptr(), y.data_ptr(), stream)
    torch.cuda.synchronize()
    ex = float((x.real.double() ** 2 + x.imag.double() ** 2).sum().item())
    ey = float((y.real.double() ** 2 + y.imag.double() ** 2).sum().item())
    parseval = abs(ey / ((1 << logn_chk) * ex) - 1.0)

    ft_info = None
    if a.ft:
        nd, nc, loc = plans[logn_chk].ft_status()
        ft_info = {"logN": logn_chk, "blocks": len(loc), "detected": nd, "corrected": nc}

    # ---- end to end through the public host-buffer API (tfft_exec_host)
    e2e = None
    if not a.no_e2e:
        host_out = torch.empty_like(host_in).pin_memory()
        # one untimed sweep through the same call: every plan builds its chunk plans, streams and
        # staging slots on first use
        for logn in points:
            plans[logn].exec_host(host_in, host_out)
        barrier()
        t0 = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        # the sweep points of a step are queued back to back (tfft_exec_host_async) and the step ends with
        # tfft_host_sync: the copy pipeline stays full across the points instead of draining after each
        for _ in range(a.e2e_steps):
            for logn in points:
                plans[logn].exec_host_async(host_in, host_out)
            tf.host_sync(dev.index)
        e1.record()
        torch.cuda.synchronize()
        e_ms = e0.elapsed_time(e1) / a.e2e_steps
        if dist is not None:
            t = torch.tensor([e_ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e_ms = float(t.item())
        e2e = {"value": world * flops_step / (e_ms * 1e-3) / 1e9, "unit": "GFLOPS",
               "h2d_bytes_per_step": int(len(points) * n * esize), "d2h_bytes_per_step": int(len(points) * n * esize),
               "steps": a.e2e_steps, "ms_per_step": e_ms, "api": "tfft_exec_host_async per sweep point + tfft_host_sync per step (pinned host buffers)",
               "pcie_gbs_per_direction": len(points) * n * esize / (e_ms * 1e-3) / 1e9}
        # what this host and link give two plain concurrent copies (one per direction), for scale
        s_up, s_dn = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        half = host_in.numel() // 2
        d_up, d_dn = torch.empty_like(x[:half]), x[half:2 * half]
        torch.cuda.synchronize()
        best = None
        for _ in range(3):
            t0 = time.perf_counter()
            with torch.cuda.stream(s_up):
                d_up.copy_(host_in[:half], non_blocking=True)
            with torch.cuda.stream(s_dn):
                host_out[:half].copy_(d_dn, non_blocking=True)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        e2e["pcie_duplex_copy_gbs_per_direction_same_run"] = half * esize / best / 1e9

    peak, peak_src = peaks()
    # ---- secondary measurements, outside every timed region above
    also = None
    if not a.no_also:
        ours_per = [sum(ev[i].elapsed_time(ev[i + 1]) for ev in all_events) / a.steps for i in range(len(points))]
        for p in plans.values():
            p.destroy()
        n_launches_of = {p["logN"]: p["launches"] for p in per_point}
        if world == 1:
            also = also_single_gpu(a, torch, tf, dev, x, y, stream, points, sum(ours_per), ours_per, peak)
        else:
            del x, y
            torch.cuda.empty_cache()
            also = {"note": "distributed single transforms, measured after the headline in the same job",
                    "fourstep": [fourstep_record(a, torch, tf, dist, dev, world, rank, 30, 0, 1, max(1, a.also_steps)),
                                 fourstep_record(a, torch, tf, dist, dev, world, rank, 29, 1, 1, max(1, a.also_steps))]}

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return 0

    achieved = alg_bytes_point * len(points) / (t_local * 1e-3) / 1e9
    dominant = max(per_point, key=lambda p: p["ms"])
    roofline = {
        "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
        # DRAM bytes per step: every launch moves its whole batch once; ncu measured 0.95 x the
        # algorithmic bytes per launch on 2^26-element cases (profiles/fft_kernel_fp32_logN16_two_launch.txt,
        # ..._logN12_single_launch.txt), scaled here by elements and by the launches per step
        "traffic": 0.95 * alg_bytes_point * sum(p["launches"] for p in per_point),
        "traffic_note": "per step = 0.95 x algorithmic bytes per launch (ncu, 2^26-element captures, scaled) x launches per step",
        "algorithmic_bytes_per_step": alg_bytes_point * len(points),
        "peak_source": peak_src, "stream_copy_gbs_same_run": copy_gbs, "frac_of_same_run_copy": achieved / copy_gbs,
        "kernel": "tfft::fft_kernel<T,LOGM,LOGE,LOGC,ROLE,FT> (every launch of the sweep is an instance)",
        "algorithmic_bytes_per_point": alg_bytes_point,
        "dominant_point": dominant,
        "per_point": per_point,
    }
    cpu = None
    if not a.no_cpu and world == 1:  # the host baseline is a single-GPU-run figure; rank 0 of a larger job skips it
        from oracle import cpu_fft

        speedup = cpu_fft.thread_speedup()
        cpu_sweep(a, host_np)  # warms the thread pool and the allocator
        gf, t, workers, ls, _ = cpu_sweep(a, host_np)
        cpu = {"value": gf, "unit": "GFLOPS", "cores": workers, "kind": "port",
               "sample": cpu_sample_text(a, ls, workers, speedup) + f", one pass after a warm-up pass, {t:.1f} s"}
    line = {
        "metric": METRIC, "value": value, "unit": "GFLOPS", "n_gpus": world, "steps": a.steps, "warmup": max(a.warmup, 3),
        "ms_per_step": t_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32" if a.datatype == 0 else "f64", "data": "synthetic",
        "config": config_of(a),
        "hbm_gbs_algorithmic": achieved,
        "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
        "check": {"parseval_rel_err_logN_%d" % logn_chk: parseval}, "ft": ft_info, "also": also,
    }
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()
    return 0


def run_fourstep(a):
    """BASELINE config 5: one long transform over all GPUs of the node (world size >= 1)."""
    import torch

    import turbofft_b200 as tf
    from turbofft_b200 import multi_gpu as mg

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    tdtype = torch.complex64 if a.datatype == 0 else torch.complex128
    rdtype = torch.float32 if a.datatype == 0 else torch.float64
    esize = 8 if a.datatype == 0 else 16
    n_local = (1 << a.logN) // world
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    x = torch.view_as_complex(torch.rand(n_local, 2, generator=g, device=dev, dtype=rdtype) * 2 - 1).to(tdtype)
    if a.fused:
        fs = mg.FusedFourStepFFT(a.logN, world, rank, a.datatype, local, natural_order=bool(a.natural),
                                 if_ft=int(a.ft >= 1), if_err=int(a.ft == 2), thread_bs=a.thread_bs, pipeline=a.pipeline,
                                 exchange=a.exchange)
        be = fs
    else:
        be = mg.DeviceBackend(a.datatype, local, if_ft=int(a.ft >= 1), if_err=int(a.ft == 2), thread_bs=a.thread_bs)
        fs = mg.FourStepFFT(a.logN, world, rank, be, natural_order=bool(a.natural))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(a.warmup, 3)):
        y = fs(x)
    barrier()
    l0 = tf.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        y = fs(x)
    e1.record()
    barrier()
    launches = tf.launch_count() - l0
    ms = e0.elapsed_time(e1) / a.steps
    ex = (x.real.double() ** 2 + x.imag.double() ** 2).sum()
    ey = (y.real.double() ** 2 + y.imag.double() ** 2).sum()
    stats = torch.stack([torch.tensor(ms, device=dev, dtype=torch.float64), ex, ey])
    if dist is not None:
        tmax = stats[:1].clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        sums = stats[1:].clone()
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)
        ms, ex, ey = float(tmax[0]), float(sums[0]), float(sums[1])
    else:
        ms, ex, ey = float(stats[0]), float(stats[1]), float(stats[2])
    nd, nc = be.ft_counts() if a.ft else (0, 0)
    if rank == 0:
        n = 1 << a.logN
        peak, peak_src = peaks()
        passes = 2  # two local FFT passes; each reads and writes the slab once at best
        alg = 2.0 * n * esize / world
        line = {
            "metric": "four_step_c2c_fft_gflops", "value": 5.0 * n * a.logN / (ms * 1e-3) / 1e9, "unit": "GFLOPS",
            "n_gpus": world, "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32" if a.datatype == 0 else "f64", "data": "synthetic",
            "config": {"workload": f"cfg5: one 2^{a.logN}-point C2C transform as 2^{fs.l1} x 2^{fs.l2}, four-step over "
                                   f"{world} GPU(s), {'natural' if a.natural else 'transposed'} output, FT {'on' if a.ft else 'off'}, "
                                   f"{('exchange fused into peer-storing transpose kernels' if a.exchange == 'stores' else 'pack kernel + copy-engine peer copies') + ', %d pieces pipelined' % a.pipeline if a.fused else 'NCCL all_to_all_single'}",
                       "exchanges": (3 if a.natural else 2) if world > 1 else 0,
                       "nvlink_bytes_per_exchange_per_gpu": int((world - 1) / world * n * esize / world)},
            "roofline": {"bound": "hbm", "achieved": alg / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": alg / (ms * 1e-3) / 1e9 / peak, "traffic": None, "peak_source": peak_src,
                         "note": "algorithmic bytes = 2*N*sizeof/world per GPU; the local path makes %d FFT passes plus "
                                 "pack/transpose passes" % passes},
            "gpu_launches": int(launches), "check": {"parseval_rel_err": abs(ey / (n * ex) - 1.0)},
            "ft": {"detected": nd, "corrected": nc} if a.ft else None,
        }
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()
    return 0


def _time_us(torch, fn, reps):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps


def run_cfg1(a):
    """BASELINE config 1: N = 2^10, batch 16, complex64, seed 0 -- a latency case (262 144
    algorithmic bytes), reported in microseconds, not as a roofline fraction."""
    import numpy as np
    import torch

    import turbofft_b200 as tf

    torch.cuda.set_device(0)
    rng = np.random.default_rng(0)
    xn = rng.uniform(-1, 1, (16, 1024, 2)).astype(np.float32).view(np.complex64).reshape(16, 1024)
    x = torch.from_numpy(xn).cuda()
    y = torch.empty_like(x)
    plan = tf.Plan(10, 16, 0)
    stream = torch.cuda.current_stream().cuda_stream
    run = lambda: plan.exec_ptr(x.data_ptr(), y.data_ptr(), stream)
    for _ in range(20):
        run()
    back_to_back = _time_us(torch, run, 2000)
    t0 = time.perf_counter()
    for _ in range(500):
        run()
        torch.cuda.synchronize()
    with_sync = (time.perf_counter() - t0) * 1e6 / 500
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        gs = torch.cuda.current_stream().cuda_stream
        plan.exec_ptr(x.data_ptr(), y.data_ptr(), gs)
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=s):
            for _ in range(10):
                plan.exec_ptr(x.data_ptr(), y.data_ptr(), torch.cuda.current_stream().cuda_stream)
    graph_us = _time_us(torch, g.replay, 200) / 10
    ref = np.fft.fft(xn.astype(np.complex128), axis=-1)
    err = float(np.linalg.norm(y.cpu().numpy() - ref) / np.linalg.norm(ref))
    print(json.dumps({
        "metric": "c2c_fft_latency_us_N1024_batch16", "value": back_to_back, "unit": "us", "n_gpus": 1, "higher_is_better": False,
        "dtype": "f32", "data": "synthetic", "config": {"workload": "cfg1: N=2^10, batch 16, complex64 uniform[-1,1) seed 0, FT off"},
        "us_per_transform_back_to_back": back_to_back, "us_per_transform_with_host_sync": with_sync,
        "us_per_transform_cuda_graph_of_10": graph_us, "rel_l2_vs_float64_fft": err,
        "gflops": 5 * 1024 * 10 * 16 / back_to_back / 1e3}))
    return 0


def run_cfg4(a):
    """BASELINE config 4: logN = 20, batch 256, complex64 uniform[-1,1), err_threshold 1e-3,
    +100 injected: (i) the reference's fault pattern (every block of the last launch) for
    thread_bs 1..32, (ii) one faulty block per 1000.  Reports detection rate, exactness of
    the located index, bit-equality of the corrected output with the fault-free run, overhead."""
    import torch

    import turbofft_b200 as tf

    torch.cuda.set_device(0)
    logn, batch = 20, 256
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.view_as_complex(torch.rand(batch << logn, 2, generator=g, device="cuda") * 2 - 1).view(batch, 1 << logn)
    y = torch.empty_like(x)
    stream = torch.cuda.current_stream().cuda_stream
    base_plan = tf.Plan(logn, batch, 0)
    clean = base_plan(x)
    run = lambda p: (lambda: p.exec_ptr(x.data_ptr(), y.data_ptr(), stream))
    for _ in range(3):
        run(base_plan)()
    t0 = _time_us(torch, run(base_plan), 20)
    rows = []
    for tbs in (1, 2, 4, 8, 16, 32):
        det = tf.Plan(logn, batch, 0, if_ft=1, thread_bs=tbs)
        t_det = _time_us(torch, run(det), 10)
        err = tf.Plan(logn, batch, 0, if_ft=1, if_err=1, thread_bs=tbs)
        t_err = _time_us(torch, run(err), 10)
        nd, nc, loc = err.ft_status()
        exact = sum(1 for b, k in enumerate(loc) if k != -1 and k == b % tbs + 1)
        sparse = tf.Plan(logn, batch, 0, if_ft=1, if_err=1, thread_bs=tbs)
        sparse.set_injection(True, launch=-1, period=1000, phase=7)
        t_sp = _time_us(torch, run(sparse), 10)
        nds, ncs, locs = sparse.ft_status()
        n_faulty = sum(1 for b in range(len(locs)) if b % 1000 == 7)
        rows.append({"thread_bs": tbs, "blocks": len(loc), "detected": nd, "located_exactly": exact, "corrected": nc,
                     "output_equals_fault_free": bool(torch.equal(y, clean)) if False else None,
                     "ft_detect_overhead_pct": 100 * (t_det / t0 - 1), "ft_inject_correct_overhead_pct": 100 * (t_err / t0 - 1),
                     "sparse": {"faulty_blocks": n_faulty, "detected": nds, "corrected": ncs,
                                "false_positives": sum(1 for b, k in enumerate(locs) if k != -1 and b % 1000 != 7),
                                "overhead_pct": 100 * (t_sp / t0 - 1)}})
        # bit-equality of the repaired output where every fault was seen
        yy = err(x)
        rows[-1]["output_equals_fault_free"] = bool(torch.equal(yy, clean))
    # how the outcome moves with err_threshold (thread_bs 8): detection rate on the reference's fault
    # pattern and false alarms on clean data
    sweep = []
    for thr in (1e-3, 3e-4, 1e-4, 3e-5, 1e-5, 3e-6):
        p = tf.Plan(logn, batch, 0, if_ft=1, if_err=1, thread_bs=8)
        p.set_ft_params(100.0, 1000.0, thr)
        yy = p(x)
        nd, nc, loc = p.ft_status()
        exact = sum(1 for b, k in enumerate(loc) if k != -1 and k == b % 8 + 1)
        ok = bool(torch.equal(yy, clean))
        p.set_injection(False)
        p(x)
        fa = p.ft_status()[0]
        sweep.append({"err_threshold": thr, "blocks": len(loc), "detected": nd, "located_exactly": exact,
                      "output_equals_fault_free": ok, "false_alarms_on_clean_input": fa})
    print(json.dumps({
        "metric": "ft_overhead_pct_logN20_batch256", "value": min(r["ft_detect_overhead_pct"] for r in rows), "unit": "%",
        "n_gpus": 1, "higher_is_better": False, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "cfg4: logN=20, batch 256, complex64 uniform[-1,1), err_inj 100, err_smoothing 1000, err_threshold 1e-3"},
        "no_ft_us": t0, "rows": rows, "threshold_sweep_thread_bs8": sweep,
        "note": "detected < blocks means the reference's own test |delta|/(1000+S) > 1e-3 stays below threshold for those blocks "
                "(S grows with the signal energy of thread_bs tiles); the CPU model of the decision predicts the same"}))
    return 0


def main():
    a = parse_args()
    if a.impl == "reference":
        return run_reference(a)
    if a.workload == "fourstep":
        return run_fourstep(a)
    if a.workload == "cfg1":
        return run_cfg1(a)
    if a.workload == "cfg4":
        return run_cfg4(a)
    return run_ours(a)


if __name__ == "__main__":
    sys.exit(main())
