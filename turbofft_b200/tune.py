"""Tuner for param/<gpu>/param_<datatype>.csv (the reference's 11-column format, readme.md:46-67).

The reference ships hand-tuned A100/T4 tables; this searches the same space on the machine
it runs on: launch split (logN1..3), lines per block (BSi), points per thread (ni) and -- per
size, for the chosen row -- thread_bs, the tiles one block loops over (the reference leaves it to
the command line, compile.sh:13-19, and records one table per value in data_ft/*.csv).  The
thread_bs choices go to param/<gpu>/thread_bs_<datatype>.csv ("logN, FT off, FT on"), which a plan
created with thread_bs = 0 follows.

  1. python -m turbofft_b200.tune emit --datatype float2          # CPU: candidate rows ->
        param/B200/extra_float2.csv, then `python -m turbofft_b200.build` compiles them
  2. python -m turbofft_b200.tune run --datatype float2 --out r.json   # GPU: times every candidate
        at logN + logBS = --log-total (default 28), FT off
  3. python -m turbofft_b200.tune apply --datatype float2 --results r.json   # CPU: best rows -> CSV
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time

from . import planner

MAX_SMEM = 200 * 1024


def _row(logn, parts):
    """parts: list of (logm, bs, n) per launch."""
    l = len(parts)
    logs = [p[0] for p in parts] + [0] * (3 - l)
    bs = [p[1] for p in parts] + [0] * (3 - l)
    n = [p[2] for p in parts] + [0] * (3 - l)
    return planner.ParamRow(logn, l, tuple(logs), tuple(bs), tuple(n))


def _launch_ok(logm, c, e, role, esize, n_first=None):
    if e > (1 << logm):
        return False
    threads = ((1 << logm) // e) * c
    if not 32 <= threads <= 1024:
        return False
    stages = (logm + (e.bit_length() - 1) - 1) // (e.bit_length() - 1)
    if role == planner.ROLE_LAST and stages < 2:
        return False
    smem = (1 << logm) * c * esize * 1.3 if stages > 1 else 0
    return smem <= MAX_SMEM


def candidates(logn: int, datatype: str):
    esize = 8 if datatype == "float2" else 16
    es = (8, 16) if datatype == "double2" else (8, 16, 32)
    out = []
    if logn <= 14:
        for e in es:
            for c in (1, 2, 4, 8, 16, 32, 64, 128):
                if _launch_ok(logn, c, min(e, 1 << logn), planner.ROLE_SINGLE, esize):
                    out.append(_row(logn, [(logn, c, min(e, 1 << logn))]))
    if logn >= 12:
        for a in range(6, 13):
            b = logn - a
            if not 6 <= b <= 12 or abs(a - b) > 3:
                continue
            # 32 points per thread only where it saves an exchange (lines of 512 and 1024)
            for e1 in es if a in (9, 10) else (8, 16):
                for e2 in es if b in (9, 10) else (8, 16):
                    for c1 in (4, 8, 16, 32):
                        for c2 in (4, 8, 16, 32):
                            if c2 > (1 << a):
                                continue
                            if _launch_ok(a, c1, e1, planner.ROLE_FIRST, esize) and _launch_ok(b, c2, e2, planner.ROLE_LAST, esize):
                                out.append(_row(logn, [(a, c1, e1), (b, c2, e2)]))
    if logn >= 20:
        base = logn // 3
        for a in range(base - 1, base + 3):
            for b in range(base - 1, base + 3):
                c = logn - a - b
                if not 6 <= c <= 10 or not 6 <= a <= 10 or not 6 <= b <= 10:
                    continue
                for e in (8, 16):
                    for cc in (8, 16, 32):
                        if all(_launch_ok(m, cc, e, r, esize) for m, r in
                               ((a, planner.ROLE_FIRST), (b, planner.ROLE_FIRST), (c, planner.ROLE_LAST))):
                            out.append(_row(logn, [(a, cc, e), (b, cc, e), (c, cc, e)]))
    # de-duplicate
    seen, uniq = set(), []
    for r in out:
        key = (r.launches, r.logni, r.bs, r.n)
        if key not in seen:
            seen.add(key)
            uniq.append(r)
    return uniq


def row_text(r: planner.ParamRow) -> str:
    return ", ".join(str(v) for v in (r.logn, r.launches) + tuple(r.logni) + tuple(r.bs) + tuple(r.n))


def cmd_emit(a):
    path = os.path.join(planner.PARAM_DIR, a.gpu, f"extra_{a.datatype}.csv")
    lines = ["# candidate rows for the tuner (python -m turbofft_b200.tune); compiled for FT off only"]
    n = 0
    for logn in range(a.lo, a.hi + 1):
        for r in candidates(logn, a.datatype):
            lines.append(row_text(r))
            n += 1
    with open(path, "w") as f:
        f.write("\n".join(lines) + "\n")
    print(f"wrote {n} candidate rows to {path}")


class _Sweep:
    """The built-in plans of the sizes lo..hi over the same buffers: run for a while before a candidate is
    timed, they put the GPU into the state the sweep benchmark sees it in (sustained load, power-capped
    clocks).  Rankings taken in short bursts on a cool GPU have turned over there more than once."""

    def __init__(self, tf, lo, hi, log_total, dt):
        self.plans = []
        for logn in range(lo, hi + 1):
            try:
                self.plans.append(tf.Plan(logn, 1 << (log_total - logn), dt, thread_bs=0))
            except tf.TurboFFTError:
                pass

    def heat(self, torch, x, y, stream, ms):
        if ms <= 0 or not self.plans:
            return
        t0 = time.perf_counter()
        while (time.perf_counter() - t0) * 1e3 < ms:
            for p in self.plans:
                p.exec_ptr(x.data_ptr(), y.data_ptr(), stream)
            torch.cuda.synchronize()

    def destroy(self):
        for p in self.plans:
            p.destroy()


def _time_plan(torch, plan, x, y, stream, burn, reps, sweep=None, sustain_ms=0):
    if sweep is not None:
        sweep.heat(torch, x, y, stream, sustain_ms)
    for _ in range(burn):
        plan.exec_ptr(x.data_ptr(), y.data_ptr(), stream)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        plan.exec_ptr(x.data_ptr(), y.data_ptr(), stream)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def cmd_run(a):
    import torch

    import turbofft_b200 as tf

    dt = 0 if a.datatype == "float2" else 1
    td = torch.complex64 if dt == 0 else torch.complex128
    n = 1 << a.log_total
    x = torch.randn(n, dtype=td, device="cuda")
    y = torch.empty_like(x)
    stream = torch.cuda.current_stream().cuda_stream
    current = planner.load_params(a.datatype, a.gpu)
    results = {}
    sweep = _Sweep(tf, a.sweep_lo, a.sweep_hi, a.log_total, dt) if a.sustain_ms > 0 else None
    for logn in range(a.lo, a.hi + 1):
        cands = [current[logn]] + candidates(logn, a.datatype)
        best = None
        rows = []
        for r in cands:
            with tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False) as f:
                f.write(row_text(r) + "\n")
                path = f.name
            try:
                plan = tf.Plan(logn, 1 << (a.log_total - logn), dt, param_csv=path)
            except tf.TurboFFTError:
                os.unlink(path)
                continue
            os.unlink(path)
            ms = _time_plan(torch, plan, x, y, stream, a.burn, a.reps, sweep, a.sustain_ms)
            plan.destroy()
            rows.append((ms, row_text(r)))
            if best is None or ms < best[0]:
                best = (ms, row_text(r))
        rows.sort()
        # thread_bs for the winning row, FT off and FT on (detect)
        tbs_ms = {}
        with tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False) as f:
            f.write(best[1] + "\n")
            path = f.name
        for ft in (0, 1):
            for tbs in a.thread_bs:
                try:
                    plan = tf.Plan(logn, 1 << (a.log_total - logn), dt, if_ft=ft, thread_bs=tbs, param_csv=path)
                except tf.TurboFFTError:
                    continue
                tbs_ms[f"{ft}:{tbs}"] = _time_plan(torch, plan, x, y, stream, a.burn, a.reps, sweep, a.sustain_ms)
                plan.destroy()
        os.unlink(path)
        pick = {ft: min((v, int(k.split(":")[1])) for k, v in tbs_ms.items() if k.startswith(f"{ft}:"))[1]
                for ft in (0, 1) if any(k.startswith(f"{ft}:") for k in tbs_ms)}
        results[str(logn)] = {"best": best, "current_ms": rows and next((m for m, t in rows if t == row_text(current[logn])), None),
                              "top": rows[:5], "tried": len(rows), "thread_bs_ms": tbs_ms,
                              "thread_bs": [pick.get(0, 1), pick.get(1, 1)]}
        print(f"logN {logn}: best {best[0]:.3f} ms [{best[1]}] current {results[str(logn)]['current_ms']} ({len(rows)} tried) "
              f"thread_bs FT off/on {results[str(logn)]['thread_bs']}", flush=True)
    if sweep is not None:
        sweep.destroy()
    with open(a.out, "w") as f:
        json.dump(results, f, indent=1)


def cmd_apply(a):
    res = json.load(open(a.results))
    path = os.path.join(planner.PARAM_DIR, a.gpu, f"param_{a.datatype}.csv")
    rows = planner.load_params(a.datatype, a.gpu)
    lines = []
    for logn in sorted(rows):
        r = rows[logn]
        key = str(logn)
        if key in res and res[key]["best"] and (res[key]["current_ms"] is None or
                                               res[key]["best"][0] < res[key]["current_ms"] * (1 - a.min_gain)):
            lines.append(res[key]["best"][1])
        else:
            lines.append(row_text(r))
    with open(path, "w") as f:
        f.write("\n".join(lines) + "\n")
    print(f"updated {path}")
    # thread_bs table: keep what is there, replace the sizes that were measured
    tpath = os.path.join(planner.PARAM_DIR, a.gpu, f"thread_bs_{a.datatype}.csv")
    table = planner.load_thread_bs(a.datatype, a.gpu)
    for key, r in res.items():
        if "thread_bs" in r:
            table[int(key)] = tuple(r["thread_bs"])
    with open(tpath, "w") as f:
        f.write("# thread_bs a plan created with thread_bs = 0 uses: logN, FT off, FT on (written by turbofft_b200.tune)\n")
        for logn in sorted(table):
            f.write(f"{logn}, {table[logn][0]}, {table[logn][1]}\n")
    print(f"updated {tpath}")


def main(argv=None):
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("emit", "run", "apply"):
        p = sub.add_parser(name)
        p.add_argument("--datatype", default="float2", choices=["float2", "double2"])
        p.add_argument("--gpu", default="B200")
        p.add_argument("--lo", type=int, default=7)
        p.add_argument("--hi", type=int, default=24)
        if name == "run":
            p.add_argument("--log-total", type=int, default=28)
            p.add_argument("--reps", type=int, default=5)
            p.add_argument("--burn", type=int, default=2, help="untimed runs before the timed ones")
            p.add_argument("--sustain-ms", type=float, default=0.0,
                           help="run the built-in sweep (--sweep-lo..--sweep-hi) this long before every timing, so that "
                                "candidates are ranked at the sustained, power-capped clocks the sweep benchmark runs at")
            p.add_argument("--sweep-lo", type=int, default=7)
            p.add_argument("--sweep-hi", type=int, default=24)
            p.add_argument("--out", default="tune_results.json")
            p.add_argument("--thread-bs", type=lambda t: [int(v) for v in t.split(",")], default=[1, 2, 4, 8],
                           help="thread_bs values tried for the winning row")
        if name == "apply":
            p.add_argument("--results", required=True)
            p.add_argument("--min-gain", type=float, default=0.01)
    a = ap.parse_args(argv)
    {"emit": cmd_emit, "run": cmd_run, "apply": cmd_apply}[a.cmd](a)


if __name__ == "__main__":
    sys.exit(main())
