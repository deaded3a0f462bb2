"""TEST INFRASTRUCTURE.  Times the reference's own kernels (recompiled for sm_100a,
oracle/_ref/libturbofft_ref.so) next to this library on the same GPU and inputs.

    python oracle/time_reference_kernels.py [log_total=26]

The reference's launcher prints its own line per run ("turboFFT, logN, logBS, ms, GFLOPS,
GB/s", main.cu:70, timed WITH its per-launch cudaDeviceSynchronize, main.cu:58); ours is timed
with CUDA events without host synchronisation.  Only sizes whose reference kernels have been
run by the parity tests are timed; float2 logN 2..4 are never run (stale kernels, see
oracle/ref_harness.cu).
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))

CASES = {0: [5, 7, 10, 12, 13, 14, 16, 17, 20, 23], 1: [10, 13, 15, 16, 20]}


def main():
    import torch

    import make_golden
    import turbofft_b200 as tf

    log_total = int(sys.argv[1]) if len(sys.argv) > 1 else 26
    lib = make_golden.load_ref()
    for dtype, logns in CASES.items():
        npdt = np.complex64 if dtype == 0 else np.complex128
        es = 8 if dtype == 0 else 16
        x = np.ascontiguousarray((np.random.default_rng(0).uniform(-1, 1, 2 << log_total)).astype(
            np.float32 if dtype == 0 else np.float64).view(npdt))
        xd = torch.from_numpy(x).cuda()
        yd = torch.empty_like(xd)
        for logn in logns:
            bs = 1 << (log_total - logn)
            sys.stdout.flush()
            out = np.empty_like(x)
            csv = os.path.join(ROOT, "oracle", "_ref", "param", "A100", "param_%s.csv" % ("float2" if dtype == 0 else "double2"))
            rc = lib.ref_run(dtype, 0, 0, logn, bs, 1, x.ctypes.data, out.ctypes.data, 10, csv.encode())  # prints its line
            plan = tf.Plan(logn, bs, dtype)
            s = torch.cuda.current_stream().cuda_stream
            for _ in range(3):
                plan.exec_ptr(xd.data_ptr(), yd.data_ptr(), s)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(10):
                plan.exec_ptr(xd.data_ptr(), yd.data_ptr(), s)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / 10
            n = 1 << log_total
            print(f"b200,     {logn}, {log_total - logn}, {ms:8.3f}, {5 * n * logn / ms / 1e6:8.3f}, {2 * n * es / ms / 1e6:8.3f}   "
                  f"(dtype {dtype}, ref rc {rc}, max |ours - ref| / max |ref| = "
                  f"{float(np.abs(yd.cpu().numpy() - out).max() / np.abs(out).max()):.2e})", flush=True)
            plan.destroy()


if __name__ == "__main__":
    main()
