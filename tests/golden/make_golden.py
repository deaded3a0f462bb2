"""Generates tests/golden/ref_outputs_*.npz on a machine with a B200.

Feeds the reference's own seeded inputs (srandom(10), include/utils/initializeData.h:6-7,
25-26,65-66 -- restated in oracle/fft_oracle.py::reference_input) through the UNMODIFIED
reference kernels (oracle/_ref/libturbofft_ref.so, built by oracle/build_ref.sh) and
stores the outputs.  Run from the repository root:
    python tests/golden/make_golden.py [outdir]
The fixtures pin the CPU oracle to what the reference actually computes.
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import fft_oracle as orc  # noqa: E402

# float2 logN 2..4 are refused by the harness (stale reference kernels, see oracle/ref_harness.cu)
CASES = [(0, 1, 64), (0, 5, 32), (0, 7, 16), (0, 10, 16), (0, 12, 4), (0, 14, 2), (0, 16, 1),
         (1, 3, 32), (1, 10, 8), (1, 13, 2), (1, 15, 1)]


def load_ref():
    lib = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libturbofft_ref.so"))
    lib.ref_run.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_longlong, C.c_int, C.c_void_p, C.c_void_p, C.c_int,
                            C.c_char_p]
    lib.ref_run.restype = C.c_int
    return lib


def ref_fft(lib, dtype, logn, bs, x, ft=0, err=0, thread_bs=1):
    out = np.empty_like(x)
    csv = os.path.join(ROOT, "oracle", "_ref", "param", "A100", "param_%s.csv" % ("float2" if dtype == 0 else "double2"))
    rc = lib.ref_run(dtype, ft, err, logn, bs, thread_bs, x.ctypes.data, out.ctypes.data, 1, csv.encode())
    if rc != 0:
        raise RuntimeError(f"ref_run failed rc={rc} (dtype {dtype}, logN {logn}, bs {bs})")
    return out


def main():
    outdir = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden")
    os.makedirs(outdir, exist_ok=True)
    lib = load_ref()
    data = {}
    for dtype, logn, bs in CASES:
        npdt = np.complex64 if dtype == 0 else np.complex128
        x = np.ascontiguousarray(orc.reference_input(bs, 1 << logn, npdt))
        y = ref_fft(lib, dtype, logn, bs, x)
        err = orc.rel_l2(y, orc.fft_forward(x))
        print(f"dtype {dtype} logN {logn} bs {bs}: reference vs oracle rel_l2 {err:.3e}")
        data[f"out_{dtype}_{logn}_{bs}"] = y
    np.savez_compressed(os.path.join(outdir, "ref_outputs_b200.npz"), **data)
    print("wrote", os.path.join(outdir, "ref_outputs_b200.npz"))


if __name__ == "__main__":
    main()
