"""The bounds-checked build of the library (libturbofft_b200_check.so, -DTFFT_BOUNDS_CHECK=1):
every global load and store of the data buffers compares its index with batch * N and records
the first access outside.  The small-case suite below runs under it in a child process (the
library is chosen when the package is first imported) and must leave the record empty for
every role, FT mode and ragged batch; the outputs must still match the oracle.
"""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHECK_LIB = os.path.join(ROOT, "turbofft_b200", "libturbofft_b200_check.so")

CHILD = textwrap.dedent("""
    import ctypes as C, sys
    import numpy as np, torch
    import turbofft_b200 as tf
    from oracle import fft_oracle as orc
    lib = tf.lib()
    CD = {0: np.complex64, 1: np.complex128}
    cases = [(logn, batch, ft, err, tbs) for logn, batch in [(1, 3), (3, 129), (4, 4097), (6, 17), (8, 33), (10, 5), (12, 3),
                                                              (13, 2), (14, 3), (16, 5), (18, 2), (20, 1), (22, 1), (23, 1)]
             for ft, err, tbs in [(0, 0, 1), (1, 0, 2), (1, 1, 3)]]
    n = 0
    for dtype in (0, 1):
        for logn, batch, ft, err, tbs in cases:
            x = orc.make_input(batch, 1 << logn, CD[dtype], seed=logn)
            plan = tf.Plan(logn, batch, dtype, if_ft=ft, if_err=err, thread_bs=tbs)
            if err:
                plan.set_injection(False)
            y = plan(torch.from_numpy(x).cuda())
            idx, site = C.c_longlong(0), C.c_int(0)
            rc = lib.tfft_bounds_status(plan._h, C.byref(idx), C.byref(site))
            assert rc == 0, (dtype, logn, batch, ft, err, tbs, rc, idx.value, site.value)
            assert orc.rel_l2(y.cpu().numpy(), orc.fft_forward(x)) <= orc.tolerance(CD[dtype], logn)
            plan.destroy()
            n += 1
    print("checked", n)
""")


def test_small_case_suite_stays_in_bounds(torch_cuda):
    if not os.path.exists(CHECK_LIB):
        pytest.fail(f"{CHECK_LIB} was not built")
    env = dict(os.environ, TURBOFFT_B200_LIB=CHECK_LIB, PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-c", CHILD], capture_output=True, text=True, env=env, cwd=ROOT, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "checked 84" in r.stdout


def test_normal_build_has_no_checks(torch_cuda):
    import ctypes as C

    import turbofft_b200 as tf

    plan = tf.Plan(10, 4, 0)
    assert tf.lib().tfft_bounds_status(plan._h, C.byref(C.c_longlong()), C.byref(C.c_int())) == -2
