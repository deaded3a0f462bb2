"""Single-pass plans (one thread-block-cluster kernel, distributed shared memory exchange)
against the CPU oracle, through the C ABI (tfft_plan_create_single_pass).

Same tolerances as the multi-launch plans: relative L2 <= 1e-6 * log2 N (complex64) and
<= 1e-14 * log2 N (complex128) against the float64 oracle.  The reference has no such
kernel: its plans for these sizes are two launches (include/param/A100/param_float2.csv
rows 13-17), so the comparison partner besides the oracle is this library's own
multi-launch plan for the same size.
"""
import os

import numpy as np
import pytest

from oracle import fft_oracle as orc

pytestmark = pytest.mark.gpu
CD = {0: np.complex64, 1: np.complex128}

# (dtype, logN, log2 cluster sizes compiled for it)
SIZES = [(0, 13, (0, 1)), (0, 14, (1, 2, 0)), (0, 15, (3, 2, 1)), (0, 16, (4, 3, 2)), (0, 17, (4, 3)),
         (1, 12, (0,)), (1, 13, (1,)), (1, 14, (2,)), (1, 15, (3,)), (1, 16, (4, 3))]
CASES = [(dt, logn, g) for dt, logn, gs in SIZES for g in gs]


@pytest.mark.parametrize("dtype,logn,log_cluster", CASES)
def test_single_pass_matches_oracle(torch_cuda, dtype, logn, log_cluster):
    import turbofft_b200 as tf

    torch = torch_cuda
    for batch, tbs in ((5, 2), (1, 1), (7, 3)):     # ragged: the last cluster runs out of signals
        x = orc.make_input(batch, 1 << logn, CD[dtype], seed=logn + batch)
        plan = tf.Plan(logn, batch, dtype, single_pass=log_cluster, thread_bs=tbs)
        assert plan.cluster_size == 1 << log_cluster and len(plan.info()) == 1
        xd = torch.from_numpy(x).cuda()
        y = plan(xd)
        torch.cuda.synchronize()
        assert torch.equal(xd.cpu(), torch.from_numpy(x))              # input untouched
        err = orc.rel_l2(y.cpu().numpy(), orc.fft_forward(x))
        assert err <= orc.tolerance(CD[dtype], logn), (logn, log_cluster, batch, err)
        y2 = plan(xd, out=xd)                                          # in place
        torch.cuda.synchronize()
        assert torch.equal(y, y2)
        assert plan.device_status() == 0                               # no bounded wait for the exchange's mbarrier gave up
        plan.destroy()


@pytest.mark.parametrize("dtype,logn", [(0, 15), (1, 14)])
def test_single_pass_agrees_with_the_launches(torch_cuda, dtype, logn):
    """Default cluster size (-1) against the multi-launch plan of the same size, and the
    inverse transform with 1/N scaling brings the signal back."""
    import turbofft_b200 as tf

    torch = torch_cuda
    batch = 6
    x = orc.make_input(batch, 1 << logn, CD[dtype], seed=3)
    xd = torch.from_numpy(x).cuda()
    csv = os.path.join(os.path.dirname(tf.__file__), "param", "B200", "param_float2.csv" if dtype == 0 else "param_double2.csv")
    y_launches = tf.Plan(logn, batch, dtype, param_csv=csv)(xd)
    sp = tf.Plan(logn, batch, dtype, single_pass=-1)
    y = sp(xd)
    scale = float(torch.linalg.vector_norm(y_launches))
    assert float(torch.linalg.vector_norm(y - y_launches)) / scale <= orc.tolerance(CD[dtype], logn)
    lib = tf.lib()
    assert lib.tfft_set_direction(sp._h, 1, 1.0 / (1 << logn)) == 0
    back = sp(y)
    torch.cuda.synchronize()
    assert orc.rel_l2(back.cpu().numpy(), x) <= 2 * orc.tolerance(CD[dtype], logn)


def test_single_pass_refuses_what_it_cannot_do(torch_cuda):
    import ctypes as C

    import turbofft_b200 as tf

    torch = torch_cuda
    lib = tf.lib()
    h = C.c_void_p()
    assert lib.tfft_plan_create_single_pass(C.byref(h), 10, 4, 0, -1, 1, 0) == -2     # no such kernel
    assert lib.tfft_plan_create_single_pass(C.byref(h), 15, 4, 0, 7, 1, 0) == -2      # no such cluster size
    assert lib.tfft_plan_create_single_pass(C.byref(h), 15, 0, 0, -1, 1, 0) == -1     # bad batch
    plan = tf.Plan(15, 2, 0, single_pass=-1)
    buf = torch.zeros((2 << 15) + 1, dtype=torch.complex64, device="cuda")
    x = torch.zeros(2 << 15, dtype=torch.complex64, device="cuda")
    # an output that is only 8-byte aligned is refused, not silently mis-stored
    rc = lib.tfft_exec(plan._h, x.data_ptr(), buf.data_ptr() + 8, torch.cuda.current_stream().cuda_stream)
    assert rc == -1


@pytest.mark.parametrize("logn,log_cluster", [(13, 1), (14, 2), (15, 3), (16, 4)])
def test_prefetching_variant_matches_oracle(torch_cuda, logn, log_cluster):
    """TFFT_SINGLE_PASS_PREFETCH: the CTAs fetch their share of the next signal with bulk
    asynchronous copies completing on an mbarrier while the current one is transformed.  Same
    results as the plain variant bit for bit (the arithmetic is the same), for one signal, for
    several per cluster and for a ragged count, and no bounded wait ever gave up."""
    import ctypes as C

    import turbofft_b200 as tf

    torch = torch_cuda
    lib = tf.lib()
    for batch, tbs in ((1, 1), (9, 4), (23, 3), (64, 8)):
        x = orc.make_input(batch, 1 << logn, np.complex64, seed=batch)
        xd = torch.from_numpy(x).cuda()
        plain = tf.Plan(logn, batch, 0, single_pass=log_cluster, thread_bs=tbs)(xd)
        plan = tf.Plan(logn, batch, 0, single_pass=log_cluster | 16, thread_bs=tbs)
        y = plan(xd)
        torch.cuda.synchronize()
        st = C.c_int(-1)
        assert lib.tfft_plan_device_status(plan._h, C.byref(st)) == 0 and st.value == 0
        assert torch.equal(y, plain)
        assert orc.rel_l2(y.cpu().numpy(), orc.fft_forward(x)) <= orc.tolerance(np.complex64, logn)


@pytest.mark.parametrize("logn,log_cluster", [(13, 1), (14, 2), (15, 3), (15, 4), (16, 4)])
def test_radix8_variant_matches_oracle(torch_cuda, logn, log_cluster):
    """TFFT_SINGLE_PASS_RADIX8: complex64 with 16 points per thread (radix-8 unit stages, one more
    stage), half the registers and twice the resident warps."""
    import turbofft_b200 as tf

    torch = torch_cuda
    for batch, tbs in ((1, 1), (11, 3)):
        x = orc.make_input(batch, 1 << logn, np.complex64, seed=batch + logn)
        plan = tf.Plan(logn, batch, 0, single_pass=log_cluster | 32, thread_bs=tbs)
        assert plan.cluster_size == 1 << log_cluster and plan.info()[0]["points_per_thread"] == 16
        y = plan(torch.from_numpy(x).cuda())
        torch.cuda.synchronize()
        assert orc.rel_l2(y.cpu().numpy(), orc.fft_forward(x)) <= orc.tolerance(np.complex64, logn)
