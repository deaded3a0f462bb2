"""The allocation-free entry point tfft_exec_static, called through the C ABI.

It exists for callers that may not allocate device memory at call time (its scratch and
tables are static device arrays of the library).  Its output must equal the ordinary
plan's, bit for bit (same kernels, same tables), on calls made back to back -- the second
call reuses the arrays the first one left dirty, and a change of size rewrites the tables.
Collected last on purpose: a failure here cannot hide any other test's result.
"""
import numpy as np
import pytest

from oracle import fft_oracle as orc

pytestmark = pytest.mark.gpu
CD = {0: np.complex64, 1: np.complex128}


def _static_fft(torch, logn, batch, dtype, x):
    from turbofft_b200 import _lib

    y = torch.empty_like(x)
    rc = _lib.lib().tfft_exec_static(logn, batch, dtype, x.data_ptr(), y.data_ptr(), x.device.index,
                                     torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return rc, y


def test_static_entry_matches_plan_on_consecutive_calls(torch_cuda):
    import turbofft_b200 as tf

    torch = torch_cuda
    # two calls in a row per size, different data each time; sizes change in between
    for dtype, logn, batch in [(0, 16, 8), (0, 16, 8), (1, 14, 16), (1, 14, 16), (0, 20, 2), (0, 15, 3), (1, 17, 4)]:
        for rep in range(2):
            xn = orc.make_input(batch, 1 << logn, CD[dtype], seed=100 * logn + rep)
            x = torch.from_numpy(xn).cuda()
            rc, y_static = _static_fft(torch, logn, batch, dtype, x)
            assert rc == 0, rc
            y_plan = tf.Plan(logn, batch, dtype)(x)
            torch.cuda.synchronize()
            assert torch.equal(y_static, y_plan)
            assert orc.rel_l2(y_static.cpu().numpy(), orc.fft_forward(xn)) <= orc.tolerance(CD[dtype], logn)


def test_static_entry_rejects_what_it_cannot_hold(torch_cuda):
    from turbofft_b200 import _lib

    torch = torch_cuda
    x = torch.zeros(1 << 22, dtype=torch.complex64, device="cuda")
    # 2^22 complex64 = 32 MiB > the 16 MiB static scratch
    rc, _ = _static_fft(torch, 16, 64, 0, x)
    assert rc == -6                                  # TFFT_ERR_TOO_LARGE
    # one-launch sizes use no scratch and are not served by this entry point
    rc, _ = _static_fft(torch, 10, 16, 0, x[: 16 << 10])
    assert rc == -2                                  # TFFT_ERR_UNSUPPORTED
    assert _lib.lib().tfft_exec_static(16, 8, 0, None, None, 0, None) == -1
