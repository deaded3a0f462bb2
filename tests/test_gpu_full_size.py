"""BASELINE-size runs checked through size-independent properties.

The oracle cannot transform 2^28 elements in test time, so the full-size configurations are
checked by Parseval, linearity, shift/impulse identities and by comparing a few sampled
signals of the batch with the float64 oracle.
"""
import numpy as np
import pytest

from oracle import fft_oracle as orc

pytestmark = pytest.mark.gpu
LOG_TOTAL = 28


def _make(torch, dtype, n, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if dtype == 0:
        return torch.view_as_complex(torch.rand(n, 2, generator=g, device="cuda") * 2 - 1)
    return torch.view_as_complex(torch.randn(n, 2, generator=g, device="cuda", dtype=torch.float64))


def _energy(torch, t):
    return float((t.real.double() ** 2 + t.imag.double() ** 2).sum())


@pytest.mark.parametrize("dtype,logn", [(0, 7), (0, 10), (0, 13), (0, 16), (0, 20), (0, 24), (1, 8), (1, 14), (1, 22)])
def test_sweep_point_full_size(torch_cuda, dtype, logn):
    """Config 2 / 3: batch 2^(28 - logN) signals of 2^logN points."""
    import turbofft_b200 as tf

    torch = torch_cuda
    log_total = LOG_TOTAL if dtype == 0 else LOG_TOTAL - 1     # keeps the fp64 case at 2 GiB per buffer
    batch, n = 1 << (log_total - logn), 1 << logn
    cd = np.complex64 if dtype == 0 else np.complex128
    tol = orc.tolerance(cd, logn)
    x = _make(torch, dtype, batch * n, seed=logn).view(batch, n)
    plan = tf.Plan(logn, batch, dtype)
    y = plan(x)
    torch.cuda.synchronize()
    # Parseval: sum |X|^2 = N sum |x|^2
    assert abs(_energy(torch, y) / (n * _energy(torch, x)) - 1.0) <= 10 * tol
    # sampled signals against the float64 oracle (first, last, a few in between)
    idx = sorted({0, batch - 1, batch // 3, (2 * batch) // 3})
    ref = orc.fft_forward(x[idx].cpu().numpy())
    assert orc.rel_l2(y[idx].cpu().numpy(), ref) <= tol
    # linearity on the full batch: F(a x + z) = a F(x) + F(z), with z a delayed impulse per signal
    z = torch.zeros_like(x)
    z[:, 3] = 1.0
    a = 0.5 - 0.25j
    w = plan(a * x + z)
    k = torch.arange(n, device="cuda", dtype=torch.float64)
    fz = torch.polar(torch.ones_like(k), -2 * np.pi * 3 * k / n).to(x.dtype)   # F(delta_3)
    lin = (w - (a * y + fz)).abs().max().item() / y.abs().max().item()
    assert lin <= 20 * tol, lin
    del w, z


def test_config4_ft_full_size(torch_cuda):
    """Config 4: logN = 20, batch 256, complex64 uniform[-1,1), FT on, +100 injected per block
    of the last launch, err_threshold 1e-3.  Whatever is detected must be located where it was
    injected and repaired exactly; blocks that stay below the threshold keep their fault."""
    import turbofft_b200 as tf

    torch = torch_cuda
    logn, batch = 20, 256
    x = _make(torch, 0, batch << logn, seed=4).view(batch, 1 << logn)
    clean = tf.Plan(logn, batch, 0)(x)
    for tbs in (1, 8, 32):
        plan = tf.Plan(logn, batch, 0, if_ft=1, if_err=1, thread_bs=tbs)
        y = plan(x)
        nd, nc, loc = plan.ft_status()
        assert nd == nc
        hit = [k for k in loc if k != -1]
        assert all(k == orc.injected_tile_iteration(b, tbs) for b, k in enumerate(loc) if k != -1)
        bad = int((y != clean).sum().item())
        # every undetected block leaves exactly one corrupted line of 2^11 outputs (the +100 spreads over it)
        assert bad <= (len(loc) - len(hit)) * (1 << 11)
        if len(hit) == len(loc):
            assert torch.equal(y, clean)
        # detect-only run on clean data: silent
        p1 = tf.Plan(logn, batch, 0, if_ft=1, thread_bs=tbs)
        assert torch.equal(p1(x), clean) and p1.ft_status()[0] == 0
