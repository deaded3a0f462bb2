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


def _chunked_energy(torch, t, chunk=1 << 26):
    flat = t.view(-1)
    tot = 0.0
    for i in range(0, flat.numel(), chunk):
        c = flat[i:i + chunk]
        tot += float((c.real.double() ** 2 + c.imag.double() ** 2).sum())
    return tot


@pytest.mark.parametrize("dtype,logn", [(0, 26), (0, 28), (0, 30), (1, 27)])
def test_single_long_transform_on_one_gpu(torch_cuda, dtype, logn):
    """Three-launch plans far beyond the reference's table (which stops at 2^25 and overflows
    32-bit indices at 2^31 elements): 64-bit indexing, checked by Parseval, by the analytic
    transform of impulse + tone, and for 2^26 against the float64 oracle."""
    import turbofft_b200 as tf

    torch = torch_cuda
    n = 1 << logn
    cd = np.complex64 if dtype == 0 else np.complex128
    tol = orc.tolerance(cd, logn)
    x = _make(torch, dtype, n, seed=logn)
    plan = tf.Plan(logn, 1, dtype)
    y = plan(x)
    torch.cuda.synchronize()
    assert abs(_chunked_energy(torch, y) / (n * _chunked_energy(torch, x)) - 1.0) <= 10 * tol
    if logn <= 26:
        ref = orc.fft_forward(x.cpu().numpy())
        assert orc.rel_l2(y.cpu().numpy(), ref) <= tol
        del ref
    del y
    # impulse at n0 plus a pure tone at k0: X[k] = exp(-2 pi i n0 k / N) + N [k == k0]
    n0, k0 = 12345, 54321
    x.zero_()
    step = 1 << 24
    for i in range(0, n, step):
        j = torch.arange(i, i + step, device="cuda", dtype=torch.int64)
        ph = ((j * k0) % n).double() * (2 * np.pi / n)
        x[i:i + step] = torch.polar(torch.full_like(ph, 1.0 / n), ph).to(x.dtype)
    x[n0] += 1.0
    y = plan(x)
    worst = 0.0
    for i in range(0, n, step):
        k = torch.arange(i, i + step, device="cuda", dtype=torch.int64)
        ph = ((k * n0) % n).double() * (-2 * np.pi / n)
        want = torch.polar(torch.ones_like(ph), ph)
        if i <= k0 < i + step:
            want[k0 - i] += 1.0
        worst = max(worst, float((y[i:i + step].to(torch.complex128) - want).abs().max()))
    assert worst <= 50 * tol, worst
