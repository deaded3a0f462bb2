"""Fault-tolerance mode on the GPU: decisions bit-exact against the CPU model.

What is compared exactly: per block, (detected?, located tile iteration).  The checksum
values themselves differ in rounding (summation order), so faults are chosen with wide
margins, as the reference's own defaults do (err_inj 100, err_smoothing 1000, err_threshold 1e-3).
"""
import numpy as np
import pytest

from oracle import fft_oracle as orc
from turbofft_b200 import planner

pytestmark = pytest.mark.gpu
CD = {0: np.complex64, 1: np.complex128}
DT = {0: "float2", 1: "double2"}


def _run(torch, logn, batch, dtype, x, **kw):
    import turbofft_b200 as tf

    plan = tf.Plan(logn, batch, dtype, **kw)
    y = plan(torch.from_numpy(x).cuda())
    torch.cuda.synchronize()
    return plan, y.cpu().numpy()


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("logn,batch,tbs", [(7, 512, 4), (10, 64, 1), (10, 64, 8), (12, 32, 4), (16, 8, 2), (20, 2, 4), (23, 1, 8)])
def test_ft_detect_only_clean_input(torch_cuda, logn, batch, tbs, dtype):
    """--if_ft 1 without faults: same numbers as the plain kernels, nothing detected."""
    x = orc.make_input(batch, 1 << logn, CD[dtype], seed=logn)
    plan, y = _run(torch_cuda, logn, batch, dtype, x, if_ft=1, thread_bs=tbs)
    _, y0 = _run(torch_cuda, logn, batch, dtype, x)
    assert np.array_equal(y, y0)
    nd, nc, loc = plan.ft_status()
    assert nd == 0 and nc == 0 and all(k == -1 for k in loc)


def last_launch_tiles(x, row):
    """Inputs of the last launch of a plan, as [tile][line][M], in tile order.

    1 launch: tiles of C consecutive signals (zero padded).  2 and 3 launches: the first
    launch's output inter[b, k1, n2] = FFT_n1(x[b, n1, n2]) * W_N^(n2 k1); a tile of the
    last launch is C consecutive k1 of one signal (csrc/fft_kernels.cuh, ROLE_LAST)."""
    ls = planner.launches_of_row(row)
    l = ls[-1]
    C, M = 1 << l.logc, 1 << l.logm
    batch, n = x.shape
    if len(ls) == 1:
        nt = -(-batch // C)
        xt = np.zeros((nt * C, M), np.complex128)
        xt[:batch] = x
        return xt.reshape(nt, C, M), l
    n1 = 1 << ls[0].logm
    n2 = n // n1
    inter = np.fft.fft(x.astype(np.complex128).reshape(batch, n1, n2), axis=1)
    k1 = np.arange(n1)[:, None]
    c2 = np.arange(n2)[None, :]
    inter = inter * np.exp(-2j * np.pi * ((k1 * c2) % n) / n)
    if len(ls) == 2:
        return inter.reshape(batch * n1 // C, C, n2), l
    # 3 launches: the middle launch transforms the middle digit of every (b, k1) row of length n2 = m2 * m3,
    # B[b, k1, k2, n3] = FFT_m2(inter[b, k1, m2, n3]) * W_(m2 m3)^(n3 k2); a tile of the last launch is C
    # consecutive k1 at one k2, tiles ordered signal, k2, k1 group (csrc/fft_kernels.cuh, ROLE_LAST with log_q)
    assert len(ls) == 3
    m2 = 1 << ls[1].logm
    m3 = n2 // m2
    mid = np.fft.fft(inter.reshape(batch, n1, m2, m3), axis=2)
    k2 = np.arange(m2)[:, None]
    c3 = np.arange(m3)[None, :]
    mid = mid * np.exp(-2j * np.pi * ((k2 * c3) % n2) / n2)
    return mid.transpose(0, 2, 1, 3).reshape(batch * m2 * n1 // C, C, m3), l


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("logn,batch,tbs", [(4, 4096, 2), (7, 512, 4), (8, 256, 32), (10, 64, 1), (10, 64, 2), (10, 64, 16),
                                            (12, 64, 8), (13, 32, 4), (16, 16, 4), (20, 4, 8)])
def test_reference_fault_pattern_located_and_corrected(torch_cuda, logn, batch, tbs, dtype):
    """--if_err 1: every block of the last launch gets +100 on element 0 of tile
    blockIdx % thread_bs (fft_codegen.py:412-415).  Per block the flag and the located
    index must equal the CPU model's; wherever the model detects, the index is
    blockIdx % thread_bs + 1 (the reference's own commented assertion, fft_codegen.py:491)
    and the recomputed output equals the fault-free run bit for bit.  (The scheme itself
    misses some faults -- e.g. a 2^13-point line, where the +100 raises S by more than
    1000 times the residual -- and the model says so too.)"""
    # small amplitudes, like the reference's own test signals (initializeData.h:25-26,65-66)
    x = (orc.make_input(batch, 1 << logn, CD[dtype], seed=logn + 50) * 0.01).astype(CD[dtype])
    plan, y = _run(torch_cuda, logn, batch, dtype, x, if_ft=1, if_err=1, thread_bs=tbs)
    _, y0 = _run(torch_cuda, logn, batch, dtype, x)
    nd, nc, loc = plan.ft_status()
    grid = len(loc)
    tiles_x, l = last_launch_tiles(x, planner.load_params(DT[dtype])[logn])
    n_tiles = tiles_x.shape[0]
    tpl = (1 << l.logm) >> l.loge
    expect, margins = [], []
    for b in range(grid):
        tiles = orc.b200_block_tiles(b, grid, n_tiles, tbs)
        xin = tiles_x[tiles]
        xf = xin.copy()
        it = orc.injected_tile_iteration(b, tbs)
        if it <= len(tiles):
            xf[it - 1, 0, 0] += 100.0
        d = orc.ft_block_decision(xin, orc.fft_forward(xf), tpl=tpl)
        expect.append(d["k"])
        margins.append(abs(d["delta"]) / (1000.0 + d["S"]) / 1e-3)
        if d["detected"]:
            assert d["k"] == it
    assert all(m < 0.8 or m > 1.25 for m in margins), "test case too close to the threshold"
    assert loc == expect
    n_hit = sum(k != -1 for k in expect)
    assert nd == n_hit and nc == n_hit
    if n_hit == grid:
        assert np.array_equal(y, y0), "corrected output differs from the fault-free run"
        assert orc.rel_l2(y, orc.fft_forward(x)) <= orc.tolerance(CD[dtype], logn)
    else:
        assert n_hit == 0 and not np.array_equal(y, y0)   # faults the scheme cannot see stay in the output


@pytest.mark.parametrize("dtype", [0, 1])
def test_detect_only_mode_reports_but_does_not_repair(torch_cuda, dtype):
    """A fault with correction off (injection on an FT_DETECT kernel is not possible in
    the reference; here: correct plan with injection, then check the located indices are
    what an uncorrected run would report)."""
    import turbofft_b200 as tf

    torch = torch_cuda
    logn, batch, tbs = 10, 128, 4
    x = orc.make_input(batch, 1 << logn, CD[dtype], seed=3)
    plan = tf.Plan(logn, batch, dtype, if_ft=1, if_err=1, thread_bs=tbs)
    plan.set_injection(enable=False)
    y = plan(torch.from_numpy(x).cuda()).cpu().numpy()
    nd, nc, loc = plan.ft_status()
    assert nd == 0 and nc == 0
    assert orc.rel_l2(y, orc.fft_forward(x)) <= orc.tolerance(CD[dtype], logn)


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("launch", [0, 1])
def test_sparse_injection_in_either_launch(torch_cuda, dtype, launch):
    """Extension: one faulty block in `period`, in the first or the last launch of a
    two-launch plan; only those blocks fire and the output is repaired."""
    import turbofft_b200 as tf

    torch = torch_cuda
    logn, batch, tbs, period, phase = 16, 16, 4, 5, 2
    x = (orc.make_input(batch, 1 << logn, CD[dtype], seed=9) * 0.01).astype(CD[dtype])
    plan = tf.Plan(logn, batch, dtype, if_ft=1, if_err=1, thread_bs=tbs)
    plan.set_injection(True, launch=launch, period=period, phase=phase)
    y = plan(torch.from_numpy(x).cuda()).cpu().numpy()
    nd, nc, loc = plan.ft_status(launch)
    expect = [orc.injected_tile_iteration(b, tbs, period) if b % period == phase else -1 for b in range(len(loc))]
    assert loc == expect
    other = plan.ft_status(1 - launch)[2]
    assert all(k == -1 for k in other)
    assert nd == nc == sum(k != -1 for k in expect)
    _, y0 = _run(torch, logn, batch, dtype, x)
    assert np.array_equal(y, y0)


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("tbs", [2, 8])
@pytest.mark.parametrize("launch", [0, 1, 2])
def test_three_launch_plan_corrects_in_every_launch(torch_cuda, dtype, tbs, launch):
    """A three-launch plan with faults in its first, middle or last launch: the located
    indices are the injected ones and the repaired output equals the fault-free run bit for
    bit, out of place and in place.  The middle launch is the one whose input would be gone
    if it ran in place in the scratch buffer; the reference alternates two buffers
    (main.cu:11-12) and recomputes from the launch's input (fft_codegen.py:149-193)."""
    import turbofft_b200 as tf

    torch = torch_cuda
    logn, batch, period, phase = 23, 1, 5, 2
    assert len(planner.launches_of_row(planner.load_params(DT[dtype])[logn])) == 3
    # Amplitude 1e-4: the clean data's share of S stays far below err_smoothing in every launch,
    # so a +100 fault clears the threshold by an order of magnitude whatever thread_bs is (with
    # larger data the scheme itself stops seeing the fault; see the two-launch test above).
    x = (orc.make_input(batch, 1 << logn, CD[dtype], seed=23) * 1e-4).astype(CD[dtype])
    _, y0 = _run(torch, logn, batch, dtype, x)
    plan = tf.Plan(logn, batch, dtype, if_ft=1, if_err=1, thread_bs=tbs)
    plan.set_injection(True, launch=launch, period=period, phase=phase)
    for inplace in (False, True):
        xd = torch.from_numpy(x).cuda()
        y = plan(xd, out=xd if inplace else None).cpu().numpy()
        nd, nc, loc = plan.ft_status(launch)
        expect = [orc.injected_tile_iteration(b, tbs, period) if b % period == phase else -1 for b in range(len(loc))]
        assert loc == expect
        for other in {0, 1, 2} - {launch}:
            assert all(k == -1 for k in plan.ft_status(other)[2])
        assert nd == nc == sum(k != -1 for k in expect) > 0
        assert np.array_equal(y, y0), (launch, inplace)


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("logn,tbs", [(10, 4), (12, 2), (8, 8)])
def test_decisions_match_cpu_model(torch_cuda, logn, tbs, dtype):
    """Per block (delta, S, delta_w) from the kernel against the CPU restatement of the
    decision on the same tiles; flags and indices must be identical, values close."""
    import turbofft_b200 as tf

    torch = torch_cuda
    batch = 256
    x = orc.make_input(batch, 1 << logn, CD[dtype], seed=logn)
    plan = tf.Plan(logn, batch, dtype, if_ft=1, if_err=1, thread_bs=tbs)
    plan.enable_ft_diag(True)
    plan(torch.from_numpy(x).cuda())
    nd, nc, loc = plan.ft_status()
    diag = plan.ft_diag()
    row = planner.load_params(DT[dtype])[logn]
    l = planner.launches_of_row(row)[0]
    C, M = 1 << l.logc, 1 << l.logm
    tpl = M >> l.loge
    n_tiles = -(-batch // C)
    grid = len(loc)
    xt = np.zeros((n_tiles * C, M), np.complex128)
    xt[:batch] = x
    xt = xt.reshape(n_tiles, C, M)
    for b in range(0, grid, max(1, grid // 16)):
        tiles = orc.b200_block_tiles(b, grid, n_tiles, tbs)
        xin = xt[tiles].copy()
        hit = orc.injected_tile_iteration(b, tbs)
        xfault = xin.copy()
        if hit <= len(tiles):
            xfault[hit - 1, 0, 0] += 100.0
        d = orc.ft_block_decision(xin, orc.fft_forward(xfault), tpl=tpl, acc_dtype=np.float64)
        assert d["k"] == loc[b], (b, d, loc[b])
        assert d["detected"] == (loc[b] != -1)
        gd, gs, gw = diag[b]
        rt = 2e-3 if dtype == 0 else 1e-9
        assert abs(gd - d["delta"]) <= rt * (abs(d["delta"]) + 1e-3 * d["S"] + 1)
        assert abs(gs - d["S"]) <= 5e-3 * d["S"] + 1
        assert abs(gw - d["delta_w"]) <= rt * (abs(d["delta_w"]) + 1e-3 * d["S"] * tbs + 1)


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("logn,batch,tbs,inplace", [(7, 512, 4, True), (10, 64, 2, True), (10, 64, 8, False), (12, 64, 4, True),
                                                   (16, 16, 4, False), (18, 8, 2, True)])
def test_correction_from_checksums(torch_cuda, logn, batch, tbs, inplace, dtype):
    """tfft_set_correction(1): the located tile is repaired with sum(y) - F(sum(x)) over the
    block's tiles (the reference's commented-out path, fft_codegen.py:356-357,422-429) instead
    of being recomputed, so single-launch plans may run in place.  Same detections and located
    indices as the recompute mode; repaired values agree with the fault-free run to rounding."""
    import turbofft_b200 as tf

    torch = torch_cuda
    x = (orc.make_input(batch, 1 << logn, CD[dtype], seed=logn + 7) * 0.01).astype(CD[dtype])
    _, y0 = _run(torch, logn, batch, dtype, x)
    ref = tf.Plan(logn, batch, dtype, if_ft=1, if_err=1, thread_bs=tbs)
    ref(torch.from_numpy(x).cuda())
    nd0, nc0, loc0 = ref.ft_status()
    plan = tf.Plan(logn, batch, dtype, if_ft=1, if_err=1, thread_bs=tbs)
    plan.set_correction(True)
    xd = torch.from_numpy(x).cuda()
    y = plan(xd, out=xd if inplace else None).cpu().numpy()
    nd, nc, loc = plan.ft_status()
    assert (nd, nc, loc) == (nd0, nc0, loc0) and nd == len(loc) > 0
    scale = np.abs(y0).max()
    assert np.abs(y - y0).max() <= (2e-5 if dtype == 0 else 1e-12) * scale * tbs
    assert orc.rel_l2(y, orc.fft_forward(x)) <= 4 * orc.tolerance(CD[dtype], logn)


def test_threshold_parameters_are_honoured(torch_cuda):
    """A tiny fault stays below err_threshold and is ignored; lowering the threshold finds it."""
    import turbofft_b200 as tf

    torch = torch_cuda
    logn, batch, tbs = 10, 64, 2
    x = orc.make_input(batch, 1 << logn, np.complex64, seed=4)
    plan = tf.Plan(logn, batch, 0, if_ft=1, if_err=1, thread_bs=tbs)
    plan.set_ft_params(err_inj=0.5, err_smoothing=1000.0, err_threshold=1e-3)
    plan(torch.from_numpy(x).cuda())
    nd, _, _ = plan.ft_status()
    assert nd == 0                       # 0.5 / (1000 + S) < 1e-3
    plan.set_ft_params(err_inj=0.5, err_smoothing=1.0, err_threshold=1e-5)
    y = plan(torch.from_numpy(x).cuda()).cpu().numpy()
    nd, nc, loc = plan.ft_status()
    assert nd == len(loc) == nc
    assert orc.rel_l2(y, orc.fft_forward(x)) <= orc.tolerance(np.complex64, logn)


def test_inplace_single_launch_correction_is_refused(torch_cuda):
    import turbofft_b200 as tf

    torch = torch_cuda
    x = torch.zeros(16, 1024, dtype=torch.complex64, device="cuda")
    plan = tf.Plan(10, 16, 0, if_ft=1, if_err=1)
    with pytest.raises(tf.TurboFFTError):
        plan(x, out=x)
