"""CPU tests of the oracle itself: it must be pinned before it is trusted."""
import ctypes
import glob
import os

import numpy as np
import pytest

from oracle import fft_oracle as orc

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_glibc_random_matches_libc():
    libc = ctypes.CDLL("libc.so.6")
    libc.random.restype = ctypes.c_long
    libc.srandom(10)
    ref = np.array([libc.random() for _ in range(4096)])
    assert np.array_equal(ref, orc.glibc_random(10, 4096))


def test_reference_input_distribution():
    x = orc.reference_input(4, 256, np.complex64)
    assert x.dtype == np.complex64 and x.shape == (4, 256)
    vals = np.unique(np.round(x.real * 100).astype(int))
    assert vals.min() >= -50 and vals.max() <= 49
    xd = orc.reference_input(2, 64, np.complex128)
    assert np.abs(xd.real).max() <= 0.05


@pytest.mark.parametrize("logn", [1, 2, 3, 5, 8, 10])
def test_fft_forward_vs_direct_dft(logn):
    x = orc.make_input(3, 1 << logn, np.complex128, seed=logn)
    assert orc.rel_l2(orc.fft_forward(x), orc.dft_direct(x)) < 1e-15 * max(4, logn * 4)


def test_sign_and_scaling_convention():
    n = 64
    x = np.zeros(n, complex)
    x[1] = 1.0
    k = np.arange(n)
    assert np.allclose(orc.fft_forward(x), np.exp(-2j * np.pi * k / n))   # forward sign
    assert np.allclose(orc.fft_forward(np.ones(n)), np.r_[n, np.zeros(n - 1)])  # unnormalised


def test_twiddle_table_layout():
    t = orc.twiddle_table(16)
    assert t.shape == (31,)
    assert np.allclose(t[0], 1)               # size 1
    assert np.allclose(t[1:3], [1, -1])       # size 2
    assert np.allclose(t[3:7], [1, -1j, -1, 1j])
    j = np.arange(16)
    assert np.allclose(t[15:31], np.exp(-2j * np.pi * j / 16), atol=1e-6)


def test_dft_bins_matches_fft():
    x = orc.make_input(1, 4096, np.complex128, seed=5)[0]
    bins = [0, 1, 77, 4095]
    assert np.allclose(orc.dft_bins(x, bins), orc.fft_forward(x)[bins], rtol=1e-12, atol=1e-10)


def test_compare_data_semantics():
    ref = np.array([1 + 1j, 2 + 2j, 3 + 3j], np.complex64)
    ok, _, _ = orc.compare_data(ref.copy(), ref)
    assert ok
    bad = ref.copy()
    bad[1] += 1e-3j
    ok, i, comp = orc.compare_data(bad, ref, 1e-4)
    assert (ok, i, comp) == (False, 1, "y")
    nan = ref.copy()
    nan[2] = complex(np.nan, 3)
    ok, i, comp = orc.compare_data(nan, ref, 1e-4)
    assert (ok, i, comp) == (False, 2, "x")


@pytest.mark.parametrize("m", [2, 8, 64, 256])
def test_checksum_identity(m):
    """r^T (W x) == (W r)^T x: the algebra both ABFT sides rest on."""
    x = orc.make_input(1, m, np.complex128, seed=m)[0]
    y = orc.fft_forward(x)
    lhs = np.sum(y * orc.checksum_weights(m))
    rhs = np.sum(x * orc.dft_matrix_checksum(m))
    assert abs(lhs - rhs) < 1e-10 * m
    # the reference's float-angle evaluation of c differs only by float32 angle error
    cf = orc.dft_matrix_checksum(m, float_angles=True)
    assert np.abs(cf - orc.dft_matrix_checksum(m)).max() < 2e-5 * m * m


def _block(nt, lines, m, seed, dtype=np.complex64):
    x = orc.make_input(nt * lines, m, dtype, seed=seed).reshape(nt, lines, m)
    return x.astype(np.complex128)


@pytest.mark.parametrize("acc", [np.float32, np.float64])
def test_ft_model_clean_run_detects_nothing(acc):
    x = _block(4, 2, 256, seed=1)
    d = orc.ft_block_decision(x, orc.fft_forward(x), tpl=16, acc_dtype=acc)
    assert not d["detected"] and d["k"] == -1
    assert abs(d["delta"]) / (1000 + d["S"]) < 1e-5


@pytest.mark.parametrize("m,tpl", [(256, 16), (512, 32), (1024, 64), (128, 8)])
@pytest.mark.parametrize("hit", [1, 2, 3, 4])
def test_ft_model_locates_injected_tile(m, tpl, hit):
    """+100 on element 0 of the first line of tile `hit` after the input checksum:
    the output checksum moves by 100*fold(sum_k r_{k%3}), detection fires and the
    weighted copy points at the tile (fft_codegen.py:412-415, 495)."""
    x = _block(4, 2, m, seed=hit)
    xin = x.copy()
    xin[hit - 1, 0, 0] += 100.0
    y = orc.fft_forward(xin)       # what the block stores
    d = orc.ft_block_decision(x, y, tpl=tpl, acc_dtype=np.float32)
    assert d["detected"] and d["k"] == hit
    shift = 100.0 * orc.fold(orc.checksum_weights(m).sum())
    assert abs(abs(d["delta"]) - abs(shift)) < 1e-2 * abs(shift) + 1e-2


def test_block_tile_orders():
    assert orc.b200_block_tiles(3, 10, 25, 4) == [3, 13, 23]
    assert orc.b200_block_tiles(7, 10, 25, 4) == [7, 17]
    # reference: tb_gap = (128K / smem) * 108; with a 32 KB tile that is 432
    t = orc.reference_block_tiles(5, 1000, 4000, 4, 32 * 1024)
    assert t == [5, 5 + 432, 5 + 864, 5 + 1296]
    assert orc.injected_tile_iteration(6, 4) == 3
    assert orc.injected_tile_iteration(6, 4, period=2) == 4


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "ref_outputs_*.npz"))) or [None])
def test_oracle_matches_reference_kernel_outputs(path):
    """Golden vectors: outputs of the unmodified reference kernels (compiled for sm_100a,
    run on a B200 by tests/golden/make_golden.py) for seeded inputs."""
    if path is None:
        pytest.skip("no golden fixtures present")
    g = np.load(path)
    for key in [k for k in g.files if k.startswith("out_")]:
        _, dt, logn, bs = key.split("_")
        dtype = np.complex64 if dt == "0" else np.complex128
        x = orc.reference_input(int(bs), 1 << int(logn), dtype)
        ref = orc.fft_forward(x)
        tol = (2e-6 if dt == "0" else 1e-14) * max(1, int(logn))
        assert orc.rel_l2(g[key], ref) <= tol, key
        # the reference's per-component test, with head-room for fp32 rounding of both sides
        ok, i, comp = orc.compare_data(g[key], ref.astype(dtype), 1e-3)
        assert ok, (key, i, comp)


def test_dft_bins_by_row_blocks_matches_fft():
    """The regrouped direct sum used to spot-check very long transforms equals the FFT bins,
    whichever way the rows are split over callers."""
    rng = np.random.default_rng(5)
    n1, n2 = 64, 128
    x = (rng.uniform(-1, 1, n1 * n2) + 1j * rng.uniform(-1, 1, n1 * n2)).astype(np.complex64)
    bins = np.array([0, 1, 77, n1 * n2 // 2, n1 * n2 - 1, 4097])
    inner = sum(orc.dft_bins_partial(x[r * n2:(r + 16) * n2], r, n1, n2, bins) for r in range(0, n1, 16))
    got = orc.dft_bins_finish(inner, n1, n2, bins)
    assert np.allclose(got, orc.fft_forward(x)[bins], rtol=1e-11, atol=1e-9)
    assert np.allclose(got, orc.dft_bins(x, bins), rtol=1e-11, atol=1e-9)
