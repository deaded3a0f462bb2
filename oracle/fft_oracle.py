"""CPU oracle for the batched C2C FFT + ABFT path.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg may import this
module; the product (turbofft_b200/) never does and has no CPU path of its own.

It restates, in numpy float64 (plus a long-double direct DFT in dft_oracle.c), what
the reference's GPU kernels and host utilities compute; every function cites the
reference lines it follows.  How it is pinned (the reference ships no tests, golden
vectors or CPU implementation, and its kernels only run on a GPU):
  * glibc_random()/reference_input() are checked against the C library's own
    srandom/random, which initializeData() calls;
  * fft_forward() is checked against the independent direct DFT and analytic
    identities (tests/test_oracle.py);
  * tests/golden/ref_outputs_*.npz hold outputs of the UNMODIFIED reference kernels
    (oracle/ref_harness.cu, compiled for sm_100a, run on a B200) for seeded inputs;
    the oracle is compared with them on the CPU and, in the GPU tests, with the
    reference library run live.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

# ------------------------------------------------------------------------------ transform


def fft_forward(x: np.ndarray) -> np.ndarray:
    """Forward unnormalised DFT along the last axis in float64.

    X[k] = sum_n x[n] exp(-2 pi i n k / N): the sign is the one of the reference's
    twiddle table (include/utils/initializeData.h:31-37, angle = -2 pi j / N) and of
    the cuFFT call it verifies against (include/cufft/cufft.h:23,64, CUFFT_FORWARD);
    no 1/N anywhere (main.cu:53-62 launches the kernels and nothing else).
    """
    return np.fft.fft(np.asarray(x, dtype=np.complex128), axis=-1)


_dft_lib = None


def _dft():
    global _dft_lib
    if _dft_lib is None:
        path = os.path.join(HERE, "libdft_oracle.so")
        if not os.path.exists(path):
            raise RuntimeError(f"{path} missing: run `make -C oracle`")
        lib = ctypes.CDLL(path)
        lib.dft_oracle.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_longlong]
        lib.dft_oracle.restype = None
        lib.dft_oracle_bins.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_int,
                                        ctypes.c_void_p]
        lib.dft_oracle_bins.restype = None
        _dft_lib = lib
    return _dft_lib


def dft_direct(x: np.ndarray) -> np.ndarray:
    """O(N^2) long-double DFT (oracle/dft_oracle.c); independent of any FFT algorithm."""
    x = np.ascontiguousarray(x, dtype=np.complex128)
    n = x.shape[-1]
    batch = x.size // n
    out = np.empty_like(x)
    _dft().dft_oracle(x.ctypes.data, out.ctypes.data, n, batch)
    return out


def dft_bins(x: np.ndarray, bins) -> np.ndarray:
    """Selected output bins of one long signal, by direct summation in long double."""
    x = np.ascontiguousarray(x, dtype=np.complex128).reshape(-1)
    bins = np.ascontiguousarray(bins, dtype=np.int64)
    out = np.empty(bins.size, dtype=np.complex128)
    _dft().dft_oracle_bins(x.ctypes.data, x.size, bins.ctypes.data, bins.size, out.ctypes.data)
    return out


def dft_bins_partial(x_rows: np.ndarray, row0: int, n1: int, n2: int, bins) -> np.ndarray:
    """Share of rows [row0, row0 + rows) of the signal x[n1 * N2 + n2], viewed as an N1 x N2
    matrix, in the inner sums of selected output bins of ONE long transform (N = N1 * N2):

        X[k] = sum_n2 W_N^(n2 k) * inner[n2, k],   inner[n2, k] = sum_n1 x[n1, n2] W_N1^(n1 k)

    Returns inner's partial sum over the given rows as [N2, len(bins)] complex128; the shares
    of all row blocks add up to inner, and dft_bins_finish() turns it into X[bins].  This is
    the direct DFT sum regrouped into one matrix product per row block -- O(N) per bin like
    dft_bins(), but in float64 BLAS, which makes 2^30-point signals checkable in seconds.  It
    is how the distributed transform (rows block-distributed over ranks) is spot-checked:
    each rank sums its own rows."""
    bins = np.asarray(bins, dtype=np.int64)
    rows = x_rows.size // n2
    x_rows = x_rows.reshape(rows, n2)
    acc = np.zeros((n2, bins.size), np.complex128)
    step = max(1, (1 << 24) // n2)
    for r in range(0, rows, step):
        r1 = min(rows, r + step)
        idx = (np.arange(row0 + r, row0 + r1, dtype=np.int64)[:, None] * (bins[None, :] % n1)) % n1
        v = np.exp(-2j * np.pi * idx / n1)
        acc += x_rows[r:r1].astype(np.complex128).T @ v
    return acc


def dft_bins_finish(inner: np.ndarray, n1: int, n2: int, bins) -> np.ndarray:
    """X[bins] from the summed inner sums of dft_bins_partial()."""
    bins = np.asarray(bins, dtype=np.int64)
    n = n1 * n2
    idx = (np.arange(n2, dtype=np.int64)[:, None] * bins[None, :]) % n
    return (np.exp(-2j * np.pi * idx / n) * inner).sum(axis=0)


def rel_l2(a: np.ndarray, ref: np.ndarray) -> float:
    """||a - ref||_2 / ||ref||_2 over the whole array, in float64."""
    a = np.asarray(a, dtype=np.complex128).reshape(-1)
    ref = np.asarray(ref, dtype=np.complex128).reshape(-1)
    den = np.linalg.norm(ref)
    return float(np.linalg.norm(a - ref) / (den if den > 0 else 1.0))


def tolerance(dtype, logn: int) -> float:
    """Relative-L2 bound: 1e-6*log2N for complex64, 1e-14*log2N for complex128."""
    return (1e-6 if np.dtype(dtype) == np.complex64 else 1e-14) * max(1, logn)


def compare_data(res: np.ndarray, ref: np.ndarray, error_bound: float = 1e-4):
    """The reference's own acceptance test, compareData() (include/utils/compareData.h:4-35).

    Per component |res - ref| / (1 + |ref|) > bound, or NaN, fails; like the reference
    it reports the first offender only.  Returns (ok, first_bad_index, component).
    """
    res = np.asarray(res).reshape(-1)
    ref = np.asarray(ref).reshape(-1)
    ex = np.abs((res.real - ref.real) / (1 + np.abs(ref.real)))
    ey = np.abs((res.imag - ref.imag) / (1 + np.abs(ref.imag)))
    badx = (ex > error_bound) | np.isnan(res.real)
    bady = (ey > error_bound) | np.isnan(res.imag)
    bad = badx | bady
    if not bad.any():
        return True, -1, ""
    i = int(np.argmax(bad))
    return False, i, ("x" if badx[i] else "y")


# ------------------------------------------------------------------------------ inputs


def make_input(batch: int, n: int, dtype, seed: int = 0) -> np.ndarray:
    """Seeded synthetic signals with the benchmark configurations' distributions:
    complex64: re/im i.i.d. uniform[-1, 1); complex128: re/im i.i.d. N(0, 1)."""
    rng = np.random.default_rng(seed)
    if np.dtype(dtype) == np.complex64:
        a = rng.uniform(-1.0, 1.0, size=(batch, n, 2)).astype(np.float32)
        return a.view(np.complex64).reshape(batch, n)
    a = rng.standard_normal(size=(batch, n, 2))
    return a.view(np.complex128).reshape(batch, n)


def glibc_random(seed: int, count: int) -> np.ndarray:
    """glibc's random() after srandom(seed) (TYPE_3 additive-feedback generator,
    r[i] = r[i-3] + r[i-31]); initializeData() draws its inputs from it
    (include/utils/initializeData.h:6-7,25-26)."""
    r = [0] * (344 + count)
    r[0] = seed
    for i in range(1, 31):
        r[i] = (16807 * r[i - 1]) % 2147483647
    for i in range(31, 34):
        r[i] = r[i - 31]
    for i in range(34, 344 + count):
        r[i] = (r[i - 31] + r[i - 3]) & 0xFFFFFFFF
    return np.array([v >> 1 for v in r[344:]], dtype=np.int64)


def reference_input(batch: int, n: int, dtype) -> np.ndarray:
    """The reference's own test signals: srandom(10), then per element
    x = (random() % 100 - 50) / 100 and y likewise for float2
    (initializeData.h:65-66), / 1000 for double2 (initializeData.h:25-26)."""
    v = glibc_random(10, 2 * batch * n)
    scale = 100.0 if np.dtype(dtype) == np.complex64 else 1000.0
    a = ((v % 100 - 50).astype(np.float64) / scale).reshape(batch, n, 2)
    if np.dtype(dtype) == np.complex64:
        return a.astype(np.float32).view(np.complex64).reshape(batch, n)
    return a.view(np.complex128).reshape(batch, n)


# ------------------------------------------------------------------------------ host tables


def twiddle_table(n: int) -> np.ndarray:
    """The reference's concatenated twiddle table (initializeData.h:31-37): entry
    size-1+j = exp(-2 pi i j / size) for size = 1, 2, 4, ..., n, with the ratio
    j/size formed in float32 as the reference does ((float)j / (float)size)."""
    out = np.empty(2 * n - 1, dtype=np.complex128)
    size = 1
    while size <= n:
        j = np.arange(size)
        ratio = (j.astype(np.float32) / np.float32(size)).astype(np.float64)
        ang = -2.0 * np.pi * ratio
        out[size - 1: 2 * size - 1] = np.cos(ang) + 1j * np.sin(ang)
        size *= 2
    return out


R_CUBE = np.array([1.0 + 0.0j, -0.5 - 0.8660253882408142j, -0.5 + 0.8660253882408142j])
"""r_j = omega^j with the float32-rounded sqrt(3)/2 of include/turbofft/constants.h:2-7."""


def checksum_weights(m: int) -> np.ndarray:
    """r_{k mod 3}, k < m: the right-side ABFT weights (fft_codegen.py:219-225, 374-384)."""
    return R_CUBE[np.arange(m) % 3]


def dft_matrix_checksum(m: int, float_angles: bool = False) -> np.ndarray:
    """c = W_m r, the left-side ABFT encoding vector of getDFTMatrixChecksum()
    (include/utils/abft.h:21-61): c_i = sum_j exp(-2 pi i i j / m) r_{j mod 3}.

    float_angles=True reproduces the reference's evaluation order, which forms the
    angle -(float)(2 pi i j) / float(m) in float32 (abft.h:34-35, 54-55); False is the
    exact vector (what the B200 library uploads).  The FT identity holds for either;
    they differ by the float32 angle error.
    """
    if not float_angles:
        return np.fft.fft(checksum_weights(m))
    i = np.arange(m, dtype=np.float64)[:, None]
    j = np.arange(m, dtype=np.float64)[None, :]
    ang = -((2.0 * np.pi * i * j).astype(np.float32) / np.float32(m)).astype(np.float64)
    w = np.cos(ang) + 1j * np.sin(ang)
    return w @ checksum_weights(m)


# ------------------------------------------------------------------------------ FT decision


def fold(z: np.ndarray) -> np.ndarray:
    """Re z + Im z: how the reference collapses a complex checksum term to one real
    number (fft_codegen.py:364-366: tmp_1.x += tmp.x + tmp.y)."""
    return z.real + z.imag


def ft_block_decision(x_tiles: np.ndarray, y_tiles: np.ndarray, tpl: int,
                      err_smoothing: float = 1000.0, err_threshold: float = 1e-3,
                      acc_dtype=np.float64, cvec: np.ndarray | None = None):
    """One thread block's ABFT decision (fft_codegen.py:359-367, 374-384, 432-503).

    x_tiles, y_tiles: [tiles_of_the_block][lines][M] -- what the block loaded and what
    it is about to store (before the inter-launch twiddle), in its iteration order.
    tpl = M / points_per_thread: thread (s, line) owns rows s + i*tpl on both sides,
    which is the element-to-thread map of the reference kernels (rows tx/BS + i*Ni/ni,
    column tx % BS; fft_codegen.py:351-372, 417-431) and of the B200 kernels alike.

    Per thread: in_t = sum fold(x c), out_t = sum fold(y r), both over all its tiles,
    and the tile-counter-weighted copies (weights 1..tiles).  Block: delta = sum(in_t
    - out_t), S = sum(|in_t| + |out_t|), delta_w likewise weighted;
    detected = |delta| / (err_smoothing + S) > err_threshold,
    k = round(|delta_w| / |delta|) is the 1-based tile iteration (fft_codegen.py:495).
    Returns dict(delta, S, delta_w, detected, k) with k = -1 when nothing is detected.
    """
    x_tiles = np.asarray(x_tiles, dtype=np.complex128)
    y_tiles = np.asarray(y_tiles, dtype=np.complex128)
    nt, lines, m = x_tiles.shape
    c = dft_matrix_checksum(m) if cvec is None else cvec
    r = checksum_weights(m)
    fin = fold(x_tiles * c[None, None, :]).astype(acc_dtype)   # [tiles][lines][rows]
    fout = fold(y_tiles * r[None, None, :]).astype(acc_dtype)
    # rows s + i*tpl belong to thread s
    fin_t = fin.reshape(nt, lines, m // tpl, tpl).sum(axis=2, dtype=acc_dtype)   # [tiles][lines][s]
    fout_t = fout.reshape(nt, lines, m // tpl, tpl).sum(axis=2, dtype=acc_dtype)
    w = np.arange(1, nt + 1, dtype=acc_dtype)[:, None, None]
    in_t = fin_t.sum(axis=0, dtype=acc_dtype)
    out_t = fout_t.sum(axis=0, dtype=acc_dtype)
    dw_t = (w * (fin_t - fout_t)).sum(axis=0, dtype=acc_dtype)
    delta = float((in_t - out_t).sum(dtype=acc_dtype))
    s = float((np.abs(in_t) + np.abs(out_t)).sum(dtype=acc_dtype))
    dw = float(dw_t.sum(dtype=acc_dtype))
    detected = abs(delta) / (err_smoothing + abs(s)) > err_threshold
    k = -1
    if detected:
        q = abs(dw) / abs(delta)
        k = int(np.floor(q + 0.5))  # C round(): halves away from zero, q >= 0
    return dict(delta=delta, S=s, delta_w=dw, detected=bool(detected), k=k)


def reference_block_tiles(block: int, grid: int, n_tiles: int, thread_bs: int, smem_bytes: int):
    """Tile ids a reference block visits, in order (fft_codegen.py:216-218, 259-265):
    tb_gap = (128 KB / smem of a tile) * 108; block b starts at
    (b / tb_gap) * tb_gap * thread_bs + b % tb_gap and advances by delta_bid."""
    tb_gap = (128 * 1024 // smem_bytes) * 108
    delta = (grid % tb_gap) if (block // tb_gap) == (grid // tb_gap) else tb_gap
    bid = (block // tb_gap) * tb_gap * thread_bs + block % tb_gap
    out = []
    while len(out) < thread_bs and bid < n_tiles:
        out.append(bid)
        bid += delta
    return out


def b200_block_tiles(block: int, grid: int, n_tiles: int, thread_bs: int):
    """Tile ids a B200 block visits: block + it * grid, it < thread_bs."""
    return [block + it * grid for it in range(thread_bs) if block + it * grid < n_tiles]


def injected_tile_iteration(block: int, thread_bs: int, period: int = 1) -> int:
    """1-based tile iteration the fault lands in: blockIdx.x % thread_bs + 1 in the
    reference (fft_codegen.py:412-415); the B200 library generalises the block index
    to block / period for sparse injection (period 1 = the reference)."""
    return (block // period) % thread_bs + 1
