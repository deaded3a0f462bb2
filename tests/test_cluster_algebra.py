"""CPU model of the single-pass cluster kernel's data movement (csrc/cluster_fft.cuh).

Replays, in numpy, what every thread of a cluster reads and writes -- stage-0 butterflies on
interleaved data, then radix-R stages on two-value units, with the per-stage thread-to-CTA
maps and the local index of every unit -- and checks that (1) the result is the DFT, (2) every
exchange but the one behind stage 1 stays inside its CTA, (3) every exchange is a bijection
onto the CTAs' unit arrays.  No GPU involved; the kernel's own parity tests are in
test_gpu_single_pass.py.
"""
import numpy as np
import pytest


def _cfg(logn, lr0, lr, logg):
    s2 = (logn - lr0) // lr
    assert lr0 + lr * s2 == logn
    logt = logn - 1 - lr
    rp = [logt - lr0 + 1 - logg, logt - logg] + [lr0 - 1 + lr - logg] * (s2 - 1)
    return dict(N=1 << logn, U=1 << (logn - 1), T=1 << logt, TH=1 << (logt - logg), G=1 << logg, R0=1 << lr0, R=1 << lr,
                S2=s2, LOGG=logg, RP=rp)


def _split(c, t, s):
    rp, lg = c["RP"][t], c["LOGG"]
    return (s >> rp) & (c["G"] - 1), ((s >> (rp + lg)) << rp) | (s & ((1 << rp) - 1))


def _w(num, den):
    return np.exp(-2j * np.pi * (num % den) / den)


def _run(c, x):
    n, u, t_, th, g, r0, r, s2 = (c[k] for k in ("N", "U", "T", "TH", "G", "R0", "R", "S2"))
    nb0 = 2 * r // r0
    smem = np.full((g, r * th, 2), np.nan, complex)
    remote, hits = [], np.zeros((g, r * th), int)
    s = np.arange(t_)
    rank, _ = _split(c, 0, s)
    nrem = 0
    for ub in range(nb0):
        b = s + ub * t_
        v = x[b[:, None] + np.arange(r0)[None, :] * (n // r0)]
        y = np.fft.fft(v, axis=1) * _w(b[:, None] * np.arange(r0)[None, :], n)
        for q in range(0, r0, 2):
            m = (q >> 1) + (r0 // 2) * b
            r1, l1 = _split(c, 1, m % t_)
            idx = (m // t_) * th + l1
            smem[r1, idx, 0], smem[r1, idx, 1] = y[:, q], y[:, q + 1]
            np.add.at(hits, (r1, idx), 1)
            nrem += int((r1 != rank).sum())
    remote.append(nrem)
    assert (hits == 1).all()
    pp_ = r0 // 2
    out = np.zeros(n, complex)
    for t in range(1, s2 + 1):
        rank, lid = _split(c, t, s)
        v = np.stack([smem[rank, j * th + lid] for j in range(r)], axis=1)      # [T][R][2]
        y = np.fft.fft(v, axis=1)
        if t == s2:
            for q in range(r):
                m = s + q * t_
                out[2 * m], out[2 * m + 1] = y[:, q, 0], y[:, q, 1]
            break
        p, nlo = s % pp_, s // pp_
        y = y * _w(nlo[:, None] * pp_ * np.arange(r)[None, :], u)[:, :, None]
        new = np.full_like(smem, np.nan)
        hits[:] = 0
        nrem = 0
        for q in range(r):
            m = p + q * pp_ + nlo * pp_ * r
            r2, l2 = _split(c, t + 1, m % t_)
            idx = (m // t_) * th + l2
            new[r2, idx] = y[:, q]
            np.add.at(hits, (r2, idx), 1)
            nrem += int((r2 != rank).sum())
            if t == 1 and g > 1 and c["LOGG"] <= int(np.log2(r)):
                # the receiving CTA of the crossing exchange depends on q alone: top bits of q
                assert (r2 == (q >> (int(np.log2(r)) - c["LOGG"]))).all()
        assert (hits == 1).all()
        remote.append(nrem)
        smem = new
        pp_ *= r
    return out, remote


@pytest.mark.parametrize("logn,lr0,lr,logg", [(13, 1, 4, 0), (13, 1, 4, 1), (14, 2, 4, 1), (14, 2, 4, 2), (15, 3, 4, 3),
                                              (16, 4, 4, 4), (17, 5, 4, 4), (12, 3, 3, 0), (13, 4, 3, 1), (14, 2, 3, 2),
                                              (15, 3, 3, 3), (16, 4, 3, 4)])
def test_cluster_index_maps_give_the_transform(logn, lr0, lr, logg):
    c = _cfg(logn, lr0, lr, logg)
    rng = np.random.default_rng(logn)
    x = rng.standard_normal(c["N"]) + 1j * rng.standard_normal(c["N"])
    out, remote = _run(c, x)
    ref = np.fft.fft(x)
    assert np.abs(out - ref).max() <= 1e-12 * np.abs(ref).max()
    # exactly one exchange crosses CTAs (none without a cluster), and it moves (G-1)/G of the units
    assert remote[0] == 0 and all(r == 0 for r in remote[2:])
    assert remote[1] == (c["U"] * (c["G"] - 1)) // c["G"]
