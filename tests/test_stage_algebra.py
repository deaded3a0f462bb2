"""CPU checks of the in-block exchange algebra the kernels rely on (csrc/fft_kernels.cuh):
the Stockham address maps of every shipped instance with its generated shared-memory layout
(PADSHIFT, EXTRA, REMLAST), and a numpy restatement of one tile for both stage orders."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from turbofft_b200 import planner
from turbofft_b200.codegen import smem_layout as sl


def stage_plan(logm, loge, remlast):
    s = (logm + loge - 1) // loge
    r0 = logm - (s - 1) * loge
    if remlast:
        return [(r0 if t == s - 1 else loge, t * loge) for t in range(s)]
    return [(r0 if t == 0 else loge, 0 if t == 0 else r0 + (t - 1) * loge) for t in range(s)]


def shipped_instances():
    out = set()
    for dt, f64 in (("float2", False), ("double2", True)):
        for logn, row in planner.load_params(dt, "B200").items():
            if row.launches == 0:
                continue
            for l in planner.launches_of_row(row):
                if l.stages >= 2:
                    out.add((f64, l.role, l.logm, l.loge, l.logc))
    return sorted(out)


def address_maps(role, logm, loge, logc, ps, ex, remlast):
    """Per stage: (write addresses, read addresses of the next stage) as flat arrays over all threads."""
    M, E, C = 1 << logm, 1 << loge, 1 << logc
    tpl = M // E
    pad = lambda a: a + (a >> ps)
    mpad = pad(M - 1) + 1
    pitch = mpad + ex
    cols = role == planner.ROLE_FIRST
    soff = (lambda a, c: pad(a) * C + c) if cols else (lambda a, c: c * pitch + pad(a))
    size = mpad * C if cols else pitch * C
    s_idx, c_idx = np.meshgrid(np.arange(tpl), np.arange(C), indexing="ij")
    s_idx, c_idx = s_idx.reshape(-1), c_idx.reshape(-1)
    plan = stage_plan(logm, loge, remlast)
    maps = []
    for t, (lr, lp) in enumerate(plan[:-1]):
        R, P, nb = 1 << lr, 1 << lp, E >> lr
        wr = []
        for u in range(nb):
            b = s_idx + u * tpl
            base = (b & (P - 1)) + ((b >> lp) << (lp + lr))
            for q in range(R):
                wr.append(soff(base + (q << lp), c_idx))
        rd = [soff(s_idx + i * tpl, c_idx) for i in range(E)]
        maps.append((np.concatenate(wr), np.concatenate(rd), size))
    return maps


def test_every_shipped_layout_is_a_bijection():
    """No two elements of a tile share a shared-memory word, nothing falls outside the buffer, and
    a stage reads exactly what the stage before it wrote -- for the generated layout of every
    instance the shipped parameter tables use."""
    cache = sl.load_cache()
    inst = shipped_instances()
    assert len(inst) > 30
    for f64, role, logm, loge, logc in inst:
        key = f"{int(f64)}_{role}_{logm}_{loge}_{logc}"
        assert key in cache, key
        ps, ex = cache[key][:2]
        rl = bool(cache[key][2]) if len(cache[key]) > 2 else False
        for wr, rd, size in address_maps(role, logm, loge, logc, ps, ex, rl):
            n = (1 << logm) << logc
            assert wr.size == n and np.unique(wr).size == n, key
            assert wr.min() >= 0 and wr.max() < size, key
            assert np.array_equal(np.sort(wr), np.sort(rd)), key


def brev(q, lr):
    return int(format(q, f"0{lr}b")[::-1], 2) if lr else 0


def dif(v):
    """Radix-len(v) decimation in frequency; X[q] is left at position brev(q)."""
    v = list(v)
    half = len(v) // 2
    while half >= 1:
        for blk in range(0, len(v), 2 * half):
            for j in range(half):
                a, b = v[blk + j], v[blk + j + half]
                v[blk + j] = a + b
                v[blk + j + half] = (a - b) * np.exp(-2j * np.pi * j / (2 * half))
        half //= 2
    return v


def line_fft(x, logm, loge, remlast):
    """One line through the register stages: thread s holds x[s + i*TPL]; the twiddle of stage t
    on butterfly b, output q, is W_M^((b >> logP) * q << logP), as the host table stores it."""
    M, E = 1 << logm, 1 << loge
    tpl = M // E
    sm = x.copy()
    plan = stage_plan(logm, loge, remlast)
    for t, (lr, lp) in enumerate(plan):
        R, P, nb = 1 << lr, 1 << lp, E >> lr
        new = np.zeros(M, complex)
        for s in range(tpl):
            v = [sm[s + i * tpl] for i in range(E)]
            for u in range(nb):
                sub = dif([v[u + j * nb] for j in range(R)])
                for j in range(R):
                    v[u + j * nb] = sub[j]
            for u in range(nb):
                b = s + u * tpl
                for q in range(R):
                    val = v[u + brev(q, lr) * nb]
                    if t < len(plan) - 1:
                        nlo = b >> lp
                        new[(b & (P - 1)) + (q << lp) + (nlo << (lp + lr))] = val * np.exp(-2j * np.pi * ((nlo * q) << lp) / M)
                    else:
                        new[s + (u + q * nb) * tpl] = val   # natural order, k = s + i*TPL
        sm = new
    return sm


@pytest.mark.parametrize("logm,loge", [(5, 3), (6, 4), (7, 4), (9, 4), (10, 4), (10, 5), (11, 4), (8, 5)])
@pytest.mark.parametrize("remlast", [False, True])
def test_both_stage_orders_give_the_transform(logm, loge, remlast):
    rng = np.random.default_rng(logm * 8 + loge)
    x = rng.standard_normal(1 << logm) + 1j * rng.standard_normal(1 << logm)
    y = line_fft(x, logm, loge, remlast)
    assert np.linalg.norm(y - np.fft.fft(x)) <= 1e-12 * np.linalg.norm(x) * logm
