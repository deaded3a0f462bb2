"""Shared-memory layout search for the in-block Stockham exchange.

The kernels (csrc/fft_kernels.cuh) place Stockham address a of line c at
    rows layout : c * PITCH + pad(a)         (ROLE_SINGLE, ROLE_LAST)
    cols layout : pad(a) * C + c             (ROLE_FIRST)
with pad(a) = a + (a >> PADSHIFT) and PITCH = pad(M - 1) + 1 + EXTRA.  This module replays
every warp-wide shared-memory access of a kernel instance (stage reads, twiddled scatter
writes, both thread mappings) against the 32 x 4-byte bank model and picks the
(PADSHIFT, EXTRA) with the fewest wavefronts, smallest footprint first among ties.  When the
line length is not a power of the per-thread radix, both stage orders are searched -- remainder
radix in the first stage, or in the last one (REMLAST) -- and the last-stage order wins ties.  The
generator writes the winners to csrc/generated/smem_layouts.h; results are cached in
smem_layouts.json next to this file because the search takes a while in Python.
"""
from __future__ import annotations

import json
import os

CACHE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "smem_layouts.json")
NO_PAD = 31


def _wavefronts(addrs, es_words):
    per = 32 // es_words          # threads served together: 16 for 8-byte, 8 for 16-byte elements
    total = 0
    for ph in range(0, 32, per):
        banks = {}
        for a in addrs[ph:ph + per]:
            for w in range(es_words):
                word = a * es_words + w
                banks.setdefault(word & 31, set()).add(word)
        total += max(len(v) for v in banks.values())
    return total, 32 // per


def simulate(role, logm, loge, logc, fp64, padshift, extra, remlast=False):
    """(wavefronts, ideal wavefronts, elements of shared memory) of one kernel instance."""
    M, E, C = 1 << logm, 1 << loge, 1 << logc
    TPL = M // E
    T = TPL * C
    S = (logm + loge - 1) // loge
    LOGR0 = logm - (S - 1) * loge
    es = 4 if fp64 else 2
    mpad = (M - 1) + ((M - 1) >> padshift) + 1
    pitch = mpad + extra

    def soff(a, c):
        p = a + (a >> padshift)
        return p * C + c if role == 1 else c * pitch + p

    def mapt(tid, cf):
        return (tid // C, tid % C) if cf else (tid % TPL, tid // TPL)

    tot = ideal = 0
    for st in range(S):
        last = st == S - 1
        if remlast:
            LR = LOGR0 if last else loge
            LP = st * loge
        else:
            LR = LOGR0 if st == 0 else loge
            LP = 0 if st == 0 else LOGR0 + (st - 1) * loge
        R, P, NB = 1 << LR, 1 << LP, E >> LR
        cf = (role != 0) if last else (role == 1)
        for w0 in range(0, T, 32):
            tids = list(range(w0, min(w0 + 32, T)))
            sc = [mapt(t, cf) for t in tids]
            if st > 0:
                for i in range(E):
                    ad = [soff(s + i * TPL, c) for s, c in sc]
                    ad += [ad[-1]] * (32 - len(ad))
                    w, idl = _wavefronts(ad, es)
                    tot += w
                    ideal += idl
            if not last:
                for u in range(NB):
                    for q in range(R):
                        ad = []
                        for s, c in sc:
                            b = s + u * TPL
                            ad.append(soff((b & (P - 1)) + (q << LP) + ((b >> LP) << (LP + LR)), c))
                        ad += [ad[-1]] * (32 - len(ad))
                        w, idl = _wavefronts(ad, es)
                        tot += w
                        ideal += idl
    elems = mpad * C if role == 1 else pitch * C
    return tot, ideal, elems


def default_layout(role, logm, loge, logc, fp64):
    """What the kernel header uses when the generator supplies nothing."""
    M = 1 << logm
    tpl = M >> loge
    if role == 1:
        return NO_PAD, 0
    ps = 3 if fp64 else 4
    bankw = 8 if fp64 else 16
    mpad = (M - 1) + ((M - 1) >> ps) + 1
    if role == 2:
        return ps, (mpad | 1) - mpad
    if tpl >= bankw:
        return ps, 0
    return ps, ((mpad + bankw - 1) // bankw) * bankw + tpl - mpad


def _search(role, logm, loge, logc, fp64, remlast):
    best = None
    d = default_layout(role, logm, loge, logc, fp64)
    cands = [d] + [(ps, ex) for ps in (4, 3, 2, 5, 1, 6, NO_PAD) for ex in (range(0, 17) if role != 1 else [0])]
    for ps, ex in cands:
        tot, ideal, elems = simulate(role, logm, loge, logc, fp64, ps, ex, remlast)
        cand = (tot, elems, ps, ex)
        if best is None or cand < best:
            best = cand
        if tot == ideal and elems <= (1 << logm << logc) * 1.07 + 64:
            break
    return best, ideal


def best_layout(role, logm, loge, logc, fp64, cache=None):
    """(PADSHIFT, EXTRA, REMLAST) of one kernel instance."""
    key = f"{int(fp64)}_{role}_{logm}_{loge}_{logc}"
    if cache is not None and key in cache and len(cache[key]) == 3:
        return tuple(cache[key])
    S = (logm + loge - 1) // loge
    if S < 2:
        res = default_layout(role, logm, loge, logc, fp64) + (0,)
    else:
        best, ideal = _search(role, logm, loge, logc, fp64, False)
        res = (best[2], best[3], 0)
        if logm % loge:
            # remainder radix last: never worse in wavefronts where it is chosen, and measured
            # neutral (fp32) to 3 % faster (fp64 sweep) than remainder first
            alt, ideal = _search(role, logm, loge, logc, fp64, True)
            if alt[0] <= best[0]:
                res = (alt[2], alt[3], 1)
    if cache is not None:
        cache[key] = list(res)
    return res


def load_cache():
    if os.path.exists(CACHE):
        with open(CACHE) as f:
            return json.load(f)
    return {}


def save_cache(cache):
    with open(CACHE, "w") as f:
        json.dump(dict(sorted(cache.items())), f, indent=0)
