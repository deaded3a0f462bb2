"""Host-side mirror of the launch planner (csrc/capi.cu: tfft_plan_create).

Turns one row of the 11-column kernel-parameter CSV of the reference
(readme.md:46-60; consumed at main.cu:8-32 and fft_codegen.py:745-752) into the
launches the B200 kernels run.  Used by the code generator (which kernels to
instantiate), by the CPU model of the FT decision and by the tests; the C++ planner
applies the same rules.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List

ROLE_SINGLE, ROLE_FIRST, ROLE_LAST = 0, 1, 2
ROLE_NAMES = {ROLE_SINGLE: "single", ROLE_FIRST: "first", ROLE_LAST: "last"}
PARAM_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "param")


@dataclass(frozen=True)
class ParamRow:
    logn: int
    launches: int
    logni: tuple
    bs: tuple
    n: tuple


@dataclass(frozen=True)
class Launch:
    role: int
    logm: int   # log2 of the line length this launch transforms
    loge: int   # log2 points per thread
    logc: int   # log2 lines per tile
    log_b: int = 0   # ROLE_FIRST: log2 of the line stride
    log_n1: int = 0  # ROLE_LAST: log2 extent of the slowest digit
    log_q: int = 0   # ROLE_LAST: log2 extent of the middle digit

    @property
    def threads(self) -> int:
        return (1 << (self.logm - self.loge)) << self.logc

    @property
    def stages(self) -> int:
        return (self.logm + self.loge - 1) // self.loge


def _ilog2(x: int) -> int:
    l = x.bit_length() - 1
    if x < 1 or (1 << l) != x:
        raise ValueError(f"{x} is not a power of two")
    return l


def parse_param_csv(text: str) -> Dict[int, ParamRow]:
    rows: Dict[int, ParamRow] = {}
    for lineno, line in enumerate(text.splitlines(), 1):
        s = line.strip()
        if not s or s.startswith("#"):
            continue
        tok = [int(t) for t in s.split(",")]
        if len(tok) != 11:
            raise ValueError(f"line {lineno}: expected 11 columns, got {len(tok)}")
        rows[tok[0]] = ParamRow(tok[0], tok[1], tuple(tok[2:5]), tuple(tok[5:8]), tuple(tok[8:11]))
    return rows


def load_params(dtype: str, gpu: str = "B200", path: str | None = None) -> Dict[int, ParamRow]:
    path = path or os.path.join(PARAM_DIR, gpu, f"param_{dtype}.csv")
    with open(path) as f:
        return parse_param_csv(f.read())


def load_thread_bs(dtype: str, gpu: str = "B200") -> Dict[int, tuple]:
    """param/<gpu>/thread_bs_<dtype>.csv: logN -> (thread_bs with FT off, with FT on); sizes that are
    not listed use 1.  A plan created with thread_bs = 0 follows this table (the C++ planner reads the
    copy compiled into the library)."""
    path = os.path.join(PARAM_DIR, gpu, f"thread_bs_{dtype}.csv")
    out: Dict[int, tuple] = {}
    if os.path.exists(path):
        for line in open(path):
            s = line.strip()
            if s and not s.startswith("#"):
                tok = [int(t) for t in s.split(",")]
                out[tok[0]] = (tok[1], tok[2])
    return out


def validate_row(r: ParamRow) -> None:
    if not 1 <= r.launches <= 3:
        raise ValueError("launches must be 1..3")
    if sum(r.logni[: r.launches]) != r.logn:
        raise ValueError("logN1+logN2+logN3 != logN")
    for i in range(r.launches):
        if r.logni[i] < 1:
            raise ValueError("logNi must be >= 1")
        _ilog2(r.bs[i])
        if not 1 <= _ilog2(r.n[i]) <= 5:
            raise ValueError("ni must be 2..32")


def launches_of_row(r: ParamRow) -> List[Launch]:
    """The (role, sizes) of every launch of a row; same clamping as the C++ planner."""
    validate_row(r)
    out: List[Launch] = []
    rest = r.logn
    for i in range(r.launches):
        logm = r.logni[i]
        logc = _ilog2(r.bs[i])
        loge = min(_ilog2(r.n[i]), logm)
        rest -= logm
        if r.launches == 1:
            out.append(Launch(ROLE_SINGLE, logm, loge, logc))
        elif i < r.launches - 1:
            out.append(Launch(ROLE_FIRST, logm, loge, min(logc, rest), log_b=rest))
        else:
            log_n1 = r.logni[0]
            log_q = r.logni[1] if r.launches == 3 else 0
            out.append(Launch(ROLE_LAST, logm, loge, min(logc, log_n1), log_n1=log_n1, log_q=log_q))
    return out
