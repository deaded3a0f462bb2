"""CPU FFT used as the timed host baseline.  TEST INFRASTRUCTURE / BASELINE ONLY.

The reference has no CPU implementation of the transform (its kernels are CUDA only and
its own verification compares against cuFFT on the GPU, main.cu:98-102), so the host
baseline is a CPU port of the same operation -- forward unnormalised batched C2C FFT,
include/utils/initializeData.h:31-37 for the sign -- computed by pocketfft through
scipy.fft with every host thread, in the precision of the input.  FFTW is not
installed in this environment.
"""
from __future__ import annotations

import os
import time


def _use_every_core() -> None:
    """The baseline is quoted on all host cores.  Launchers of multi-process jobs narrow them
    (torch.distributed.run exports OMP_NUM_THREADS=1, which pocketfft's pool obeys; some pin the
    process), so before scipy.fft loads: widen the affinity mask to every CPU of the box and lift
    a thread cap that is lower than that."""
    n = os.cpu_count() or 1
    try:
        os.sched_setaffinity(0, range(n))
    except (AttributeError, OSError):
        pass
    for key in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        try:
            if int(os.environ.get(key, n)) < n:
                os.environ[key] = str(n)
        except ValueError:
            os.environ[key] = str(n)


_use_every_core()

import numpy as np  # noqa: E402
import scipy.fft  # noqa: E402


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def thread_speedup(log_elems: int = 22) -> float:
    """How much faster the transform runs with every host thread than with one, measured: the
    figure printed beside the thread count, so that a capped pool cannot pass for a full one."""
    rng = np.random.default_rng(0)
    x = rng.uniform(-1, 1, size=(1 << (log_elems - 10), 1 << 11)).astype(np.float32).view(np.complex64)
    best = {}
    for w in (1, host_threads()):
        scipy.fft.fft(x, axis=-1, workers=w)
        t = []
        for _ in range(3):
            t0 = time.perf_counter()
            scipy.fft.fft(x, axis=-1, workers=w)
            t.append(time.perf_counter() - t0)
        best[w] = min(t)
    return best[1] / best[host_threads()]


def cpu_fft(x: np.ndarray, workers: int | None = None) -> np.ndarray:
    return scipy.fft.fft(x, axis=-1, workers=workers or host_threads())
