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

import numpy as np
import scipy.fft


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_fft(x: np.ndarray, workers: int | None = None) -> np.ndarray:
    return scipy.fft.fft(x, axis=-1, workers=workers or host_threads())
