"""turbofft_b200: batched power-of-two C2C FFT with fused ABFT for B200 (sm_100a).

Python face of the C ABI (include/turbofft_b200.h).  `Plan` mirrors the launch
protocol of the reference's test_turbofft() (main.cu:4-73) with the CLI's flag names
(--logN, --bs as `batch`, --datatype, --if_ft, --if_err, --thread_bs;
include/utils/CommandLineParser.h:47-79); `fft` is the torch-style entry point for
complex64 / complex128 CUDA tensors.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

from . import _lib
from ._lib import TurboFFTError, lib

__all__ = ["Plan", "fft", "ifft", "TurboFFTError", "lib", "stream_copy", "launch_count", "host_sync"]

FLOAT2, DOUBLE2 = 0, 1


def _torch():
    import torch

    return torch


def _dtype_code(t) -> int:
    torch = _torch()
    if t == torch.complex64:
        return FLOAT2
    if t == torch.complex128:
        return DOUBLE2
    raise TypeError(f"turbofft_b200 supports complex64 and complex128, got {t}")


class Plan:
    """One (logN, batch, dtype, FT mode) plan on one device."""

    def __init__(self, logN: int, batch: int, dtype: int = FLOAT2, if_ft: int = 0, if_err: int = 0,
                 thread_bs: int = 1, param_csv: Optional[str] = None, device: int = 0,
                 single_pass: Optional[int] = None):
        """single_pass = g asks for the one-kernel cluster plan with 2^g CTAs per cluster (-1 = the
        size's default); None lets tfft_plan_create choose (built-in tables)."""
        self._h = C.c_void_p()
        self.logN, self.batch, self.dtype = int(logN), int(batch), int(dtype)
        self.if_ft, self.if_err, self.thread_bs, self.device = int(bool(if_ft or if_err)), int(if_err), int(thread_bs), int(device)
        if single_pass is not None:
            rc = lib().tfft_plan_create_single_pass(C.byref(self._h), self.logN, self.batch, self.dtype, int(single_pass),
                                                    self.thread_bs, self.device)
            _lib.check(rc, f"tfft_plan_create_single_pass(logN={logN}, batch={batch}, dtype={dtype}, log_cluster={single_pass})")
            return
        rc = lib().tfft_plan_create(C.byref(self._h), self.logN, self.batch, self.dtype, int(if_ft), int(if_err),
                                    self.thread_bs, param_csv.encode() if param_csv else None, self.device)
        _lib.check(rc, f"tfft_plan_create(logN={logN}, batch={batch}, dtype={dtype}, ft={if_ft}, err={if_err})")

    def fuse_launches(self, log_chunk_signals: int, lag: int = 1) -> None:
        """Run both launches of a two-launch plan as one persistent kernel whose intermediate stays in
        L2 (tfft_plan_fuse_launches); raises if the plan or the device does not allow it."""
        _lib.check(lib().tfft_plan_fuse_launches(self._h, int(log_chunk_signals), int(lag)), "tfft_plan_fuse_launches", self._h)

    def device_status(self) -> int:
        """1 if a bounded device-side wait of this plan's kernel ever gave up, else 0 (synchronises)."""
        st = C.c_int(0)
        _lib.check(lib().tfft_plan_device_status(self._h, C.byref(st)), "tfft_plan_device_status", self._h)
        return st.value

    @property
    def cluster_size(self) -> int:
        """CTAs per cluster of a single-pass plan, 0 for a plan made of ordinary launches."""
        return lib().tfft_plan_cluster_size(self._h)

    # -- execution
    def exec_ptr(self, in_ptr: int, out_ptr: int, stream: int = 0) -> None:
        _lib.check(lib().tfft_exec(self._h, in_ptr, out_ptr, stream), "tfft_exec", self._h)

    def exec_host_ptr(self, in_ptr: int, out_ptr: int, stream: int = 0) -> None:
        _lib.check(lib().tfft_exec_host(self._h, in_ptr, out_ptr, stream), "tfft_exec_host", self._h)

    def exec_host_async_ptr(self, in_ptr: int, out_ptr: int, stream: int = 0) -> None:
        """tfft_exec_host without the final synchronisation: results are complete after host_sync(device)."""
        _lib.check(lib().tfft_exec_host_async(self._h, in_ptr, out_ptr, stream), "tfft_exec_host_async", self._h)

    def __call__(self, x, out=None):
        """x: CUDA tensor [batch, N] (or [N] when batch == 1) of the plan's dtype."""
        torch = _torch()
        if not x.is_cuda:
            raise ValueError("input must be a CUDA tensor (use exec_host for host buffers)")
        if _dtype_code(x.dtype) != self.dtype or x.numel() != self.batch << self.logN:
            raise ValueError("tensor does not match the plan")
        if x.device.index != self.device:
            raise ValueError("tensor is on another device than the plan")
        x = x.contiguous()
        if out is None:
            out = torch.empty_like(x)
        elif not (out.is_cuda and out.is_contiguous() and out.dtype == x.dtype and out.numel() == x.numel()):
            raise ValueError("bad output tensor")
        stream = torch.cuda.current_stream(x.device).cuda_stream
        self.exec_ptr(x.data_ptr(), out.data_ptr(), stream)
        return out

    def exec_host(self, x, out=None):
        """x: CPU tensor (pinned for full speed); returns a CPU tensor.  Synchronous."""
        torch = _torch()
        if x.is_cuda or _dtype_code(x.dtype) != self.dtype or x.numel() != self.batch << self.logN:
            raise ValueError("tensor does not match the plan")
        x = x.contiguous()
        if out is None:
            out = torch.empty_like(x, pin_memory=x.is_pinned())
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream().cuda_stream
            self.exec_host_ptr(x.data_ptr(), out.data_ptr(), stream)
        return out

    def exec_host_async(self, x, out):
        """exec_host without the final synchronisation, for a sequence of transforms whose chunks should keep
        the copy pipeline full: x and out (CPU tensors, pinned) must stay alive and untouched until
        turbofft_b200.host_sync(device) has returned."""
        torch = _torch()
        if x.is_cuda or out.is_cuda or _dtype_code(x.dtype) != self.dtype or x.numel() != self.batch << self.logN \
                or out.dtype != x.dtype or out.numel() != x.numel() or not (x.is_contiguous() and out.is_contiguous()):
            raise ValueError("tensors do not match the plan")
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream().cuda_stream
            self.exec_host_async_ptr(x.data_ptr(), out.data_ptr(), stream)
        return out

    # -- introspection
    def info(self):
        buf = (C.c_int * 19)()
        _lib.check(lib().tfft_plan_info(self._h, buf), "tfft_plan_info", self._h)
        keys = ("logNi", "lines_per_tile", "points_per_thread", "grid", "threads", "smem_bytes")
        return [dict(zip(keys, buf[1 + 6 * i: 7 + 6 * i])) for i in range(buf[0])]

    @property
    def workspace_bytes(self) -> int:
        return int(lib().tfft_workspace_bytes(self._h))

    def set_correction(self, from_checksums: bool = True):
        """Repair located tiles from the running checksums (no recompute; allows 1-launch in place)."""
        _lib.check(lib().tfft_set_correction(self._h, int(from_checksums)), "tfft_set_correction", self._h)

    def set_direction(self, inverse: bool = False, scale: float = 1.0):
        """inverse: scale * conj(F(conj(x))) (the inverse DFT for scale = 1/N); else scale * F(x)."""
        _lib.check(lib().tfft_set_direction(self._h, int(inverse), float(scale)), "tfft_set_direction")

    # -- fault tolerance
    def set_ft_params(self, err_inj: float = 100.0, err_smoothing: float = 1000.0, err_threshold: float = 1e-3):
        _lib.check(lib().tfft_set_ft_params(self._h, err_inj, err_smoothing, err_threshold), "tfft_set_ft_params")

    def set_injection(self, enable: bool = True, launch: int = -1, period: int = 1, phase: int = 0):
        _lib.check(lib().tfft_set_injection(self._h, int(enable), launch, period, phase), "tfft_set_injection")

    def set_ft_accumulate(self, enable: bool = True):
        """FT counters add up over calls until ft_status() reads (and clears) them."""
        _lib.check(lib().tfft_set_ft_accumulate(self._h, int(enable)), "tfft_set_ft_accumulate")

    def enable_ft_diag(self, enable: bool = True):
        _lib.check(lib().tfft_enable_ft_diag(self._h, int(enable)), "tfft_enable_ft_diag")

    def ft_status(self, launch: int = -1):
        """(n_detected, n_corrected, located[list per block of `launch`])."""
        nd, nc, nb = C.c_int(), C.c_int(), C.c_int()
        _lib.check(lib().tfft_ft_status(self._h, C.byref(nd), C.byref(nc), launch, None, 0, C.byref(nb)),
                   "tfft_ft_status", self._h)
        loc = (C.c_int * max(nb.value, 1))()
        _lib.check(lib().tfft_ft_status(self._h, C.byref(nd), C.byref(nc), launch, loc, nb.value, C.byref(nb)),
                   "tfft_ft_status", self._h)
        return nd.value, nc.value, list(loc[: nb.value])

    def ft_diag(self, launch: int = -1):
        """Per block (delta, S, delta_w) of `launch`; needs enable_ft_diag() before exec."""
        _, _, loc = self.ft_status(launch)
        buf = (C.c_double * (3 * max(len(loc), 1)))()
        _lib.check(lib().tfft_ft_diag(self._h, launch, buf, len(loc)), "tfft_ft_diag", self._h)
        return [(buf[3 * i], buf[3 * i + 1], buf[3 * i + 2]) for i in range(len(loc))]

    def destroy(self):
        if self._h:
            lib().tfft_plan_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


_plan_cache = {}


_NORM_FWD = {None: 0.0, "backward": 0.0, "ortho": -0.5, "forward": -1.0}  # exponent of N in the forward scale


def _fft_strided(x, dim: int, norm, inverse: bool):
    """Transform along a middle axis of a contiguous tensor: [outer][N][inner], lines strided by inner."""
    torch = _torch()
    x = x.contiguous()
    n = x.shape[dim]
    logn = n.bit_length() - 1
    inner = 1
    for s in x.shape[dim + 1:]:
        inner *= s
    outer = x.numel() // (n * inner)
    if n < 2 or (1 << logn) != n or inner & (inner - 1):
        raise ValueError("the transformed axis and the product of the axes behind it must be powers of two")
    expo = _NORM_FWD[norm] if not inverse else -1.0 - _NORM_FWD[norm]
    key = ("strided", x.device.index, logn, inner, outer, _dtype_code(x.dtype), bool(inverse), expo)
    plan = _plan_cache.get(key)
    if plan is None:
        plan = Plan.__new__(Plan)
        plan._h = C.c_void_p()
        plan.logN, plan.batch, plan.dtype, plan.device = logn, outer * inner, _dtype_code(x.dtype), x.device.index
        plan.if_ft = plan.if_err = 0
        plan.thread_bs = 1
        _lib.check(lib().tfft_plan_create_strided(C.byref(plan._h), logn, inner, outer, plan.dtype, plan.device),
                   f"tfft_plan_create_strided(logN={logn}, inner={inner}, outer={outer})")
        plan.set_direction(inverse, float(n) ** expo)
        _plan_cache[key] = plan
    y = torch.empty_like(x)
    plan.exec_ptr(x.data_ptr(), y.data_ptr(), torch.cuda.current_stream(x.device).cuda_stream)
    return y


def fft(x, ft: bool = False, err: bool = False, thread_bs: int = 1, out=None, norm=None, inverse: bool = False, dim: int = -1):
    """FFT along one axis of a complex64/complex128 CUDA tensor (forward, unnormalised by
    default, which is the reference's transform).

    Power-of-two lengths 2..2^30 along the last axis; leading axes are the batch.  ft/err are
    the reference's --if_ft / --if_err.  norm follows torch.fft ("backward", "ortho", "forward");
    inverse=True is what ifft() calls.  dim other than the last axis runs the strided-batch plan
    (no copy, no transpose; lengths with a compiled strided-line kernel, FT off).  Plans are
    cached per (device, shape, mode).
    """
    if not x.is_cuda:
        raise ValueError("turbofft_b200.fft needs a CUDA tensor: there is no CPU path")
    if norm not in _NORM_FWD:
        raise ValueError(f"unknown norm {norm!r}")
    dim = dim % x.dim()
    if dim != x.dim() - 1:
        if ft or err or out is not None:
            raise ValueError("the strided-batch plan has no FT mode and allocates its output")
        return _fft_strided(x, dim, norm, inverse)
    n = x.shape[-1]
    logn = n.bit_length() - 1
    if n < 2 or (1 << logn) != n:
        raise ValueError("last axis must be a power of two >= 2")
    batch = x.numel() // n
    if norm not in _NORM_FWD:
        raise ValueError(f"unknown norm {norm!r}")
    expo = _NORM_FWD[norm] if not inverse else -1.0 - _NORM_FWD[norm]
    key = (x.device.index, logn, batch, _dtype_code(x.dtype), bool(ft), bool(err), thread_bs, bool(inverse), expo)
    plan = _plan_cache.get(key)
    if plan is None:
        plan = Plan(logn, batch, _dtype_code(x.dtype), int(ft or err), int(err), thread_bs, device=x.device.index)
        plan.set_direction(inverse, float(n) ** expo)
        _plan_cache[key] = plan
    y = plan(x.reshape(batch, n), out=None if out is None else out.reshape(batch, n))
    return y.reshape(x.shape)


def ifft(x, ft: bool = False, err: bool = False, thread_bs: int = 1, out=None, norm=None, dim: int = -1):
    """Inverse FFT along one axis (1/N scaling by default, as torch.fft.ifft)."""
    return fft(x, ft=ft, err=err, thread_bs=thread_bs, out=out, norm=norm, inverse=True, dim=dim)


def fft2(x, norm=None, inverse: bool = False):
    """2-D transform over the last two axes: the strided-batch plan along the rows' axis, then the
    ordinary plan along the last axis (both lengths powers of two)."""
    return fft(fft(x, dim=-2, norm=norm, inverse=inverse), norm=norm, inverse=inverse)


def host_sync(device: int = 0) -> None:
    """Waits for every chunk queued by Plan.exec_host_async_ptr on this device (tfft_host_sync)."""
    _lib.check(lib().tfft_host_sync(int(device)), "tfft_host_sync")


def stream_copy(src, dst) -> None:
    """STREAM-style device copy (128-bit accesses) used as the measured HBM peak."""
    torch = _torch()
    nbytes = src.numel() * src.element_size()
    stream = torch.cuda.current_stream(src.device).cuda_stream
    _lib.check(lib().tfft_stream_copy(src.data_ptr(), dst.data_ptr(), nbytes, stream), "tfft_stream_copy")


def launch_count() -> int:
    return int(lib().tfft_launch_count())
