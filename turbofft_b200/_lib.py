"""ctypes binding of libturbofft_b200.so (the C ABI of include/turbofft_b200.h).

The library is the only compute path: if it is missing this module raises, it never
falls back to another FFT.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
# TURBOFFT_B200_LIB selects another build of the same library (the bounds-checked one,
# libturbofft_b200_check.so, for debugging); there is still no fallback if it is missing.
LIB_PATH = os.environ.get("TURBOFFT_B200_LIB") or os.path.join(PKG, "libturbofft_b200.so")

TFFT_OK = 0
STATUS = {
    0: "TFFT_OK", -1: "TFFT_ERR_BAD_ARG", -2: "TFFT_ERR_UNSUPPORTED", -3: "TFFT_ERR_CUDA",
    -4: "TFFT_ERR_PARAM_FILE", -5: "TFFT_ERR_ALLOC", -6: "TFFT_ERR_TOO_LARGE",
}

# name -> (restype, argtypes); every symbol include/turbofft_b200.h declares
SIGNATURES = {
    "tfft_plan_create": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_int,
                                   C.c_char_p, C.c_int]),
    "tfft_plan_create_single_pass": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_int]),
    "tfft_plan_cluster_size": (C.c_int, [C.c_void_p]),
    "tfft_plan_fuse_launches": (C.c_int, [C.c_void_p, C.c_int, C.c_int]),
    "tfft_plan_device_status": (C.c_int, [C.c_void_p, C.POINTER(C.c_int)]),
    "tfft_plan_create_strided": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.c_longlong, C.c_longlong, C.c_int, C.c_int]),
    "tfft_exec": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "tfft_scratch_bytes": (C.c_size_t, [C.c_void_p]),
    "tfft_exec_ws": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "tfft_exec_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "tfft_exec_host_async": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "tfft_host_sync": (C.c_int, [C.c_int]),
    "tfft_workspace_bytes": (C.c_size_t, [C.c_void_p]),
    "tfft_plan_info": (C.c_int, [C.c_void_p, C.POINTER(C.c_int)]),
    "tfft_set_ft_params": (C.c_int, [C.c_void_p, C.c_double, C.c_double, C.c_double]),
    "tfft_set_correction": (C.c_int, [C.c_void_p, C.c_int]),
    "tfft_set_direction": (C.c_int, [C.c_void_p, C.c_int, C.c_double]),
    "tfft_set_injection": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int]),
    "tfft_ft_status": (C.c_int, [C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_int),
                                 C.c_int, C.POINTER(C.c_int)]),
    "tfft_enable_ft_diag": (C.c_int, [C.c_void_p, C.c_int]),
    "tfft_set_ft_accumulate": (C.c_int, [C.c_void_p, C.c_int]),
    "tfft_ft_diag": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_double), C.c_int]),
    "tfft_plan_destroy": (C.c_int, [C.c_void_p]),
    "tfft_bounds_status": (C.c_int, [C.c_void_p, C.POINTER(C.c_longlong), C.POINTER(C.c_int)]),
    "tfft_exec_static": (C.c_int, [C.c_int, C.c_longlong, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "tfft_mg_plan_create": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.c_int,
                                      C.c_int]),
    "tfft_mg_exec": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]),
    "tfft_mg_sync": (C.c_int, [C.c_void_p]),
    "tfft_mg_ft_status": (C.c_int, [C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "tfft_mg_last_cuda_error": (C.c_int, [C.c_void_p]),
    "tfft_mg_destroy": (C.c_int, [C.c_void_p]),
    "tfft_last_cuda_error": (C.c_int, [C.c_void_p]),
    "tfft_status_string": (C.c_char_p, [C.c_int]),
    "tfft_launch_count": (C.c_longlong, []),
    "tfft_stream_copy": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "tfft_transpose": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_longlong, C.c_int, C.c_void_p]),
    "tfft_permute102": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_longlong, C.c_longlong, C.c_int, C.c_void_p]),
    "tfft_scatter_transpose": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_longlong, C.c_longlong, C.c_longlong,
                                        C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "tfft_scatter_transpose_part": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_longlong, C.c_longlong,
                                             C.c_longlong, C.c_longlong, C.c_int, C.c_int, C.c_longlong, C.c_longlong, C.c_int,
                                             C.c_int, C.c_void_p]),
    "tfft_scatter_transpose_ex": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_longlong), C.POINTER(C.c_longlong),
                                           C.c_int, C.c_longlong, C.c_longlong, C.c_longlong, C.c_int, C.c_int, C.c_longlong,
                                           C.c_longlong, C.c_int, C.c_int, C.c_void_p]),
    "tfft_copy_2d": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p]),
    "tfft_peer_alloc": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p)]),
    "tfft_peer_free": (C.c_int, [C.c_void_p]),
    "tfft_peer_export": (C.c_int, [C.c_void_p, C.c_void_p]),
    "tfft_peer_open": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "tfft_peer_close": (C.c_int, [C.c_void_p]),
    "tfft_twiddle_transpose": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_longlong, C.c_longlong,
                                         C.c_longlong, C.c_int, C.c_int, C.c_void_p]),
}

_lib = None


class TurboFFTError(RuntimeError):
    def __init__(self, status: int, where: str, cuda_error: int = 0):
        self.status = status
        self.cuda_error = cuda_error
        msg = f"{where}: {STATUS.get(status, status)}"
        if cuda_error:
            msg += f" (CUDA error {cuda_error})"
        super().__init__(msg)


def lib() -> C.CDLL:
    """Loads the shared library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m turbofft_b200.build` "
                "(there is no fallback path)")
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(l, name)
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


def check(status: int, where: str, plan=None) -> None:
    if status != TFFT_OK:
        cuda = lib().tfft_last_cuda_error(plan) if plan else 0
        raise TurboFFTError(status, where, cuda)
