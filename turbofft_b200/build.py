"""In-tree build of the CUDA libraries for sm_100a.

Mirrors what compile.sh does for the reference (compile.sh:1-11: six generator
passes, then the native build), with nvcc driven directly instead of CMake:
  1. codegen/fft_codegen.py, three passes per datatype (plain, --if_ft 1,
     --if_ft 1 --if_err_injection 1)
  2. every translation unit -> csrc/build/*.o, in parallel
  3. libturbofft_b200.so (the product: kernels + C ABI, no cuFFT),
     libturbofft_cufft_cmp.so (cuFFT timing wrapper, comparison only) and the
     `turbofft` command-line driver.
Objects are rebuilt only when their sources or any header changed.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(PKG, "libturbofft_b200.so")
CMP_LIB = os.path.join(PKG, "libturbofft_cufft_cmp.so")
CLI = os.path.join(PKG, "turbofft")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-std=c++17", "-O3", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-Xcudafe", "--diag_suppress=177",
]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA libraries cannot be built")
    return exe


def run_codegen(verbose: bool = True) -> None:
    gen = os.path.join(PKG, "codegen", "fft_codegen.py")
    for dt in ("float2", "double2"):
        for extra in ([], ["--if_ft", "1"], ["--if_ft", "1", "--if_err_injection", "1"],
                      ["--if_ft", "1", "--if_err_injection", "2"]):
            cmd = [sys.executable, gen, "--gpu", "B200", "--datatype", dt] + extra
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"codegen failed: {' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
            if verbose:
                print(res.stdout.strip())


def _newest_header() -> float:
    hdrs = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        glob.glob(os.path.join(CSRC, "generated", "*.h")) + glob.glob(os.path.join(CSRC, "generated", "*.inc")) + \
        glob.glob(os.path.join(PKG, "..", "include", "*.h"))
    return max(os.path.getmtime(h) for h in hdrs)


CHECK_LIB = os.path.join(PKG, "libturbofft_b200_check.so")
CHECK_FLAGS = ("-DTFFT_BOUNDS_CHECK=1",)


def _compile(src: str, obj: str, extra=()) -> str:
    cmd = [nvcc()] + NVCC_FLAGS + list(extra) + ["-c", src, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{res.stderr}")
    return obj


def _objects(sources, jobs: int, verbose: bool, extra=(), suffix: str = ""):
    os.makedirs(OBJ, exist_ok=True)
    hdr_time = _newest_header()
    todo, objs = [], []
    for src in sources:
        rel = os.path.relpath(src, CSRC).replace(os.sep, "_")
        obj = os.path.join(OBJ, os.path.splitext(rel)[0] + suffix + ".o")
        objs.append(obj)
        if not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_time):
            todo.append((src, obj))
    if verbose and todo:
        print(f"[build] compiling {len(todo)} of {len(sources)} translation units with {jobs} jobs")
    with cf.ThreadPoolExecutor(max_workers=jobs) as ex:
        for f in [ex.submit(_compile, s, o, extra) for s, o in todo]:
            f.result()
    return objs, bool(todo)


def build_all(verbose: bool = True, jobs: int | None = None, with_cli: bool = True) -> str:
    jobs = jobs or max(1, os.cpu_count() or 1)
    run_codegen(verbose)
    gen = sorted(glob.glob(os.path.join(CSRC, "generated", "*", "inst_*.cu")))
    core = [os.path.join(CSRC, f) for f in ("capi.cu", "aux_kernels.cu", "cluster_fft.cu", "pair_fft.cu", "multi_gpu.cu", "registry.cpp", "params.cpp")]
    objs, changed = _objects(core + gen, jobs, verbose)
    if changed or not os.path.exists(LIB):
        cmd = [nvcc(), "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stderr}")
        if verbose:
            print(f"[build] linked {LIB}")
    # the same library with every global index of the data buffers checked (tfft_bounds_status)
    kobjs, kchanged = _objects(core + gen, jobs, verbose, CHECK_FLAGS, "_check")
    if kchanged or not os.path.exists(CHECK_LIB):
        cmd = [nvcc(), "-shared", "-o", CHECK_LIB] + kobjs + ["-gencode", "arch=compute_100a,code=sm_100a"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stderr}")
        if verbose:
            print(f"[build] linked {CHECK_LIB}")
    cmp_src = os.path.join(CSRC, "cufft_compare.cu")
    if os.path.exists(cmp_src):
        cobjs, cchanged = _objects([cmp_src], jobs, verbose)
        if cchanged or not os.path.exists(CMP_LIB):
            cmd = [nvcc(), "-shared", "-o", CMP_LIB] + cobjs + ["-lcufft", "-gencode", "arch=compute_100a,code=sm_100a"]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"link failed:\n{res.stderr}")
    cli_src = os.path.join(CSRC, "turbofft_cli.cu")
    if with_cli and os.path.exists(cli_src):
        mobjs, mchanged = _objects([cli_src], jobs, verbose)
        if mchanged or changed or not os.path.exists(CLI):
            cmd = [nvcc(), "-o", CLI] + mobjs + ["-L" + PKG, "-lturbofft_b200", "-lturbofft_cufft_cmp",
                                                 "-Xlinker", "-rpath=$ORIGIN", "-gencode",
                                                 "arch=compute_100a,code=sm_100a"]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"link failed:\n{res.stderr}")
            if verbose:
                print(f"[build] linked {CLI}")
    return LIB


if __name__ == "__main__":
    build_all()
