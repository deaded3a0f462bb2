"""CPU tests of the host logic: parameter files, planner mirror, generator, C ABI surface."""
import ctypes
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

from turbofft_b200 import planner  # noqa: E402


@pytest.mark.parametrize("dt", ["float2", "double2"])
def test_b200_param_tables_are_valid(dt):
    rows = planner.load_params(dt)
    assert rows[0].launches == 0            # row 0 is the all-zero filler, as in the reference CSVs
    for logn in range(1, 31):
        r = rows[logn]
        planner.validate_row(r)
        ls = planner.launches_of_row(r)
        assert len(ls) == r.launches
        assert sum(l.logm for l in ls) == logn
        for l in ls:
            assert 1 <= l.threads <= 1024
            if l.role == planner.ROLE_LAST:
                assert l.stages >= 2 and l.logc <= l.log_n1
            if l.role == planner.ROLE_FIRST:
                assert l.logc <= l.log_b


def test_reference_format_rows_parse():
    # rows in the reference's own format (readme.md:48-60)
    text = "14, 2, 7, 7, 0, 16, 16, 0, 8, 8, 0\n24, 3, 8, 8, 8, 16, 16, 16,  16, 16, 16\n"
    rows = planner.parse_param_csv(text)
    assert rows[14].logni[:2] == (7, 7) and rows[24].launches == 3
    ls = planner.launches_of_row(rows[24])
    assert [l.role for l in ls] == [planner.ROLE_FIRST, planner.ROLE_FIRST, planner.ROLE_LAST]
    assert ls[0].log_b == 16 and ls[1].log_b == 8 and ls[2].log_n1 == 8 and ls[2].log_q == 8


def test_bad_rows_rejected():
    with pytest.raises(ValueError):
        planner.parse_param_csv("1, 2, 3\n")
    rows = planner.parse_param_csv("10, 1, 9, 0, 0, 1, 0, 0, 16, 0, 0\n")
    with pytest.raises(ValueError):
        planner.validate_row(rows[10])       # sizes do not add up
    rows = planner.parse_param_csv("10, 1, 10, 0, 0, 3, 0, 0, 16, 0, 0\n")
    with pytest.raises(ValueError):
        planner.validate_row(rows[10])       # BS not a power of two


def test_codegen_cli_flags(tmp_path):
    """Same flags as the reference generator (fft_codegen.py:709-723)."""
    gen = os.path.join(ROOT, "turbofft_b200", "codegen", "fft_codegen.py")
    out = tmp_path / "gen"
    for extra, mode in ([], 0), (["--if_ft", "1"], 1), (["--if_ft", "1", "--if_err_injection", "1"], 2):
        subprocess.run([sys.executable, gen, "--datatype", "float2", "--gpu", "B200", "--err_inj", "7",
                        "--err_smoothing", "500", "--err_threshold", "0.01", "--out", str(out)] + extra, check=True)
        files = sorted(os.listdir(out / "float2"))
        assert any(f.startswith(f"inst_ft{mode}_p") for f in files)
    text = (out / "ft_defaults.h").read_text()
    assert "TFFT_DEFAULT_ERR_INJ 7.0" in text and "TFFT_DEFAULT_ERR_SMOOTHING 500.0" in text
    assert "TFFT_DEFAULT_ERR_THRESHOLD 0.01" in text
    inst = (out / "float2" / "inst_ft2_p0.cu").read_text()
    assert "TFFT_INST(float, 0," in inst
    assert (out / "default_params_float2.inc").read_text().count("\\n") == 31


def _declared_symbols():
    hdr = open(os.path.join(ROOT, "include", "turbofft_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    return sorted(set(re.findall(r"\b(tfft_[a-z0-9_]+)\s*\(", hdr)))


def test_library_exports_every_declared_symbol():
    from turbofft_b200 import _lib

    lib = _lib.lib()                      # raises if the .so was not built
    names = _declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/turbofft_b200.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"


def test_bad_arguments_fail_before_any_cuda_call():
    from turbofft_b200 import _lib

    lib = _lib.lib()
    h = ctypes.c_void_p()
    assert lib.tfft_plan_create(ctypes.byref(h), 0, 1, 0, 0, 0, 1, None, 0) == -1
    assert lib.tfft_plan_create(ctypes.byref(h), 10, 0, 0, 0, 0, 1, None, 0) == -1
    assert lib.tfft_plan_create(ctypes.byref(h), 10, 1, 7, 0, 0, 1, None, 0) == -1
    assert lib.tfft_plan_create(None, 10, 1, 0, 0, 0, 1, None, 0) == -1
    assert lib.tfft_plan_create(ctypes.byref(h), 10, 1, 0, 0, 0, 1, b"/nonexistent.csv", 0) == -4
    assert lib.tfft_exec(None, None, None, None) == -1
    assert lib.tfft_stream_copy(None, None, 16, None) == -1
    assert lib.tfft_status_string(-2).startswith(b"unsupported")
    assert lib.tfft_launch_count() == 0


def test_no_cpu_fallback_without_gpu():
    """Without a device the product path must fail loudly, not compute elsewhere."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("GPU present")
    import turbofft_b200 as tf

    with pytest.raises(tf.TurboFFTError):
        tf.Plan(10, 16, 0)
    with pytest.raises((ValueError, RuntimeError, tf.TurboFFTError)):
        tf.fft(torch.zeros(4, 16, dtype=torch.complex64))


def test_product_never_imports_oracle():
    """The oracle is test infrastructure: nothing under turbofft_b200/ may use it."""
    pkg = os.path.join(ROOT, "turbofft_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"(import\s+oracle|from\s+oracle|oracle/)", text), os.path.join(dirpath, f)


def test_tuner_candidates_are_plannable():
    """Every row the tuner proposes must pass the planner's checks (so that a compiled
    candidate can never be launched with an impossible geometry)."""
    from turbofft_b200 import tune

    for dt in ("float2", "double2"):
        for logn in (3, 9, 13, 16, 21, 24):
            cands = tune.candidates(logn, dt)
            assert cands, (dt, logn)
            for r in cands:
                planner.validate_row(r)
                for l in planner.launches_of_row(r):
                    assert 32 <= l.threads <= 1024
                    assert l.role != planner.ROLE_LAST or l.stages >= 2
                assert tune.row_text(r).count(",") == 10


def test_tuner_proposes_32_points_per_thread_only_where_it_saves_an_exchange():
    """E = 32 turns lines of 512 and 1024 points into two register stages instead of three;
    for other line lengths of a multi-launch split it saves nothing and is not proposed."""
    from turbofft_b200 import tune

    rows = [r for r in tune.candidates(19, "float2") if r.launches == 2]
    with32 = [r for r in rows if 32 in r.n[:2]]
    assert with32
    for r in with32:
        for logm, n in zip(r.logni[:2], r.n[:2]):
            assert n != 32 or logm in (9, 10), tune.row_text(r)
    assert not [r for r in tune.candidates(19, "double2") if 32 in r.n]   # no registers for it in fp64
    # the shipped fp32 table uses it for 2^13 and for the long lines of 17..21
    shipped = planner.load_params("float2", "B200")
    assert shipped[13].n[0] == 32 and all(32 in shipped[k].n for k in (18, 19, 20))
    for k in (13, 17, 18, 19, 20, 21):
        for l in planner.launches_of_row(shipped[k]):
            if l.loge == 5:
                assert l.stages == 2 or l.logm >= 13


def test_shipped_shared_memory_layouts_are_conflict_free():
    """The generator's bank model on a few shipped instances: the chosen (PADSHIFT, EXTRA)
    reaches the ideal wavefront count, the unpadded layout does not."""
    from turbofft_b200.codegen import smem_layout as sl

    cache = sl.load_cache()
    for key in ("0_0_12_4_0", "0_1_8_4_4", "0_2_8_4_4", "1_0_12_4_0", "0_0_13_5_0", "1_0_10_4_0"):
        assert key in cache, key
        f64, role, logm, loge, logc = (int(t) for t in key.split("_"))
        ps, ex = cache[key][:2]
        rl = bool(cache[key][2]) if len(cache[key]) > 2 else False
        tot, ideal, _ = sl.simulate(role, logm, loge, logc, bool(f64), ps, ex, rl)
        assert tot == ideal, (key, tot, ideal)
    tot, ideal, _ = sl.simulate(0, 12, 4, 0, False, sl.NO_PAD, 0)
    assert tot > ideal


def test_bench_reference_arm_prints_one_json_line():
    import json

    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0",
                          "--cpu-log-sample", "18", "--lo", "7", "--hi", "12"], capture_output=True, text=True, check=True).stdout
    lines = [l for l in out.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "GFLOPS" and d["value"] > 0
    assert d["cpu_baseline"]["kind"] == "port" and d["e2e"]["h2d_bytes_per_step"] == 0
