"""The `turbofft` command-line driver with the reference's flags (CommandLineParser.h:26-110):
the README's verify case and one benchmark line in the reference's print format (main.cu:70)."""
import os
import re
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CLI = os.path.join(ROOT, "turbofft_b200", "turbofft")


def _run(*args):
    if not os.path.exists(CLI):
        pytest.fail(f"{CLI} was not built")
    return subprocess.run([CLI, *args], capture_output=True, text=True, timeout=300)


@pytest.mark.parametrize("datatype", ["0", "1"])
def test_readme_verify_case(torch_cuda, datatype):
    """./turbofft --if_bench 0 --if_verify 1 --logN 10 --bs 16 (readme.md): compares with cuFFT
    by the reference's own 1e-4 test (compareData.h:4-35) and reports no offender."""
    r = _run("--if_bench", "0", "--if_verify", "1", "--logN", "10", "--bs", "16", "--bs_end", "16", "--datatype", datatype)
    assert r.returncode == 0, r.stderr
    assert "Compare begin." in r.stdout and "Compare finished." in r.stdout
    assert "Error detected" not in r.stdout


def test_benchmark_line_format(torch_cuda):
    """--if_profile 1 prints 'turboFFT, logN, logBS, ms, GFLOPS, GB/s' per batch size from --bs to
    --bs_end in steps of --bs_gap, after the cuFFT lines (main.cu:70,104-111)."""
    r = _run("--if_bench", "0", "--if_profile", "1", "--logN", "12", "--bs", "64", "--bs_end", "128", "--bs_gap", "64")
    assert r.returncode == 0, r.stderr
    rows = [ln for ln in r.stdout.splitlines() if ln.startswith("turboFFT,")]
    assert len(rows) == 2
    for ln, logbs in zip(rows, (6, 7)):
        m = re.match(r"turboFFT, (\d+), (\d+),\s*([\d.]+),\s*([\d.]+),\s*([\d.]+)$", ln)
        assert m and int(m.group(1)) == 12 and int(m.group(2)) == logbs and float(m.group(3)) > 0


def test_ft_mode_reports_counts(torch_cuda):
    r = _run("--if_bench", "0", "--if_profile", "1", "--logN", "10", "--bs", "256", "--bs_end", "256", "--if_ft", "1",
             "--if_err", "1", "--thread_bs", "4")
    assert r.returncode == 0, r.stderr
    m = re.search(r"turboFFT_ft, 10, 8, blocks=(\d+), detected=(\d+), corrected=(\d+)", r.stdout)
    assert m and m.group(1) == m.group(2) == m.group(3)


def test_bad_arguments_exit_nonzero(torch_cuda):
    assert _run("--if_bench", "0").returncode != 0            # --logN and --bs are required
    assert _run("--logN").returncode != 0                     # incomplete argument
