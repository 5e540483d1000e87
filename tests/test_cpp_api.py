"""Runs the C++ API test binary (tests/cpp/api_tests.cpp, built by scicompute_attention_b200.build).
Without a GPU the device-level cases skip themselves and only the host-logic cases run; on a GPU
every case must run and pass."""
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "api_tests")


def _run():
    if not os.path.exists(EXE):
        from scicompute_attention_b200 import build
        build.build_all()
    proc = subprocess.run([EXE], capture_output=True, text=True, timeout=900)
    m = re.search(r"SUMMARY passed=(\d+) failed=(\d+) skipped=(\d+)", proc.stdout)
    assert m, proc.stdout[-2000:] + proc.stderr[-2000:]
    return proc, tuple(int(x) for x in m.groups())


def test_host_logic_cases_pass_without_a_gpu():
    proc, (passed, failed, skipped) = _run()
    assert failed == 0 and proc.returncode == 0, proc.stdout[-4000:]
    assert passed >= 8


@pytest.mark.gpu
def test_every_case_runs_and_passes_on_the_gpu():
    proc, (passed, failed, skipped) = _run()
    assert failed == 0 and proc.returncode == 0, "\n".join(l for l in proc.stdout.splitlines() if "FAIL" in l or "SKIP" in l)[-4000:]
    assert skipped == 0 and passed >= 19
