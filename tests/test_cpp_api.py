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


ROLLOUT = os.path.join(ROOT, "examples", "rollout_engine")


def test_rollout_example_reports_a_missing_gpu_instead_of_crashing():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    if not os.path.exists(ROLLOUT):
        from scicompute_attention_b200 import build
        build.build_all()
    proc = subprocess.run([ROLLOUT, "--requests", "2"], capture_output=True, text=True, timeout=120)
    assert proc.returncode == 2 and "no CUDA device" in proc.stdout


@pytest.mark.gpu
def test_rollout_example_serves_and_its_two_decode_backends_agree():
    """Prefill through flash on token-major views, paged caches per layer, batched appends, paged decode; the
    last step is recomputed by the split-K backend on the gathered cache (--verify)."""
    if not os.path.exists(ROLLOUT):
        from scicompute_attention_b200 import build
        build.build_all()
    proc = subprocess.run([ROLLOUT, "--requests", "12", "--layers", "2", "--new-tokens", "5", "--prompt-min", "17",
                           "--prompt-max", "300", "--verify"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-2000:]
    assert "verify: paged vs contiguous decode" in proc.stdout and "generated tokens/s" in proc.stdout
    # follow-up prompts: one chunked-prefill launch per layer over the paged cache, checked against flash on the gathered cache
    assert "verify: chunked prefill over the paged cache vs flash" in proc.stdout and "follow-up:" in proc.stdout


@pytest.mark.gpu
def test_rollout_example_on_every_visible_gpu():
    """--gpus G: one copy per GPU on its own requests and caches (no collective); the parent adds up the rates."""
    import torch
    gpus = torch.cuda.device_count()
    if gpus < 2:
        pytest.skip("needs at least 2 GPUs")
    proc = subprocess.run([ROLLOUT, "--gpus", str(gpus), "--requests", "8", "--layers", "2", "--new-tokens", "4",
                           "--prompt-min", "33", "--prompt-max", "200", "--followup", "40", "--verify"],
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-2000:]
    assert f"{gpus} GPUs together" in proc.stdout
    assert proc.stdout.count("verify: paged vs contiguous decode") == gpus


@pytest.mark.gpu
def test_api_level_benchmark_writes_the_reference_record_format(tmp_path):
    """examples/bench_attention times one public API call per sample and writes the JSON / CSV records of the
    reference's benchmark suite (benchmarks/common/bench_utils.hpp:261-330): same keys, same CSV header."""
    import json
    exe = os.path.join(ROOT, "examples", "bench_attention")
    if not os.path.exists(exe):
        from scicompute_attention_b200 import build
        build.build_all()
    proc = subprocess.run([exe, "--small", "--runs", "10", "--warmup", "3", "--out-dir", str(tmp_path)],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-2000:]
    record = json.load(open(tmp_path / "bench_attention.json"))
    for key in ("benchmark_name", "git_sha", "build_type", "gpu", "compute_cap", "driver", "cuda", "sm_clock_mhz",
                "timestamp", "warmup", "runs", "seed", "cases"):
        assert key in record, key
    assert record["runs"] == 10 and len(record["cases"]) == 4
    for case in record["cases"]:
        for key in ("case_id", "impl", "params", "latency_ms", "flops_effective", "tflops", "bytes_moved_modeled",
                    "effective_bw_gbps", "peak_mem_mb", "workspace_mb", "registers_per_thread", "smem_bytes",
                    "achieved_occupancy_pct", "reference_max_abs_err", "note"):
            assert key in case, key
        lat = case["latency_ms"]
        assert set(lat) == {"mean", "median", "std", "p50", "p90", "p95", "p99"}
        assert 0 < lat["p50"] <= lat["p90"] <= lat["p99"]
    header = open(tmp_path / "bench_attention.csv").readline().strip()
    assert header == ("name,case_id,warmup,runs,mean_ms,median_ms,std_ms,p50_ms,p90_ms,p95_ms,p99_ms,tflops,"
                      "effective_bw_gbps,peak_mem_mb,unit")
