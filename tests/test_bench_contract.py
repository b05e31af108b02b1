"""The benchmark's reference arm runs without a GPU (it times the CPU oracle): check the JSON line it prints
against the fields the measurement contract names, and that the product arm refuses to run without CUDA
instead of falling back to the CPU."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, env=None):
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=300,
                          cwd=ROOT, env=e)


def test_reference_arm_prints_one_contract_line():
    r = _run("--impl", "reference", "--workload", "tiny", "--steps", "2", "--warmup", "1")
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    j = json.loads(lines[0])
    assert j["impl"] == "reference" and j["metric"] == "decode_tokens_per_s" and j["unit"] == "tokens/s"
    assert j["n_gpus"] == 1 and j["steps"] == 2 and j["warmup"] == 1 and j["higher_is_better"] is True
    assert j["value"] > 0 and j["ms_per_step"] > 0 and j["vs_baseline"] is None and j["data"] == "synthetic"
    assert j["config"]["workload"] == "tiny"
    cb = j["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == j["value"] and cb["sample"]
    e2e = j["e2e"]
    assert e2e["value"] == j["value"] and e2e["unit"] == j["unit"]
    assert e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0


def test_reference_arm_under_torchrun_env_only_rank0_prints():
    r = _run("--impl", "reference", "--workload", "tiny", "--steps", "1", "--warmup", "1", "--gpus", "2",
             env={"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2"})
    assert r.returncode == 0, r.stderr[-2000:]
    assert not [l for l in r.stdout.splitlines() if l.startswith("{")]


def test_product_arm_fails_loudly_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        import pytest
        pytest.skip("a GPU is present")
    r = _run("--workload", "tiny", "--steps", "1", "--warmup", "1", "--no-cpu-baseline")
    assert r.returncode != 0
    assert not [l for l in r.stdout.splitlines() if l.startswith("{")]


def test_reference_arm_ignores_an_inherited_single_thread_setting():
    """torch.distributed.run exports OMP_NUM_THREADS=1 for every rank; the CPU arm sets its own thread count."""
    r = _run("--impl", "reference", "--workload", "tiny", "--steps", "1", "--warmup", "1", env={"OMP_NUM_THREADS": "1"})
    assert r.returncode == 0, r.stderr[-2000:]
    j = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][0])
    assert j["cpu_baseline"]["cores"] == (os.cpu_count() or 1)
    # same config keys as the product arm prints for this workload
    assert set(j["config"]) == {"workload", "batch_per_gpu", "prompt", "decode_steps", "parallelism", "sampling", "mask", "norm", "l2"}


def test_clock_record_counts_only_samples_inside_the_timed_region():
    """The sampler runs from before the warm-up; a sample counts when its timestamp lies in the timed region, and a
    region too short for two samples widens to the warm-up steps and says so."""
    import datetime
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_mod", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    base = datetime.datetime(2025, 1, 2, 3, 4, 5).timestamp()

    def row(dt, mhz, watts, cap):
        ts = datetime.datetime.fromtimestamp(base + dt).strftime("%Y/%m/%d %H:%M:%S.%f")[:-3]
        return "%s, %d, 1965, %.2f, 0x4, Not Active, Not Active, Not Active, %s, 1000.00" % (ts, mhz, watts, cap)

    text = "\n".join([row(0.00, 1400, 950.0, "Active"), row(0.10, 1410, 500.0, "Active"),     # right after the prefill
                      row(0.30, 1950, 600.0, "Not Active"), row(0.32, 1960, 610.0, "Not Active"), row(0.34, 1965, 620.0, "Not Active"),
                      row(0.50, 210, 90.0, "Not Active"), "garbage line"])
    rec = bench.ClockSampler.summarise(text, base + 0.05, base + 0.29, base + 0.35)
    assert rec["samples"] == 3 and rec["window"] == "timed region"
    assert rec["sm_mhz"] == 1960.0 and rec["sm_max_mhz"] == 1965.0 and rec["reasons"] == []
    assert rec["power_w"] == 610.0 and rec["power_limit_w"] == 1000.0
    short = bench.ClockSampler.summarise(text, base + 0.05, base + 0.31, base + 0.33)
    assert short["samples"] == 3 and short["window"].startswith("warm-up + timed region") and short["reasons"] == ["sw_power_cap"]
