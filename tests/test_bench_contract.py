"""CPU test of the benchmark's reference arm: `bench.py --impl reference` needs
no GPU, so the shape of its JSON line can be checked anywhere."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


@pytest.mark.parametrize("workload", ["dgemm4096", "sgemm1024", "ssyrk16384", "mvt32768", "chain2mm"])
def test_reference_arm_prints_one_contract_line(workload):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                        "--workload", workload, "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and "unavailable" not in d
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step",
                "higher_is_better", "scaling", "vs_baseline", "dtype", "data", "config", "e2e",
                "cpu_baseline"):
        assert key in d, key
    assert d["steps"] == 1 and d["warmup"] == 0 and d["n_gpus"] == 1
    assert d["higher_is_better"] is True and d["vs_baseline"] is None and d["data"] == "synthetic"
    assert d["value"] > 0 and d["ms_per_step"] > 0
    assert "workload" in d["config"] and "model" not in d["config"]
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["sample"]
    assert cb["value"] == d["value"] and cb["unit"] == d["unit"]
    e = d["e2e"]
    assert e["value"] == d["value"] and e["unit"] == d["unit"]
    assert e["h2d_bytes_per_step"] == 0 and e["d2h_bytes_per_step"] == 0
    assert d["unit"] == ("GB/s" if workload.startswith("mvt") else "GFLOP/s")


def _bench_module():
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    return bench


def test_default_workload_is_the_largest_single_gpu_config_and_steps_are_honoured():
    """No --workload: configs[4]b (fp32 GEMM 32768^3), strong scaling; the
    reference arm runs exactly the steps it is asked for and prints the same
    `config` object as the GPU arm for the same --gpus."""
    bench = _bench_module()
    assert bench.DEFAULT_WORKLOAD == "sgemm32768"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                        "--gpus", "2", "--steps", "7", "--warmup", "1"],
                       capture_output=True, text=True, cwd=ROOT, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    d = json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("{")][0])
    assert d["steps"] == 7 and d["warmup"] == 1 and d["n_gpus"] == 2 and d["scaling"] == "strong"
    assert d["config"] == bench.config_of("sgemm32768", bench.WORKLOADS["sgemm32768"], 2)
    assert "configs[4]b" in d["config"]["workload"] and d["dtype"] == "f32"


def test_trimmed_mean_protocol():
    """5 runs, fastest and slowest dropped, mean of the middle three and their
    largest deviation from it (the reference's time_benchmark.sh)."""
    bench = _bench_module()
    mean, dev = bench.trimmed([5.0, 1.0, 2.0, 3.0, 100.0])
    assert mean == pytest.approx(10.0 / 3.0) and dev == pytest.approx((5.0 - 10.0 / 3.0) / (10.0 / 3.0) * 100)
    labels = [c for c, _ in bench.PER_CONFIG]
    assert labels == ["configs[0]", "configs[1]", "configs[2]", "configs[3]", "configs[4]a", "configs[4]b"]


def test_workload_tables():
    """Algorithmic units and operand sizes the roofline arithmetic rests on."""
    bench = _bench_module()
    w = bench.WORKLOADS
    assert bench.algorithmic_work("dgemm4096", w["dgemm4096"]) == 2 * 4096 ** 3
    assert bench.algorithmic_work("sgemm32768", w["sgemm32768"]) == 2 * 32768 ** 3
    assert bench.algorithmic_work("ssyrk16384", w["ssyrk16384"]) == 16384 * 16385 * 8192
    assert bench.algorithmic_work("mvt32768", w["mvt32768"]) == 32768 * 32768 * 8 + 6 * 32768 * 8
    assert bench.algorithmic_work("chain2mm", w["chain2mm"]) == \
        2 * 4096 * 5120 * 6144 + 2 * 4096 * 8192 * 5120
    assert bench.operand_bytes("dgemm4096", w["dgemm4096"]) == 3 * 4096 * 4096 * 8
    # only the workloads below twice the L2 size take the flushed, step-by-step timing
    small = sorted(n for n in w if bench.operand_bytes(n, w[n]) < 2 * bench.L2_BYTES)
    assert small == ["sgemm1024", "sgemm4096"]
    for name in w:
        metric, unit, scale = bench.metric_of(name)
        assert unit == ("GB/s" if name.startswith("mvt") else "GFLOP/s") and scale == 1e9
