"""bench.py's host-side pieces, checked without a GPU: the workload table against the benchmark configurations,
the algorithmic-byte count, the traffic table's scaling rule, the bounded CPU sample, and the reference arm's JSON
line (the reference's own CPU code when it is built, else the C restatement)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bench  # noqa: E402


def test_workloads_are_the_benchmark_configurations():
    cfgs = json.load(open(os.path.join(ROOT, "BASELINE.json")))["configs"]
    assert bench.DEFAULT_WORKLOAD in bench.WORKLOADS and bench.DEFAULT_WORKLOAD in bench.STRONG_SCALING
    rows, hidden, dtype, eps = bench.WORKLOADS[bench.DEFAULT_WORKLOAD]
    assert (rows, hidden, dtype, eps) == (64 * 8192, 8192, "bfloat16", 1e-6)
    assert len(cfgs) >= 5
    # cfg 2, cfg 3a-d and the default are all in the table; cfg 3 takes the wide input distribution
    for name in bench.OTHER_CONFIGS:
        assert name in bench.WORKLOADS
    assert bench.WORKLOADS["rmsnorm_fwd_vjp_fp32_16x2048x4096"] == (32768, 4096, "float32", 1e-5)
    assert {bench.WORKLOADS[n][1] for n in bench.OTHER_CONFIGS if "bf16" in n} == {1000, 5120, 8192, 12288}
    assert all(bench.DISTRIBUTIONS[n] == (3.0, 0.1, 0.01) for n in bench.OTHER_CONFIGS if "bf16" in n)
    assert bench.DEFAULT_WORKLOAD not in bench.DISTRIBUTIONS
    assert bench.STACK_WORKLOADS[bench.OTHER_STACK] == (32, 16384, 4096, 0)


def test_algorithmic_bytes_per_row():
    # forward: read x, write y, rstd; VJP: read x, gy, rstd, write dx
    assert bench.bytes_per_row(4096, 4) == 81928 and bench.bytes_per_row(8192, 2) == 81928
    assert bench.bytes_per_row(1000, 2) == 10008 and bench.bytes_per_row(12288, 2) == 122888


def test_traffic_table_scales_by_rows_only_within_one_width_and_type():
    exact = bench.ncu_traffic(65536, 8192, "bfloat16")
    assert exact and exact["rows"] == 65536
    assert 0.97 < exact["dram_bytes_per_launch"] / exact["algorithmic_bytes_per_launch"] <= 1.0
    big = bench.ncu_traffic(524288, 8192, "bfloat16")
    assert big["dram_bytes_per_launch"] == 8 * exact["dram_bytes_per_launch"] and "scaled x8" in big["source"]
    assert bench.ncu_traffic(524288, 5120, "bfloat16") is None          # no capture of that width: no figure
    assert bench.ncu_traffic(16384, 8192, "bfloat16") is None           # never scaled up from a larger capture
    assert bench.ncu_traffic(32768, 4096, "float32")["rows"] == 32768


def test_cpu_sample_is_bounded():
    assert bench.cpu_sample_rows(524288, 8192) == 2048 and bench.cpu_sample_rows(100, 8192) == 100
    assert bench.cpu_sample_rows(10**9, 1) == 1 << 24


def test_measured_peak_is_the_driver_file_or_the_stated_fallback():
    peak, kind = bench.measured_peak()
    assert (kind == "measured" and peak > 1000) or (kind == "fallback" and peak == bench.FALLBACK_HBM_GBS)


def test_reference_arm_prints_the_contract_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-500:]
    d = json.loads(r.stdout.strip().splitlines()[-1])
    assert d["impl"] == "reference" and d["metric"] == bench.METRIC and d["unit"] == bench.UNIT
    assert d["higher_is_better"] is True and d["value"] > 0 and d["steps"] == 1
    assert d["config"]["workload"] == bench.DEFAULT_WORKLOAD and d["config"]["hidden"] == 8192
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["value"] == d["value"]
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0 and d["e2e"]["value"] == d["value"]
