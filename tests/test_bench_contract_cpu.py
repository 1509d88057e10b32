"""The reference arm of bench.py runs without a GPU and prints one JSON line with the agreed keys."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "decode_attention_host_kv_gbps" and d["unit"] == "GB/s"
    assert d["higher_is_better"] is True and d["value"] > 0 and d["gpu_launches"] == 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in d["config"] and "parallelism" in d["config"]
    assert d["steps"] == 1 and "all 16 requests" in d["cpu_baseline"]["sample"]


def test_reference_arm_other_ranks_exit_quietly():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                         capture_output=True, text=True, timeout=120, cwd=ROOT, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_longctx_csv_has_the_reference_columns(tmp_path):
    """benchmarks/bench_offload_longctx.py:65-71 in the reference."""
    import csv
    import importlib.util

    spec = importlib.util.spec_from_file_location("bench_mod", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    assert bench.LONGCTX_CSV_HEADER == [
        "system", "model", "seq_length", "mean_latency_s", "p50_latency_s", "p90_latency_s", "p99_latency_s",
        "mean_e2e_latency_s", "p50_e2e_latency_s", "p90_e2e_latency_s", "p99_e2e_latency_s", "gpu_memory_peak_mb",
        "memory_saving_pct", "throughput_tps"]
    path = tmp_path / "fig11.csv"
    bench.write_longctx_csv(str(path), [{"system": "s", "model": "m", "seq_length": 32768, "mean_latency_s": 0.085}])
    bench.write_longctx_csv(str(path), [{"system": "s", "model": "m", "seq_length": 131072, "mean_latency_s": 0.334}])
    rows = list(csv.DictReader(open(path)))
    assert [r["seq_length"] for r in rows] == ["32768", "131072"] and rows[0]["p99_e2e_latency_s"] == ""
    assert bench._pct([5, 1, 3], 0.5) == 3 and bench._pct([1.0], 0.99) == 1.0
