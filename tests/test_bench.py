"""The benchmark's contract: one JSON line per arm with the agreed keys, the same `config` in both arms, the
reference arm runnable without a GPU, the profile mode a short run of the same forwards."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BENCH = os.path.join(ROOT, "bench.py")


def _run(*args, timeout=600):
    proc = subprocess.run([sys.executable, BENCH, *args], capture_output=True, text=True, timeout=timeout, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [l for l in proc.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, lines           # stdout carries the one JSON line and nothing else
    return json.loads(lines[0])


def test_reference_arm_prints_one_line_on_the_host_cores():
    line = _run("--impl", "reference", "--workload", "c2", "--steps", "1", "--warmup", "1")
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["metric"] == "gla_fwd_tokens_per_s" and line["unit"] == "tokens/s"
    assert line["value"] > 0 and line["vs_baseline"] is None and line["higher_is_better"] is True
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["config"]["workload"].startswith("configs[1]") and line["config"]["T"] == 1600


def test_both_arms_name_the_workload_identically():
    sys.path.insert(0, ROOT)
    import bench
    from gtr_b200 import workloads
    for name, cfg in workloads.CONFIGS.items():
        if name not in bench.WORKLOADS:
            continue
        c = bench.workload_config(name, cfg["B"], cfg["H"], cfg["T"], cfg.get("K", 64))
        assert c["workload"] == bench.WORKLOADS[name] and c["grid"] == list(cfg["grid"]) and "model" not in c


def test_traffic_figure_comes_from_the_committed_profile():
    sys.path.insert(0, ROOT)
    import bench
    with open(os.path.join(ROOT, "profiles", "gla_fwd_kernel.json")) as f:
        want = json.load(f)["c3"]["dram_bytes_per_launch"]
    assert bench.ncu_traffic_bytes("c3") == float(want)
    assert bench.ncu_traffic_bytes("no such workload") is None


@pytest.mark.gpu
def test_profile_mode_runs_the_bench_forwards_and_exits():
    line = _run("--profile-forwards", "2", "--warmup", "1", "--workload", "c2")
    assert line["profile_forwards"] == 2 and line["config"]["T"] == 1600
