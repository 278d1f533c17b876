"""The benchmark's reference arm runs on the host alone: its one JSON line must carry the contract's keys."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0", "--cpu-len", "256"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["impl"] == "reference" and d["unit"] == "TFLOP/s" and d["value"] > 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in d["config"]


def test_non_zero_ranks_of_the_reference_arm_stay_silent():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                         capture_output=True, text=True, timeout=120, cwd=ROOT, env=env)
    assert res.returncode == 0 and res.stdout.strip() == ""


def test_clock_sampler_keeps_only_the_samples_of_the_timed_region():
    sys.path.insert(0, ROOT)
    import bench
    s = bench.ClockSampler("GPU-none")
    s.rows = [["300", "1965", "Not Active", "Not Active", "Not Active", "Not Active"],       # before the region (idle)
              ["1700", "1965", "Not Active", "Not Active", "Not Active", "Active"],
              ["1720", "1965", "Not Active", "Not Active", "Not Active", "Active"],
              ["210", "1965", "Active", "Not Active", "Not Active", "Not Active"]]            # after it
    s.stamps = [1.0, 2.0, 2.1, 3.0]
    assert s.window(1.5, 2.5) == 2
    out = s.summary()
    assert out["sm_mhz"] == 1710 and out["sm_max_mhz"] == 1965 and out["reasons"] == ["sw_power_cap"] and out["samples"] == 2
    s.rows, s.stamps = [], []
    assert s.summary()["reasons"] == ["unavailable"]
