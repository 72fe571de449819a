"""The benchmark program's host-side contract, checked without a GPU: the reference arm prints one JSON line with
the required keys on the same `config` object the GPU arm uses, and the timing bookkeeping reports medians."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def test_reference_arm_prints_one_line_with_the_contract_keys():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "2",
                          "--warmup", "1"], capture_output=True, text=True, timeout=600, check=True).stdout
    lines = [l for l in out.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["unit"] == "tok/s" and line["steps"] == 2 and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    # the GPU arm builds its `config` with the same function and arguments
    caps = bench.config1_caps(1000)
    assert line["config"] == bench.config1_dict(caps, bench.PREFILL_TOKENS, 1)
    assert line["config"]["kv_slots_per_row"] == sum(caps) == 67328


def test_block_statistics_and_plans_are_deterministic():
    st = bench.block_stats([2.0, 1.0, 4.0, 3.0, 100.0], 10)
    assert st["blocks"] == 5 and st["ms_per_step_median"] == 0.3 and st["ms_per_step_min"] == 0.1
    assert st["ms_per_step_max"] == 10.0 and st["timed_region_ms"] == 110.0
    a = bench.draw_plan(3000, 32, [512, 1024, 2048, 4096], 0.3, 65536)
    assert a == bench.draw_plan(3000, 32, [512, 1024, 2048, 4096], 0.3, 65536)
    assert all(s == 1 for s in a[0]) and min(a[1]) >= 8 and max(a[1]) <= 1024
    assert bench.decode_bytes_of(bench.config1_caps(1000)) == 552075264
