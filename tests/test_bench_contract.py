"""The benchmark's reference arm on the CPU: one JSON line with the contract's keys, and the
same `config` object the GPU arm prints for the same command line."""

import argparse
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.reference
def test_reference_arm_prints_the_contract_line_with_the_gpu_arms_config():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "c1",
                          "--steps", "4", "--warmup", "3"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads([t for t in out.stdout.splitlines() if t.startswith("{")][-1])
    assert line["impl"] == "reference" and line["steps"] == 4 and line["warmup"] == 3
    assert line["metric"] == "param_updates_per_s" and line["unit"] == "param-updates/s"
    assert line["higher_is_better"] is True and line["value"] > 0
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}
    base = line["cpu_baseline"]
    assert base["kind"] in ("reference", "port") and base["cores"] >= 1 and base["value"] == line["value"]
    sys.path.insert(0, str(ROOT))
    import bench

    args = argparse.Namespace(workload="c1", graph=False, apply_gradient=False, in_place_grads=False,
                              no_l2_flush=False, layout="contiguous", frozen_pattern="random")
    w = dict(bench.WORKLOADS["c1"], dtype="f32")
    assert line["config"] == bench.run_config(args, w, 1)


@pytest.mark.gpu
def test_sub_records_of_the_default_line_on_small_cases(cuda):
    """The extra records of the default line, at sizes that take a second: the callbacks'
    one-launch forms and the two forms of `apply_gradient` agree bit for bit inside the record."""
    sys.path.insert(0, str(ROOT))
    import bench

    both = bench.measure_apply_gradient(None, cuda, 6444.1, rows=8)
    assert both["same_bits"] is True
    assert both["scatter_then_step"]["launches_per_call"] == 3 and both["in_place"]["launches_per_call"] == 2
    ticks = bench.measure_callbacks(cuda, n=700)
    assert ticks["early_stopping"]["same_bits"] and ticks["early_stopping"]["launches_per_tick"] == 1
    assert ticks["lr_schedule_warm_restarts"]["same_bits"] and ticks["lr_schedule_warm_restarts"]["launches_per_tick"] == 1
    assert ticks["snapshot"]["launches_per_commit"] == 1 and ticks["snapshot"]["device_to_pinned_gbs"] > 0
