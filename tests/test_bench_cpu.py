"""bench.py's host-side pieces that need no GPU: the reference arm's JSON line (a reduced workload so that the CPU suite
stays short), the job description shared by both arms, and the recipe that places the reference's modules."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def run_reference_arm(*extra):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "2", "--warmup", "1",
                        "--batch", "2", "--seq", "256", *extra], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    return json.loads(r.stdout.strip().splitlines()[-1])


def test_reference_arm_prints_the_contract_line():
    line = run_reference_arm()
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e", "scaled"):
        assert key in line, key
    assert line["impl"] == "reference" and line["steps"] == 2 and line["warmup"] == 1
    assert line["value"] > 0 and line["ms_per_step"] > 0
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert set(line["config"]) == {"workload", "global_batch", "parallelism", "l2"}
    # one step is one batch element of S tokens: the value follows from the step time as the line says
    if line["scaled"]["seq"] is None:
        assert abs(line["value"] - 256 / (line["ms_per_step"] * 1e-3)) / line["value"] < 1e-6


def test_both_arms_describe_the_job_with_the_same_dictionary():
    import bench
    from multitokenatention_triton_b200.synthetic import WORKLOADS
    a, b = bench.job_config(WORKLOADS["c4"], 1), bench.job_config(WORKLOADS["c4"], 1)
    assert a == b and "B8 H16 S4096 D128" in a["workload"] and a["global_batch"] == 8
    assert bench.job_config(WORKLOADS["c4"], 8)["global_batch"] == 64


def test_make_ref_refuses_a_folder_that_is_not_the_reference(tmp_path):
    from oracle import make_ref
    with pytest.raises(FileNotFoundError):
        make_ref.make_ref(str(tmp_path))
    assert len(make_ref.HOT_PATH_MODULES) == 7
