"""bench.py's contract where it can be checked without a GPU: the reference arm's JSON line, and that both arms
describe the workload with the same `config` object."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_complete_line():
    done = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                           "--warmup", "0", "--workload", "poisson1d"], cwd=ROOT, capture_output=True, text=True,
                          timeout=300)
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [l for l in done.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["scaling"] == "strong" and line["higher_is_better"] is True
    assert line["metric"] == "collocation_points_per_second_per_adam_step" and line["unit"] == "points/s"
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["cpu_baseline"]["value"] == line["value"] == line["e2e"]["value"] > 0
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["config"]["workload"] == "poisson1d" and line["config"]["interior_points"] == 128


def test_both_arms_share_the_config_object():
    sys.path.insert(0, ROOT)
    import bench

    a = bench.workload_config("heat3d", None, 1)
    assert a["workload"] == "heat3d" and a["interior_points"] == 1048576 and a["parameters"] == 330497
    assert bench.workload_config("heat3d", None, 8)["sharding"].startswith("8 contiguous equal axis-0 shard")
    # Nothing arm-specific (engine, streams, timings) lives in `config`.
    assert set(a) == {"workload", "description", "interior_points", "other_sets", "parameters", "optimizer", "sharding"}


def test_rank_other_than_zero_of_the_reference_arm_prints_nothing():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    done = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                           "--steps", "1", "--warmup", "0"], cwd=ROOT, env=env, capture_output=True, text=True,
                          timeout=120)
    assert done.returncode == 0 and done.stdout.strip() == ""
