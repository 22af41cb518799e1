"""CPU tests of the benchmark's bookkeeping: the algorithmic-byte formula, the peak and traffic tables, the
workload table, and the reference arm's behaviour on ranks other than 0 and on the smallest workload."""
import json
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_algorithmic_bytes_per_query():
    import bench
    assert bench.algorithmic_bytes_per_query(8, 16, 1, 2) == 1312          # q, k, v, out + offsets + attn_out, float16
    assert bench.algorithmic_bytes_per_query(8, 16, 1, 4) == 2624
    assert bench.algorithmic_bytes_per_query(8, 16, 1, 2, with_attn=False) == 2 * (4 * 128 + 16)
    assert bench.algorithmic_bytes_per_query(4, 32, 2, 2) == 2 * (4 * 128 + 8 + 4 * 36)


def test_workload_table_is_consistent():
    import bench
    assert bench.DEFAULT_WORKLOAD in bench.WORKLOADS
    for name in bench.SHAPE_WORKLOADS:
        assert name in bench.WORKLOADS
    for name, (B, H, W, h, hd, r, dtype, kind, spread, border, per_head) in bench.WORKLOADS.items():
        assert f"{H}x{W}" in name and f"b{B}" in name and f"h{h}x{hd}" in name and f"r{r}" in name
        assert bench.DTYPE_NAME[dtype] in name
        assert 2 * r + 2 <= min(H, W)


def test_peak_and_traffic_tables():
    import bench
    peak, kind = bench.measured_peak()
    assert peak > 1000 and ("measured" in kind or "fallback" in kind)
    traffic = bench.ncu_traffic_per_launch(bench.DEFAULT_WORKLOAD)
    assert traffic is None or traffic > 1e8
    assert bench.ncu_traffic_per_launch("no such workload") is None


def _run(args, env_extra):
    env = dict(os.environ, **env_extra)
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py")] + args, capture_output=True, text=True,
                          env=env, timeout=600)


def test_reference_arm_is_silent_on_other_ranks():
    res = _run(["--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "1"],
               {"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2"})
    assert res.returncode == 0 and res.stdout.strip() == ""


def test_reference_arm_prints_one_line_on_the_cpu_runnable_workload():
    res = _run(["--impl", "reference", "--steps", "1", "--warmup", "1", "--workload", "op_104x208_b1_h8x16_r1_f32_cross"], {})
    assert res.returncode == 0, res.stderr[-500:]
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["unit"] == "queries/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["gpu_launches"] == 0
    assert line["config"]["workload"] == "op_104x208_b1_h8x16_r1_f32_cross"
