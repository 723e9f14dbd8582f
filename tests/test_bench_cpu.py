"""bench.py contract pieces that can be checked without a GPU: the reference (CPU) arm prints one
JSON line with the agreed keys, and the algorithmic byte counts match the formulas."""
import json
import os
import subprocess
import sys

import bench

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_algorithmic_bytes_match_the_published_table():
    # 64x56x56x64 G4 fp32: each tensor counted once -> 192.7 MB forward, 334.0 MB backward
    fwd, bwd = bench.algorithmic_bytes(64, 56, 64, 4, 4)
    assert round(fwd / 1e6, 1) == 192.7 and round(bwd / 1e6, 1) == 334.0
    fwd, bwd = bench.algorithmic_bytes(64, 7, 512, 32, 2)
    assert round(fwd / 1e6, 2) == 11.84 and round(bwd / 1e6, 2) == 20.47


def test_reference_arm_prints_one_json_line():
    env = dict(os.environ, OMP_NUM_THREADS="4")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "1"], capture_output=True, text=True, env=env, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == bench.METRIC and d["unit"] == "GB/s"
    assert d["value"] > 0 and d["higher_is_better"] is True
    from oracle import ref_core
    # the reference's own pure-PyTorch core when its file is mounted or installed under oracle/_ref,
    # else the restatement of the same algorithm
    assert d["cpu_baseline"]["kind"] == ("reference" if ref_core.available() else "port")
    assert d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["sample"]
    c0 = d["cpu_baseline"]["config0"]
    assert c0["fwd_ms"] > 0 and c0["fwd_bwd_ms"] > c0["fwd_ms"]
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert d["config"]["workload"] == bench.WORKLOAD


def test_non_zero_ranks_of_the_reference_arm_exit_quietly():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                         capture_output=True, text=True, env=env, timeout=120, cwd=ROOT)
    assert out.returncode == 0 and out.stdout.strip() == ""
