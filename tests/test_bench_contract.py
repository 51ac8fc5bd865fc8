"""bench.py prints exactly one JSON line on stdout, whatever the libraries it loads print (CPU: the reference arm;
GPU: the default arm with a small step count)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REQUIRED = ["metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
            "dtype", "data", "config", "cpu_baseline", "e2e"]


def _run(args, timeout):
    env = dict(os.environ, NCCL_DEBUG="VERSION")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py")] + args, cwd=ROOT, env=env, capture_output=True,
                       text=True, timeout=timeout)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [ln for ln in p.stdout.split("\n") if ln.strip()]
    assert len(lines) == 1, f"stdout must hold one line, got {len(lines)}: {p.stdout[:300]!r}"
    return json.loads(lines[0])


def test_reference_arm_prints_one_json_line():
    sys.path.insert(0, ROOT)
    import bench
    from oracle import ref_gold
    line = _run(["--impl", "reference", "--steps", "1", "--warmup", "0"], 600)
    # the reference's own gold recipes when they are installed under oracle/_ref, else the C restatement
    assert line["impl"] == "reference" and line["cpu_baseline"]["kind"] == ("reference" if ref_gold.available() else "port")
    for k in REQUIRED:
        assert k in line, k
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["value"] == line["value"]
    assert line["config"] == bench.CONFIG and line["metric"] == bench.METRIC      # the same workload as the GPU arm
    assert line["cpu_baseline"]["cores"] >= 1 and "rows" in line["cpu_baseline"]["sample"]


def test_reference_arm_under_torchrun_prints_once():
    """N > 1: the launcher starts N processes; rank 0 alone measures and prints, the others exit 0 without work."""
    env = dict(os.environ, NCCL_DEBUG="VERSION")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29541", os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
           "--warmup", "0"]
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [ln for ln in p.stdout.split("\n") if ln.strip().startswith("{")]
    assert len(lines) == 1, p.stdout[:500]
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["n_gpus"] == 2


@pytest.mark.gpu
def test_default_arm_prints_one_json_line():
    line = _run(["--steps", "3", "--warmup", "3"], 900)
    for k in REQUIRED + ["roofline", "gpu_launches", "clocks"]:
        assert k in line, k
    sys.path.insert(0, ROOT)
    import bench
    assert line["gpu_launches"] == 9 and line["n_gpus"] == 1          # mxfp8 (+ amax), exchange warp, nvfp4 per step
    assert line["config"] == bench.CONFIG and line["scaling"] == "strong"
    assert line["roofline"]["bound"] == "hbm" and 0.3 < line["roofline"]["frac"] < 1.2
    assert line["roofline"]["launch_ms_avg"] <= line["ms_per_step"]
    assert line["roofline"]["step"]["bit_identical"] is True
    assert line["e2e"]["h2d_bytes_per_step"] > 0 and line["e2e"]["d2h_bytes_per_step"] > 0
    assert line["cpu_baseline"]["kind"] in ("reference", "port")
