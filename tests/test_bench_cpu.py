"""The reference arm of bench.py runs without a GPU: it times the reference's
CPU path (oracle/_ref, or the C restatement when the reference was not built)
and prints one JSON line with the keys the bench contract names."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_contract_line():
    done = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "diamond1000", "--steps", "2", "--warmup", "1"],
        capture_output=True, text=True, timeout=300, cwd=ROOT,
    )
    assert done.returncode == 0, done.stderr[-2000:]
    line = json.loads(done.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    assert line["metric"] == "neighbor pairs/s" and line["unit"] == "pairs/s" and line["higher_is_better"] is True
    assert line["n_gpus"] == 1 and line["steps"] == 2
    assert line["value"] > 0 and line["ms_per_step"] > 0
    assert line["config"]["n_points"] == 1000 and line["config"]["n_pairs"] == 89072
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["e2e"]["value"] == line["value"]


def test_our_arm_refuses_to_run_without_a_gpu():
    """No CPU fallback: without a CUDA device the product arm stops with a message."""
    import torch

    if torch.cuda.is_available():
        return
    done = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bench.py"), "--workload", "diamond1000", "--steps", "1", "--warmup", "1"],
        capture_output=True, text=True, timeout=300, cwd=ROOT,
    )
    assert done.returncode != 0
    assert "CUDA" in done.stderr
