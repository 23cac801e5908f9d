"""The benchmark harness contract that can be checked without a GPU: defaults, the reference arm's JSON line."""
import json
import os
import subprocess
import sys

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_and_exits_zero():
    res = subprocess.run([sys.executable, os.path.join(REPO, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2",
                          "--warmup", "3"], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and ("unavailable" in rec or "value" in rec)


def test_defaults_follow_the_timing_rules():
    sys.path.insert(0, REPO)
    import importlib

    bench = importlib.import_module("bench")
    argv, sys.argv = sys.argv, ["bench.py"]
    try:
        a = bench.parse()
    finally:
        sys.argv = argv
    assert a.gpus == 1 and a.warmup >= 3 and a.steps >= 1 and a.model == "llama3-8b"
    assert a.global_batch == 64 and a.seq_len == 4096 and a.layers == 0 and not a.no_e2e
