"""What bench.py answers without a GPU: more than one GPU is refused with exit code 2 and one line; the reference
arm, which needs a GPU to draw the model it gives the reference program, prints its `unavailable` record and exits 0."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=300)


def test_more_than_one_gpu_is_refused():
    r = run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert r.returncode == 2 and len(r.stdout.strip().splitlines()) == 1 and "N=2" in r.stdout


def test_reference_arm_answers_in_one_line_without_a_gpu():
    r = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert r.returncode == 0
    d = json.loads(r.stdout)
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and "\n" not in d["unavailable"]
