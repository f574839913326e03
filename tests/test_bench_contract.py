"""What bench.py answers without measuring anything: more than one GPU, and the reference arm on a
machine without a device."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args, env=None):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          env=env, timeout=300)


def test_more_than_one_gpu_is_refused_in_one_line():
    r = run("--gpus", "2", "--steps", "4", "--warmup", "3")
    assert r.returncode == 2
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_the_reference_arm_says_why_the_engine_is_unavailable():
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")                   # no device: nothing is built or timed
    r = run("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3", env=env)
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "Rust" in line["unavailable"]
    assert "\n" not in line["unavailable"]
