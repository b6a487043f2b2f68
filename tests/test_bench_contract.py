"""The parts of bench.py's contract that need no GPU: more than one GPU is refused with one line
and exit code 2; the reference arm prints its one JSON line and exits 0 (one layer of the bench
sizes through the reference's own CPU engine where a copy of the reference is at hand, else the
line that says why it is unavailable)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args, timeout=120):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=timeout)


def test_more_than_one_gpu_is_refused_with_one_line():
    p = run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert p.returncode == 2
    assert len(p.stdout.strip().splitlines()) == 1 and "one GPU" in p.stdout


def test_reference_arm_prints_one_line_of_the_same_shape():
    p = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1", "--layers", "1", "--batch", "2",
            "--skip-points", timeout=900)
    assert p.returncode == 0, p.stderr[-1000:]
    lines = p.stdout.strip().splitlines()
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference"
    if "unavailable" in line:
        assert isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]
        return
    assert line["value"] > 0 and line["unit"] == "tokens/s" and line["e2e"]["value"] > 0
    assert line["config"]["layers"] == 1 and line["config"]["layers_full"] == 32 and line["config"]["global_batch"] == 2
    assert line["steps"] == 2 and line["warmup"] == 3 and line["gpu_launches"] == 0
