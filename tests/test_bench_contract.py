"""The parts of bench.py's contract that need no GPU: the reference arm says why it is unavailable and exits 0;
more than one GPU is refused with one line and exit code 2; without a GPU the own arm fails loudly."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _run(*args):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, cwd=ROOT,
                          timeout=300)


def test_reference_arm_is_unavailable_and_says_why():
    r = _run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "3")
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "\n" not in line["unavailable"] and len(line["unavailable"]) > 20


def test_more_than_one_gpu_is_refused_with_one_line():
    r = _run("--gpus", "2")
    assert r.returncode == 2
    out = (r.stdout + r.stderr).strip().splitlines()
    assert len(out) == 1 and "one GPU" in out[0]
