"""bench.py's contract where no GPU is needed: more than one GPU is refused with one line
and exit code 2; the reference arm says why it is unavailable and exits 0."""

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def run(*args):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True,
                          text=True, timeout=300)


def test_more_than_one_gpu_is_refused():
    out = run("--gpus", "2")
    assert out.returncode == 2
    assert len(out.stdout.strip().splitlines()) == 1 and "one GPU" in out.stdout


def test_reference_arm_without_a_gpu_or_install_says_so():
    import torch
    if torch.cuda.is_available():
        return                      # on a GPU box the arm runs the reference; not timed here
    out = run("--impl", "reference")
    assert out.returncode == 0
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unavailable"]
