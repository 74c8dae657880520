"""bench.py's contract: more than one GPU is refused with one line and exit code 2; the
reference arm prints the contract's line where the reference is installed and a GPU is there,
and otherwise says why it is unavailable and exits 0."""

import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def run(*args):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True,
                          text=True, timeout=900)


def test_more_than_one_gpu_is_refused():
    out = run("--gpus", "2")
    assert out.returncode == 2
    assert len(out.stdout.strip().splitlines()) == 1 and "one GPU" in out.stdout


def check_reference_line(out):
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    if "unavailable" in line:
        assert line["unavailable"]
        return None
    assert line["unit"] == "tokens/s" and line["value"] > 0 and line["n_gpus"] == 1
    assert line["config"]["model"] == "Qwen2.5-1.5B shape" and line["config"]["layers"] == 28
    assert line["prefill"]["tokens"] == 2048 and line["steps"] == 2
    return line


def test_reference_arm_without_a_gpu_says_why_it_is_unavailable():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present: the arm is run by the gpu-marked test below")
    assert check_reference_line(run("--impl", "reference", "--steps", "2", "--batch", "1")) is None


@pytest.mark.gpu
def test_reference_arm_on_a_gpu_prints_the_contracts_line_or_says_why_not():
    """Where the reference is installed it runs, unmodified, and its line names the same
    metric and shape as the engine's; where it is not, the arm says so and exits 0."""
    check_reference_line(run("--impl", "reference", "--steps", "2", "--batch", "1"))
