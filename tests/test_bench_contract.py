"""The parts of bench.py's contract that need no GPU: more than one GPU is refused with one line and exit code 2,
and the reference arm always prints one JSON line and exits 0 (here, without a CUDA device, its `unavailable` form)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=300)


def test_more_than_one_gpu_is_refused_in_one_line():
    r = run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert r.returncode == 2
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_prints_one_json_line():
    import torch
    if torch.cuda.is_available():
        import pytest
        pytest.skip("with a GPU the arm runs gpt-fast itself, which takes minutes; bench.py --impl reference is run by hand")
    r = run("--impl", "reference", "--steps", "2", "--warmup", "1")
    assert r.returncode == 0, r.stderr[-500:]
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    out = json.loads(lines[0])
    assert out["impl"] == "reference" and "unavailable" in out


def test_reference_arm_imports_nothing_of_this_library():
    src = open(os.path.join(ROOT, "baseline", "reference_arm.py")).read()
    assert "gpt_fast_b200" not in src.replace("Nothing of gpt_fast_b200 is imported here", "")
