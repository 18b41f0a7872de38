"""The benchmark's command line, as far as it can be checked without a GPU: more than one GPU is refused with one
line and exit code 2."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args, timeout=600):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=timeout, cwd=ROOT)


def test_more_than_one_gpu_is_refused_with_one_line():
    r = run("--gpus", "2")
    assert r.returncode == 2
    assert len(r.stdout.strip().splitlines()) == 1 and "single GPU" in r.stdout
