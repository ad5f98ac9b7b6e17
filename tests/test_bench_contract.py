"""What `bench.py` promises whoever drives it, as far as a machine without a GPU can show it: more than
one GPU is refused with one line and exit code 2."""

from __future__ import annotations

import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench(*args: str) -> subprocess.CompletedProcess:
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          cwd=ROOT, timeout=600)


@pytest.mark.parametrize("gpus", ["2", "8"])
def test_more_than_one_gpu_is_refused_in_one_line(gpus):
    p = _bench("--gpus", gpus, "--steps", "2", "--warmup", "1")
    assert p.returncode == 2
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]
