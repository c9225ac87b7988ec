"""The benchmark's command line where it needs no GPU: more than one GPU is refused in one line."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_code_2():
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", "2", "--steps", "2", "--warmup", "1"],
                       capture_output=True, text=True, timeout=120)
    assert p.returncode == 2
    lines = [l for l in (p.stdout + p.stderr).splitlines() if l.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]
