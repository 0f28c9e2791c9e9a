"""The benchmark's command line parses without a GPU and offers the legs the documentation names."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_bench_help_lists_the_legs():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--help"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    for flag in ("--gpus", "--steps", "--warmup", "--impl", "--sweep", "--group", "--tp-only", "--c3-only", "--fused", "--strict"):
        assert flag in out.stdout, flag
