"""The examples stay runnable: the minimal manifest through the host-memory executor."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_minimal_example_on_cpu():
    p = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "python", "minimal.py"), "--cpu"], capture_output=True,
                       text=True, timeout=300)
    assert p.returncode == 0 and '"ok": true' in p.stdout, (p.stdout, p.stderr[-2000:])
