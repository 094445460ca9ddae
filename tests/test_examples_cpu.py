"""The examples stay runnable: the minimal manifest through the host-memory executor."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_minimal_example_on_cpu():
    p = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "python", "minimal.py"), "--cpu"], capture_output=True,
                       text=True, timeout=300)
    assert p.returncode == 0 and '"ok": true' in p.stdout, (p.stdout, p.stderr[-2000:])


def test_pipeline_chain_example_on_cpu():
    p = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "python", "pp_chain.py"), "--cpu"], capture_output=True,
                       text=True, timeout=300)
    assert p.returncode == 0 and '"ok": true' in p.stdout, (p.stdout, p.stderr[-2000:])


def test_agent_replay_example_on_cpu():
    p = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "python", "agent_replay.py"), "--cpu"], capture_output=True,
                       text=True, timeout=300)
    assert p.returncode == 0 and '"ok": true' in p.stdout, (p.stdout, p.stderr[-2000:])
