"""`extern:nccl_*` launches through the host-memory executor: a group of one (every collective is a copy) in this
process, and two gloo ranks as child processes (all-reduce, all-gather, reduce-scatter, all-to-all)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_manifest_with_collectives_verifies_and_names_its_group():
    from kern_b200.parallel.coll_check import manifest
    from kern_b200.runtime import verify

    m, diags = verify(manifest(4, 128))
    assert m is not None, diags
    bad = manifest(2, 128)
    bad["programs"]["step"]["calls"][0]["args"][3] = {"rank": "nope"}
    m, diags = verify(bad)
    assert m is None and any("nope" in d for d in diags), diags


def test_group_of_one_copies(capsys):
    from kern_b200.parallel import coll_check

    assert coll_check.main(["--cpu", "--sizes", "1", "37"]) == 0
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["world"] == 1 and all(r["ok"] for r in line["results"]) and len(line["results"]) == 4


def test_two_gloo_ranks():
    env = dict(os.environ, PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29641", "-m", "kern_b200.parallel.coll_check", "--cpu", "--sizes", "1", "100", "4096"]
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, (p.stdout[-2000:], p.stderr[-2000:])
    line = next(json.loads(l) for l in p.stdout.splitlines() if l.startswith("{"))
    assert line["world"] == 2 and all(r["ok"] for r in line["results"]) and len(line["results"]) == 6
