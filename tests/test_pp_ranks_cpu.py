"""Pipelined prefill with a process per stage on CPU ranks (gloo, host-memory runtimes): every chunk of every prompt is
in flight before the first token is read, and the tokens equal the uncut model's; a stage that stops answering (made on
the host: it stops calling) ends its neighbours' waits with a timeout error that names it, not with a hang."""
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(world, port, *extra, timeout=300):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), "-m", "kern_b200.parallel.pp_pipeline_check", "--cpu", *extra]
    p = subprocess.run(cmd, cwd=ROOT, env=dict(os.environ, PYTHONPATH=ROOT), capture_output=True, text=True, timeout=timeout)
    lines = [json.loads(l) for l in p.stdout.splitlines() if l.startswith("{")]
    return p, lines


def test_three_stages_equal_the_uncut_model_with_every_chunk_in_flight():
    p, lines = _run(3, 29741)
    assert p.returncode == 0, (p.stdout[-2000:], p.stderr[-2000:])
    assert lines and lines[0]["ok"] and lines[0]["stages"] == 3 and lines[0]["items"] >= 10, lines


def test_a_stage_that_stops_answering_ends_in_a_timeout_naming_it():
    t0 = time.monotonic()
    p, lines = _run(3, 29742, "--stall-stage", "1", "--timeout", "3")
    assert time.monotonic() - t0 < 120
    assert p.returncode != 0
    hit = [l for l in lines if l.get("timeout")]
    assert hit and "stage 1" in hit[0]["timeout"] and not hit[0]["ok"], (lines, p.stderr[-1500:])


def test_items_round_trip_the_wire():
    from kern_b200.serve.pp_ranks import Item

    it = Item(k=3, program="prefill", vars={"tokens": 5, "seqs": 1}, columns={"token_ids": ["i64", [1, 2, 3, 4, 5]]}, emits="next_token",
              groups=1, real=1)
    back = Item.from_wire(it.to_wire())
    assert back == it
