"""Rank *processes* (spawned, host-memory runtimes) behind the head: a data-parallel tier of the exact integer model
answers exactly; a rank process that is killed ends the serving loop's connection (fail fast is observable)."""
import random

import pytest

from kern_b200.models import toy_int
from kern_b200.serve import launch
from kern_b200.serve.scheduler import Request


@pytest.mark.timeout(120)
def test_two_rank_processes_serve_exactly():
    spec = {"manifest": toy_int.build_manifest(False), "cpu": True, "tokens": 16 * 30}
    sched, ex, procs = launch.launch(spec, world=2, tp=1, chunk=32, max_seqs=2, timeout=60)
    ex.watch.on_lost = lambda who: None          # the test ends the ranks itself
    try:
        rng = random.Random(2)
        reqs = [Request(id=f"r{i}", prompt=[rng.randrange(256) for _ in range(rng.randint(3, 50))], max_tokens=5,
                        stop_ids=(toy_int.EOS,)) for i in range(6)]
        spots = [sched.submit(r) for r in reqs]
        assert set(spots) == {0, 1}
        for _ in range(400):
            if sched.idle():
                break
            sched.step()
        assert sched.idle()
        for r in reqs:
            assert [t for t in r.out if t != toy_int.EOS] == toy_int.generate(r.prompt, 5)
        assert sched.stats.decode_tokens > 0 and sched.metrics()["kv_total_blocks"] == 2 * 30
    finally:
        launch.shutdown(ex, procs)
    assert all(not p.is_alive() for p in procs)


@pytest.mark.timeout(300)
def test_pipeline_of_stage_processes_under_the_scheduler():
    """`launch_pp`: the launching process is the head, the second stage a process of its own (gloo, host-memory runtimes);
    chunked prompts and decode steps of several requests give the tokens of one engine."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, "-m", "kern_b200.serve.launch", "--stages", "2", "--cpu"], cwd=root, capture_output=True, text=True,
                       timeout=280, env=dict(os.environ, PYTHONPATH=root))
    assert p.returncode == 0, (p.stdout[-1500:], p.stderr[-3000:])
    line = json.loads([l for l in p.stdout.splitlines() if l.startswith("{")][-1])
    assert line["ok"] and line["stages"] == 2 and line["tokens"] == 20


@pytest.mark.timeout(300)
def test_prefill_and_decode_tiers_under_the_scheduler():
    """`launch_pd` with host-memory executors: requests wait for a seat on the decode tier (it holds two at a time), are
    prefilled in chunks by the local scheduler, pushed into the granted seats and finished by the decode tier; the
    tokens are those of one engine, and the exact integer model with a per-sequence state slot agrees with its twin."""
    spec = {"manifest": toy_int.build_manifest(True), "cpu": True, "tokens": 16 * 30, "slots": 6}
    tier, worker = launch.launch_pd(spec, dict(spec, tokens=16 * 12, slots=3), chunk=32, max_seqs=3, decode_max_seqs=2,
                                    stop_ids=(toy_int.EOS,), timeout=60)
    try:
        rng = random.Random(7)
        reqs = [Request(id=f"r{i}", prompt=[rng.randrange(256) for _ in range(rng.randint(3, 60))], max_tokens=6,
                        stop_ids=(toy_int.EOS,)) for i in range(7)]
        reqs.append(Request(id="one", prompt=[5, 6, 7, 8], max_tokens=1, stop_ids=(toy_int.EOS,)))     # ends with its first token
        for r in reqs:
            tier.submit(r)
        with pytest.raises(ValueError):
            tier.submit(Request(id="big", prompt=[1] * 600, max_tokens=4))
        seen_waiting = 0
        for _ in range(4000):
            if tier.idle():
                break
            tier.step()
            seen_waiting = max(seen_waiting, tier.metrics()["pd"]["waiting_for_seat"])
        assert tier.idle() and seen_waiting > 0
        for r in reqs:
            assert r.finished in ("stop", "length"), (r.id, r.finished)
            assert [t for t in r.out if t != toy_int.EOS] == toy_int.generate(r.prompt, r.max_tokens, True), r.id
        m = tier.metrics()
        assert m["pd"]["decode_tier"]["seqs"] <= 2 and m["kv_used_blocks"] >= 0
        # an abort while a request decodes on the other tier gives its seat back
        late = Request(id="late", prompt=[9] * 20, max_tokens=50, stop_ids=())
        tier.submit(late)
        for _ in range(2000):
            tier.step()
            if len(late.out) >= 3:
                break
        assert tier.abort("late") and late.finished == "abort" and tier.idle()
    finally:
        launch.shutdown_pd(tier, worker)
    assert not worker.is_alive()
