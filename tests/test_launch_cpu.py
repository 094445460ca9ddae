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


def test_clients_state_machine_who_answers_a_client():
    """The head answers from submission until it finishes, rejects or hands over; the front after. Tokens of a request
    the front has retired are dropped; a client that leaves a decoding request retires it at once and has the head free
    its seats; the head is told once of any other."""
    from kern_b200.serve.front import Clients

    c = Clients()
    for rid in ("a", "b", "c", "d"):
        c.submit(rid)
    with pytest.raises(ValueError):
        c.submit("a")
    assert c.note(("admit", "a", 32)) == [] and c.note(("emit", "a", 7)) == [("token", "a", 7)]
    assert c.tokens("a", 9, False) == []                       # not handed over yet: nothing of the decode tier's is its
    assert c.note(("decode", "a")) == [] and c.decoding() == 1
    assert c.tokens("a", 9, False) == [("token", "a", 9)]
    with pytest.raises(RuntimeError):
        c.note(("emit", "a", 1))                               # the head does not write to a request it handed over
    assert c.tokens("a", 4, True, "stop") == [("token", "a", 4), ("finish", "a", "stop")] and c.open() == 3
    assert c.tokens("a", 5, False) == [] and c.note(("emit", "a", 5)) == []      # retired: late words are dropped
    assert c.note(("emit", "b", 3)) == [("token", "b", 3)] and c.note(("finish", "b", "length")) == [("finish", "b", "length")]
    assert c.note(("reject", "c", "exceeds_pool")) == [("finish", "c", "abort")]
    # d's client leaves while the head still has it: told once; after the hand-over the front retires it itself
    gone = lambda rid: rid == "d"
    assert c.sweep(gone) == ([], [("gone", "d")]) and c.sweep(gone) == ([], [])
    c.note(("decode", "d"))
    assert c.sweep(gone) == ([("finish", "d", "abort")], [("abort", "d")]) and c.open() == 0


@pytest.mark.timeout(300)
@pytest.mark.parametrize("front", [False, True])
def test_prefill_and_decode_tiers_under_the_scheduler(front):
    """`launch_pd` with host-memory executors: requests wait for a seat on the decode tier (it holds two at a time), are
    prefilled in chunks by the local scheduler, pushed into the granted seats and finished by the decode tier; the
    tokens are those of one engine, and the exact integer model with a per-sequence state slot agrees with its twin.
    `front`: the prefill scheduler on a head thread, the tier object only relaying (`serve/front.py`)."""
    spec = {"manifest": toy_int.build_manifest(True), "cpu": True, "tokens": 16 * 30, "slots": 6}
    tier, worker = launch.launch_pd(spec, dict(spec, tokens=16 * 12, slots=3), chunk=32, max_seqs=3, decode_max_seqs=2,
                                    stop_ids=(toy_int.EOS,), timeout=60, front=front)
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
            seen_waiting = max(seen_waiting, tier.metrics()["pd"].get("waiting_for_seat", 1))
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
        assert tier.abort("late")
        for _ in range(2000):
            if tier.idle():
                break
            tier.step()
        assert late.finished == "abort" and tier.idle() and 3 <= len(late.out) < 50
    finally:
        launch.shutdown_pd(tier, worker)
    assert not worker.is_alive()
