"""Seeded simulations of the serving loop against the model engine (no runtime): every schedule must drain with
exact answers, no foreign reads and no leaks; across seeds the interesting paths (prefix hits, evictions, aborts) occur."""
import pytest

from kern_b200.testing import sim


@pytest.mark.parametrize("lined", [False, True])
def test_seeded_schedules_hold_the_invariants(lined):
    hits = evictions = aborted = 0
    for seed in range(30):
        o = sim.run(seed, lined=lined)
        assert o.violations == [], (seed, o.violations[:3])
        assert o.finished + o.aborted == o.requests
        hits += o.prefix_hits
        evictions += o.evictions
        aborted += o.aborted
    assert hits > 0 and evictions > 0 and aborted > 0


def test_the_simulator_notices_a_wrong_page():
    """Hand a sequence someone else's page: the model engine reports the foreign read and a wrong token."""
    eng = sim.SimEngine(pages=8)
    a, b = eng.open(32), eng.open(32)
    eng.step([(a, list(range(20)))])
    eng.step([(b, list(range(100, 120)))])
    eng.mem[b.lease.pages[0]] = dict(eng.mem[a.lease.pages[0]])        # the bug: b's first page now holds a's tokens
    got = eng.step([(b, [5])])[0][0]
    from kern_b200.models import toy_int
    want = toy_int.next_of(sum(toy_int.slot_sum(t, p) for p, t in enumerate(list(range(100, 120)) + [5])) & toy_int.M)
    assert got != want


@pytest.mark.parametrize("chunk", range(4))
def test_fleet_of_head_tiers_and_clients_holds_the_protocol_invariants(chunk):
    """1000 seeded schedules of the whole deployment (clients, prefill head, two or three decode tiers, delayed links,
    slow tiers, aborts mid-flight) over the production state machines: every stream is the model's, every request ends
    once, no seat or page is left behind — and the paths that make this hard all occur."""
    from kern_b200.testing import sim_fleet

    finished = refused = aborted = busy = 0
    for seed in range(chunk * 250, (chunk + 1) * 250):
        o = sim_fleet.run(seed, lined=bool(seed % 2), tiers=2 + seed % 2, requests=10)
        assert o.violations == [], (seed, o.violations[:3])
        finished += o.finished
        refused += o.refused
        aborted += o.aborted
        busy += o.busy_seen
    assert finished > 1000 and aborted > 100 and busy > 50 and refused > 0
