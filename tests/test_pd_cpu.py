"""Prefill/decode disaggregation on CPU: a prefill engine and a decode engine (two runtimes of the exact integer
model), seats reserved before prefill, pages and the state slot pushed by the plan, tokens streamed back."""
import random

import pytest

from kern_b200.cpu import CpuRuntime
from kern_b200.engine import Engine
from kern_b200.models import toy_int
from kern_b200.serve import pd


def push(plan, p_rt, d_rt):
    """Execute a push plan between two host-memory runtimes (on GPUs: copies into the mapped peer pools)."""
    for name, s in p_rt.doc["states"].items():
        src, dst = p_rt.states[name], d_rt.states[name]
        if s.get("bytes_per_token"):
            n = s["bytes_per_token"] * p_rt.page_unit
            for a, b in plan["pages"]:
                dst[b * n:(b + 1) * n] = src[a * n:(a + 1) * n]
        elif s.get("bytes_per_seq") and plan["slot"] is not None:
            n = s["bytes_per_seq"]
            a, b = plan["slot"]
            dst[b * n:(b + 1) * n] = src[a * n:(a + 1) * n]


@pytest.mark.parametrize("lined", [False, True])
def test_handoff_matches_twin(lined):
    doc = toy_int.build_manifest(lined)
    p_rt = CpuRuntime(doc, tokens=16 * 30, slots=6 if lined else 0)
    d_rt = CpuRuntime(doc, tokens=16 * 12, slots=3 if lined else 0)        # a small decode tier: it will say Busy
    p_eng, d_eng = Engine(p_rt), Engine(d_rt)
    assert pd.cover(p_rt.doc, p_rt.page_unit, pd.pools_message(d_rt.doc, d_rt.page_unit, 1, 256)) == []
    dec = pd.Decoder(d_eng, max_seqs=3, stop_ids=(toy_int.EOS,))
    hand = pd.Handoffs(p_rt.page_unit)
    relay = pd.Relay()
    rng = random.Random(5)
    prompts = {f"r{i}": [rng.randrange(256) for _ in range(rng.randint(5, 60))] for i in range(6)}
    out = {r: [] for r in prompts}
    done = set()
    for r in prompts:
        relay.watch(r, lambda tok, last, r=r: (out[r].append(tok), done.add(r) if last else None))
    max_tokens = 7
    to_d = [hand.ask(r, len(p) + max_tokens) for r, p in prompts.items()]
    seqs = {}
    busy_seen = False
    for _ in range(400):
        to_p = []
        for m in to_d:
            to_p += dec.handle(m)
        to_p += dec.step()
        to_d = []
        for m in to_p:
            busy_seen |= "busy" in m
            events = hand.told(m)
            relay.deliver(events)
            for kind, req, val in events:
                if kind == "granted":
                    # prefill on P (whole prompt, one call), push, hand over with the first token
                    s = p_eng.open(len(prompts[req]))
                    first = p_eng.step([(s, prompts[req])])[0][0]
                    for plan in hand.prefilled(req, s.lease, len(prompts[req])):
                        push(plan, p_rt, d_rt)
                    out[req].append(first)
                    to_d.append(hand.pushed(req, first, len(prompts[req]), max_tokens - 1, stop_ids=(toy_int.EOS,)))
                    p_eng.close(s)
        if len(done) == len(prompts):
            break
    assert len(done) == len(prompts) and busy_seen
    for r, p in prompts.items():
        want = toy_int.generate(p, max_tokens, lined)
        got = [t for t in out[r] if t != toy_int.EOS]
        assert got == want, r
    assert d_eng.pool.free_pages == d_eng.pool.total_pages and not dec.seats


def test_cover_names_every_mismatch_and_moves_checks_room():
    a, b = toy_int.build_manifest(False), toy_int.build_manifest(True)
    errs = pd.cover(a, 16, pd.pools_message(b, 8, 1, 256))
    assert any("line" in e for e in errs) and any("page of 16" in e for e in errs)
    assert pd.moves([5, 6, 7], {"pages": [1, 2], "slot": 4}, 20, 16, src_slot=2) == {"pages": [[5, 1], [6, 2]], "slot": [2, 4]}
    with pytest.raises(ValueError):
        pd.moves([5], {"pages": [1, 2], "slot": -1}, 20, 16)


def test_refuse_and_abort_and_two_choices():
    doc = toy_int.build_manifest(False)
    d_eng = Engine(CpuRuntime(doc, tokens=16 * 4))
    dec = pd.Decoder(d_eng)
    assert "refuse" in dec.handle({"reserve": {"req": "big", "tokens": 16 * 40}})[0]
    g = dec.handle({"reserve": {"req": "a", "tokens": 16 * 4}})[0]["grant"]
    assert len(g["seats"][0]["pages"]) == 4
    assert "busy" in dec.handle({"reserve": {"req": "b", "tokens": 16}})[0]
    replies = dec.handle({"abort": {"req": "a"}})
    assert "grant" in replies[0] and replies[0]["grant"]["req"] == "b" and "room" in replies[1]
    t = pd.Tiers(3, seed=1)
    t.report(0, {"seqs": 50, "free_pages": 1, "total_pages": 100})
    t.report(1, {"seqs": 0, "free_pages": 100, "total_pages": 100})
    t.report(2, {"seqs": 50, "free_pages": 1, "total_pages": 100})
    picks = [t.pick() for _ in range(200)]
    assert picks.count(1) > 100 and t.pick(busy={0, 1, 2}) is None and t.pick(busy={0, 2}) == 1
