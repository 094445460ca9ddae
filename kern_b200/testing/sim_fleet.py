"""Deterministic simulation of a whole deployment: clients, a prefill head, several decode tiers, and the links between
them — no runtime, no GPU, no clock, no threads. Every actor is the production state machine (`serve.pd.Handoffs`,
`Decoder`, `Tiers`, `Relay`; the prefill side steps a real `Engine`-shaped model engine) over `sim.SimEngine`, whose
"device" is a table of what every KV slot and state slot holds. A seeded driver interleaves the actors one event at a
time: requests arrive, links deliver their messages late (in order per link), a tier is slow for a while, clients
abort mid-flight. After every event the invariants of the protocol are checked:

  * every token a client receives is the exact integer model's, in order, and every request ends exactly once
    (finished, refused or aborted);
  * a seat is granted before anything is pushed into it, and a push only ever lands in pages of that seat;
  * nothing leaks: when the schedule has drained, every pool of every tier is whole and no seat is left.

Reference counterpart: crates/kern-serve/tests/sim.rs:1-116 (head + stages + tiers + decoder + clients, 1000 seeds).
"""
from __future__ import annotations

import random
from collections import deque
from dataclasses import dataclass, field

from ..models import toy_int
from ..serve import pd
from . import sim


@dataclass
class FleetOutcome:
    seed: int
    requests: int = 0
    finished: int = 0
    refused: int = 0
    aborted: int = 0
    events: int = 0
    busy_seen: int = 0
    late_deliveries: int = 0
    violations: list[str] = field(default_factory=list)


class _Link:
    """One direction between two actors: FIFO, each message held back a random number of events."""

    def __init__(self, rng: random.Random, max_delay: int):
        self.rng, self.max_delay = rng, max_delay
        self.q: deque = deque()

    def send(self, now: int, msg) -> None:
        due = now + self.rng.randint(0, self.max_delay)
        if self.q and due < self.q[-1][0]:
            due = self.q[-1][0]                    # in order per link
        self.q.append((due, msg))

    def take(self, now: int) -> list:
        out = []
        while self.q and self.q[0][0] <= now:
            out.append(self.q.popleft()[1])
        return out


def run(seed: int, lined: bool = False, tiers: int = 2, requests: int = 14, max_events: int = 6000) -> FleetOutcome:
    rng = random.Random(seed)
    unit = 16
    out = FleetOutcome(seed=seed, requests=requests)
    p_eng = sim.SimEngine(unit=unit, pages=40, slots=8 if lined else 0, rows_max=256)
    d_engs = [sim.SimEngine(unit=unit, pages=rng.choice([6, 10, 16]), slots=4 if lined else 0) for _ in range(tiers)]
    decs = [pd.Decoder(e, max_seqs=rng.randint(2, 4), stop_ids=(toy_int.EOS,)) for e in d_engs]
    hand = pd.Handoffs(unit)
    pick = pd.Tiers(tiers, seed=seed)
    relay = pd.Relay()
    to_d = [_Link(rng, rng.randint(0, 4)) for _ in range(tiers)]
    to_p = [_Link(rng, rng.randint(0, 4)) for _ in range(tiers)]
    slow_until = [0] * tiers

    prompts, max_tok, got, state, tier_of = {}, {}, {}, {}, {}
    arrivals = deque()
    for i in range(requests):
        rid = f"r{i}"
        prompts[rid] = [rng.randrange(256) for _ in range(rng.randint(1, 70) if rng.random() < 0.9 else rng.randint(90, 140))]
        max_tok[rid] = rng.randint(1, 9)
        arrivals.append(rid)
    waiting_for_tier: deque[str] = deque()          # every tier said Busy: ask again on Room

    def sink(rid):
        def f(tok, last):
            if state[rid] in ("finished", "aborted", "refused"):
                if state[rid] != "aborted":
                    out.violations.append(f"{rid}: a token after the request ended ({state[rid]})")
                return
            if tok is None:
                state[rid] = "refused"
                out.refused += 1
                return
            got[rid].append(tok)
            if last:
                state[rid] = "finished"
                out.finished += 1
        return f

    def ask(rid, now) -> bool:
        t = pick.pick(busy=hand.busy_tiers)
        if t is None:
            return False
        tier_of[rid] = t
        need = len(prompts[rid]) + max_tok[rid]
        to_d[t].send(now, hand.ask(rid, need, tier=t))
        state[rid] = "asked"
        return True

    def prefill_and_push(rid, now):
        """A granted request: prefill on the head's engine, run the push plan into the tier's model device, hand over."""
        t = tier_of[rid]
        p = prompts[rid]
        s = p_eng.open(len(p))
        first = p_eng.step([(s, p)])[0][0]
        h = hand.items[rid]
        seat_pages = {pg for seat in h.seats for pg in seat["pages"]}
        for plan in hand.prefilled(rid, s.lease, len(p)):
            for a, b in plan["pages"]:
                if b not in seat_pages:
                    out.violations.append(f"{rid}: a page was pushed outside the granted seat")
                d_engs[t].mem[b] = dict(p_eng.mem.get(a, {}))
            if plan["slot"] is not None:
                a, b = plan["slot"]
                d_engs[t].carry[b] = p_eng.carry.get(a, 0)
        p_eng.close(s)
        got[rid].append(first)
        if first == toy_int.EOS or max_tok[rid] == 1:
            state[rid] = "finished"
            out.finished += 1
            relay.sinks.pop(rid, None)
            m = hand.abort(rid)                      # nothing to decode: give the seat back
            if m:
                to_d[t].send(now, m)
            return
        state[rid] = "started"
        to_d[t].send(now, hand.pushed(rid, first, len(p), max_tok[rid] - 1, stop_ids=(toy_int.EOS,)))

    now = 0
    while now < max_events:
        now += 1
        out.events = now
        active = [r for r, s in state.items() if s in ("asked", "granted", "started")]
        if not arrivals and not active and not waiting_for_tier and not any(l.q for l in to_d + to_p):
            break
        roll = rng.random()
        if arrivals and roll < 0.25:
            rid = arrivals.popleft()
            got[rid], state[rid] = [], "new"
            relay.watch(rid, sink(rid))
            if not ask(rid, now):
                waiting_for_tier.append(rid)
                state[rid] = "waiting"
        elif active and roll < 0.29:
            rid = rng.choice(active)                  # the client goes away mid-flight
            m = hand.abort(rid)
            relay.sinks.pop(rid, None)
            state[rid] = "aborted"
            out.aborted += 1
            if m:
                to_d[tier_of[rid]].send(now, m)
        elif roll < 0.33:
            slow_until[rng.randrange(tiers)] = now + rng.randint(5, 40)      # a tier stops stepping for a while
        # the tiers: take what has arrived, step
        for t in range(tiers):
            msgs = to_d[t].take(now)
            out.late_deliveries += len(msgs)
            for m in msgs:
                for reply in decs[t].handle(m):
                    to_p[t].send(now, reply)
            if now >= slow_until[t]:
                for reply in decs[t].step():
                    to_p[t].send(now, reply)
        # the head: take what has arrived
        for t in range(tiers):
            for m in to_p[t].take(now):
                out.busy_seen += "busy" in m
                if "tokens" in m or "grant" in m:
                    pick.report(t, (m.get("tokens") or m.get("grant"))["load"])
                if "busy" in m:
                    rid = m["busy"]["req"]           # the tier queued the ask itself; nothing to do but note it
                events = hand.told(m, tier=t)
                relay.deliver(events)
                for kind, rid, val in events:
                    if kind == "granted":
                        if state.get(rid) == "aborted":
                            continue                  # the abort is already on its way; the tier frees the seat
                        state[rid] = "granted"
                        prefill_and_push(rid, now)
                    elif kind == "room":
                        while waiting_for_tier and ask(waiting_for_tier[0], now):
                            waiting_for_tier.popleft()
        while waiting_for_tier and state.get(waiting_for_tier[0]) == "aborted":
            waiting_for_tier.popleft()
    else:
        out.violations.append("the schedule did not drain")
    # every stream is the model's
    for rid, p in prompts.items():
        if state.get(rid) == "finished":
            want = toy_int.generate(p, max_tok[rid], lined)
            have = [t for t in got[rid] if t != toy_int.EOS]
            if have != want:
                out.violations.append(f"{rid}: client got {have}, the model says {want}")
        elif state.get(rid) not in ("aborted", "refused"):
            out.violations.append(f"{rid}: never ended (state {state.get(rid)})")
    for t, (e, d) in enumerate(zip(d_engs, decs)):
        out.violations += [f"tier {t}: {v}" for v in e.violations]
        if d.seats:
            out.violations.append(f"tier {t}: seats left behind: {sorted(d.seats)}")
        if e.pool.free_pages != e.pool.total_pages:
            out.violations.append(f"tier {t}: {e.pool.total_pages - e.pool.free_pages} pages leaked")
    out.violations += [f"head: {v}" for v in p_eng.violations]
    if p_eng.pool.free_pages != p_eng.pool.total_pages:
        out.violations.append("head: pages leaked")
    return out
