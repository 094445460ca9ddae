"""Deterministic simulation of the serving loop: no runtime, no GPU, no clock — a model engine whose "device" is a
table of what every KV slot and state slot holds, answering with the exact integer model's arithmetic. A seeded
driver feeds the real scheduler arrivals, aborts and tight pools; after every step the simulator checks the
invariants a serving loop must keep: every emitted token is the twin's, no page or slot is owned twice, nothing leaks,
a sequence only ever reads slots it wrote (or inherited through a kept prefix).
Reference counterpart: crates/kern-serve/tests/sim.rs (seeded schedules against a model pool).
"""
from __future__ import annotations

import random
from dataclasses import dataclass, field

from .. import _native, fills
from ..models import toy_int


class SimEngine:
    """The engine interface over a dictionary 'device'. page -> list of (token, position) per offset; slot -> carry."""

    def __init__(self, unit: int = 16, pages: int = 64, slots: int = 0, rows_max: int = 128, groups_max: int = 8,
                 max_context: int = 1024):
        self.unit, self.rows_max, self.groups_max = unit, rows_max, groups_max
        self.pool = _native.Pool(unit, pages, slots, -(-max_context // unit))
        self.mem: dict[int, dict[int, tuple[int, int]]] = {}
        self.carry: dict[int, int] = {}
        self.lined = slots > 0
        self.forwards = [{"name": "prefill", "rows": "var", "groups": groups_max, "emits": "next", "count": None, "graph": False},
                         {"name": "decode", "rows": 1, "groups": groups_max, "emits": "next", "count": None, "graph": True}]
        self.page_tables = [{"name": "block_table", "width": -(-max_context // unit), "stride": unit, "state": "kv"}]
        self.rt = self
        self.steps = 0
        self.violations: list[str] = []

    # runtime-side acts
    def run_copies(self, copies: dict) -> None:
        for a, b in copies["pages"]:
            self.mem[b] = dict(self.mem.get(a, {}))
        if copies["slot"] is not None:
            a, b = copies["slot"]
            self.carry[b] = self.carry.get(a, 0)

    def zero_slot(self, slot: int) -> None:
        self.carry[slot] = 0

    def open(self, tokens_capacity: int, sampling=None):
        from ..engine import Sequence

        lease = self.pool.lease(tokens_capacity)
        if lease.slot >= 0:
            self.zero_slot(lease.slot)
        return Sequence(lease=lease, sampling=sampling or fills.Sampling())

    def close(self, seq) -> None:
        seq.lease.release()

    def step(self, batch, eager=False, read=True, timed=False, pad=0, round=False):
        if sum(len(t) for _, t in batch) > self.rows_max or len(batch) + pad > self.groups_max:
            raise ValueError("call exceeds the model's limits")
        out = []
        for seq, new in batch:
            pages = seq.lease.pages
            for j, t in enumerate(new):
                p = seq.length + j
                slot = seq.lease.slot_of(p)            # raises if the page is frozen: only a lease writes, only its own
                self.mem.setdefault(slot // self.unit, {})[slot % self.unit] = (t, p)
                if self.lined:
                    c = self.carry.get(seq.lease.slot, 0)
                    self.carry[seq.lease.slot] = toy_int.rotl(c, 11) ^ toy_int.mark(t, p, 0xFFFF)
            L = seq.length + len(new)
            s = 0
            for p in range(L):
                cell = self.mem.get(pages[p // self.unit], {}).get(p % self.unit)
                if cell is None or cell[1] != p:
                    self.violations.append(f"position {p} of a sequence reads a slot holding {cell}")
                    cell = (0, p)
                s = (s + toy_int.slot_sum(cell[0], p)) & toy_int.M
            if self.lined:
                s = (s + self.carry.get(seq.lease.slot, 0)) & toy_int.M
            out.append([toy_int.next_of(s)])
            seq.length = L
            seq.tokens.extend(new)
        self.steps += 1
        return out


@dataclass
class Outcome:
    seed: int
    requests: int = 0
    finished: int = 0
    aborted: int = 0
    steps: int = 0
    prefix_hits: int = 0
    evictions: int = 0
    violations: list[str] = field(default_factory=list)


def run(seed: int, lined: bool = False, requests: int = 40, pages: int = 24, max_seqs: int = 4, chunk: int = 48,
        max_steps: int = 5000) -> Outcome:
    """One seeded schedule: arrivals interleaved with steps, shared prefixes, a few aborts, a pool small enough to evict."""
    from ..serve.scheduler import Request, Scheduler

    rng = random.Random(seed)
    eng = SimEngine(pages=pages, slots=(max_seqs + 6) if lined else 0)
    sch = Scheduler(eng, chunk=chunk, max_seqs=max_seqs)
    out = Outcome(seed=seed, requests=requests)
    bases = [[rng.randrange(256) for _ in range(rng.randint(20, 120))] for _ in range(4)]
    pending, live, done = [], {}, []
    for i in range(requests):
        b = rng.choice(bases)
        prompt = b[: rng.randint(1, len(b))] + [rng.randrange(256) for _ in range(rng.randint(0, 6))]
        pending.append(Request(id=f"r{i}", prompt=prompt, max_tokens=rng.randint(1, 12), stop_ids=(toy_int.EOS,)))
    while (pending or not sch.idle()) and out.steps < max_steps:
        for _ in range(rng.randint(0, 2)):
            if pending:
                r = pending.pop()
                if sch.pool.pages_for(len(r.prompt) + r.max_tokens) <= sch.pool.total_pages:
                    sch.submit(r)
                    live[r.id] = r
        if live and rng.random() < 0.03:
            rid = rng.choice(list(live))
            if sch.abort(rid):
                out.aborted += 1
                live.pop(rid)
        sch.step()
        out.steps += 1
        for rid in [k for k, r in live.items() if r.finished]:
            r = live.pop(rid)
            want = toy_int.generate(r.prompt, r.max_tokens, lined)
            got = [t for t in r.out if t != toy_int.EOS]
            if got != want:
                out.violations.append(f"{rid}: emitted {got}, the model says {want}")
            out.finished += 1
    if pending or not sch.idle():
        out.violations.append("the schedule did not drain")
    out.violations += eng.violations
    out.prefix_hits, out.evictions = sch.stats.prefix_hits, sch.stats.evictions
    # nothing leaks: once the prefix cache lets go, the pool is whole again
    while sch.prefix is not None and len(sch.prefix):
        sch.prefix.evict()
    if eng.pool.free_pages != eng.pool.total_pages:
        out.violations.append(f"{eng.pool.total_pages - eng.pool.free_pages} pages leaked")
    return out
