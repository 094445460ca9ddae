"""Data-parallel tier: one pool, one prefix cache and one batch per replica (a rank, or a tensor-parallel group of
ranks), stepped in lockstep through one fan-out. A request is placed where the longest cached prefix of its prompt
lives, unless that replica's backlog is more than PATIENCE requests above the least loaded one; ties go to the
least backlog. An idle replica simply gets no order that step.
Reference counterpart: crates/kern-serve/src/dp.rs:73-103 (placement), :254-338 (lockstep step), PATIENCE :48.
"""
from __future__ import annotations

from .ranks import GroupEngine, Ranks
from .scheduler import Request, Scheduler

PATIENCE = 8


class DpTier:
    def __init__(self, executors, protocol: dict, unit: int, tp: int = 1, chunk: int | None = None,
                 max_seqs: int | None = None, prefix_cache: bool = True, patience: int = PATIENCE):
        self.ex = executors
        self.ranks = Ranks(protocol, unit, executors.pages, executors.slots, tp)
        self.engines = [GroupEngine(executors, protocol, unit, tp, g, ranks=self.ranks) for g in range(self.ranks.groups.count)]
        self.scheds = [Scheduler(e, chunk=chunk, max_seqs=max_seqs, prefix_cache=prefix_cache) for e in self.engines]
        self.patience = patience
        self.placed: dict[str, int] = {}

    # ---- placement ----
    def backlog(self, g: int) -> int:
        s = self.scheds[g]
        return len(s.waiting) + len(s.running)

    def place(self, req: Request) -> int:
        loads = [self.backlog(g) for g in range(len(self.scheds))]
        least = min(range(len(loads)), key=lambda g: (loads[g], g))
        best, best_hit = least, 0
        if len(req.prompt) > 1:
            for g, s in enumerate(self.scheds):
                if s.prefix is None:
                    continue
                hit = s.prefix.lookup(req.prompt, len(req.prompt) - 1)
                n = hit[0] if hit else 0
                if n > best_hit or (n == best_hit and n > 0 and loads[g] < loads[best]):
                    best, best_hit = g, n
        if best_hit and loads[best] - loads[least] > self.patience:
            best = least                      # the cache hit is not worth the queue
        return best

    def submit(self, req: Request) -> int:
        g = self.place(req)
        self.scheds[g].submit(req)
        self.placed[req.id] = g
        return g

    def abort(self, req_id: str) -> bool:
        g = self.placed.get(req_id)
        return g is not None and self.scheds[g].abort(req_id)

    def idle(self) -> bool:
        return all(s.idle() for s in self.scheds)

    # ---- one lockstep step over every replica ----
    def step(self):
        plans = [s.plan() for s in self.scheds]
        staged = {g: self.ranks.stage(g, p["batch"], p["pad"], p["round"]) for g, p in enumerate(plans) if p is not None}
        if not staged and not any(self.ranks.acts):
            return []
        answers = self.ex.run(self.ranks.orders(list(staged.values())))
        out = []
        for g, st in staged.items():
            toks = st.emitted([answers[q] for q in self.ranks.groups.members(g)])
            st.commit()
            out += self.scheds[g].finish(plans[g], toks)
        return out

    def metrics(self) -> dict:
        ms = [s.metrics() for s in self.scheds]
        tot = lambda k: sum(m[k] for m in ms)
        return {"replicas": ms, "num_running_reqs": tot("num_running_reqs"), "num_waiting_reqs": tot("num_waiting_reqs"),
                "kv_used_blocks": tot("kv_used_blocks"), "kv_total_blocks": tot("kv_total_blocks"),
                "spec_decode": {k: sum(m["spec_decode"][k] for m in ms) for k in ("accepted", "proposed")},
                "prefix_cache": {k: sum(m["prefix_cache"][k] for m in ms) for k in ("queries", "hits", "hit_tokens", "entries")}}

    @property
    def stats(self):
        """The replicas' counters summed (what the metrics endpoint reports for the tier)."""
        import dataclasses

        from .scheduler import Stats

        out = Stats()
        for s in self.scheds:
            for f in dataclasses.fields(Stats):
                setattr(out, f.name, getattr(out, f.name) + getattr(s.stats, f.name))
        return out
