"""Continuous batching over one engine (one rank, or the head's view of a rank group).

Each `step()`:
  1. admits waiting requests while the pool can hold their worst case (prompt + max_tokens): a prefix
     lookup first — a hit restores the kept pages (whole pages shared, a half page and the state slot
     copied) and only the rest of the prompt is computed; when the pool is full, kept prefixes are
     evicted until the request fits or nothing is left to evict;
  2. builds one call: prompt rows of the admitted / still-prefilling requests up to the chunk budget
     (prefill first), plus one decode row (or one speculative round) for every running request;
     a pure-decode call is padded up to a bucket so captured graphs are reused;
  3. hands tokens back, finishes requests (stop token, length), and keeps their prefix: pure-KV models at
     the last page boundary, stateful models at the exact end (`retire`, no copy).

Reference: crates/kern-serve/src/scheduler.rs:122 (buckets), :552-861 (admit), :867-967 (keep / finish),
:985-1062 (prefill / step), :1067-1116 (stats line).
"""
from __future__ import annotations

import logging
import time
from collections import deque
from dataclasses import dataclass, field

from .. import _native
from ..engine import Engine, Sampling, Sequence

log = logging.getLogger("kern.scheduler")

BUCKETS = [1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512, 640, 768, 1024]


def bucket_for(n: int, limit: int) -> int:
    for b in BUCKETS:
        if n <= b <= limit:
            return b
    return min(max(n, 1), limit)


@dataclass
class Request:
    id: str
    prompt: list[int]
    max_tokens: int = 16
    sampling: Sampling = field(default_factory=Sampling)
    stop_ids: tuple[int, ...] = ()
    history_tokens: int | None = None     # prompt length up to the last turn boundary (where a stateful model snapshots)
    arrival: float = field(default_factory=time.monotonic)
    # filled by the scheduler
    seq: Sequence | None = None
    fed: int = 0                # prompt tokens already in the states
    cached: int = 0             # of which came from the prefix cache
    out: list[int] = field(default_factory=list)
    first_token_at: float | None = None
    finished: str | None = None  # "stop" | "length" | "abort"
    token_times: list[float] = field(default_factory=list)


@dataclass
class Stats:
    steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    prefix_hits: int = 0
    prefix_hit_tokens: int = 0
    prefix_queries: int = 0
    pooled_hit_tokens: int = 0
    evictions: int = 0
    accepted: int = 0
    proposed: int = 0
    step_seconds: float = 0.0
    denied: int = 0


class Scheduler:
    def __init__(self, engine: Engine, chunk: int | None = None, max_seqs: int | None = None, prefix_cache: bool = True,
                 rows: int | None = None, stats_every: float = 5.0, pooled=None):
        """`pooled`: a `PooledCache` (a tier shared with other engines, or an SSD arena) consulted after the local
        prefix cache at admission and fed when requests finish."""
        self.eng = engine
        self.pooled = pooled
        self.pool = engine.pool
        self.chunk = min(chunk or engine.rows_max, engine.rows_max)
        row_shapes = sorted(f["rows"] for f in engine.forwards if f["rows"] != "var")
        self.rows = rows if rows is not None else (row_shapes[-1] if row_shapes else 1)   # widest declared round
        self.round = next((f for f in engine.forwards if f["rows"] == self.rows and self.rows > 1), None)
        step_groups = max((f["groups"] for f in engine.forwards if f["rows"] != "var"), default=engine.groups_max)
        self.max_seqs = min(max_seqs or step_groups, engine.groups_max)
        # The ragged (prefill) program of a package may take fewer sequences per call than a step does (one, in packages
        # whose prefill is a per-sequence program), and may emit nothing (the prompt's last token is then fed by the
        # first step, as the reference's paged packages do: tools/toy/gen.py:107-113, crates/kern-serve/src/scheduler.rs:985-1062).
        ragged = next((f for f in engine.forwards if f["rows"] == "var"), None)
        self.ragged_groups = ragged["groups"] if ragged else 0
        self.prefill_emits = ragged is None or ragged["emits"] is not None
        self.split = ragged is not None and self.ragged_groups < self.max_seqs
        self.prefix = _native.Prefix(self.pool.unit) if prefix_cache else None
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.done: list[Request] = []
        self.stats = Stats()
        self._last_stats = time.monotonic()
        self._stats_every = stats_every
        self._last_counts = (0, 0)
        self.on_finish = None        # called with a finished request while its lease is still held (a hand-over to another tier)

    # ---- the three calls of the Scheduler interface: submit / step / metrics ----
    def submit(self, req: Request) -> None:
        need = len(req.prompt) + req.max_tokens
        if self.pool.pages_for(need) > self.pool.total_pages:
            req.finished = "abort"
            self.done.append(req)
            raise ValueError(f"request {req.id} needs {need} tokens, more than the pool holds")
        self.waiting.append(req)

    def abort(self, req_id: str) -> bool:
        for q in (self.waiting, self.running):
            for r in list(q):
                if r.id == req_id:
                    q.remove(r)
                    if r.seq is not None:
                        self.eng.close(r.seq)
                        r.seq = None
                    r.finished = "abort"
                    self.done.append(r)
                    return True
        return False

    def idle(self) -> bool:
        return not self.waiting and not self.running

    def metrics(self) -> dict:
        p = self.pool
        return {"kv_used_blocks": p.total_pages - p.free_pages, "kv_total_blocks": p.total_pages,
                "num_running_reqs": len(self.running), "num_waiting_reqs": len(self.waiting),
                "spec_decode": {"accepted": self.stats.accepted, "proposed": self.stats.proposed},
                "prefix_cache": {"queries": self.stats.prefix_queries, "hits": self.stats.prefix_hits,
                                 "hit_tokens": self.stats.prefix_hit_tokens, "entries": len(self.prefix) if self.prefix is not None else 0}}

    # ---- admission ----
    def _make_room(self, pages: int, slot: bool) -> bool:
        """Evict kept prefixes until the ask fits; allocation and 'is there room' stay one action: the caller
        retries the lease itself."""
        while not self.pool.room(pages, slot):
            if self.prefix is None or len(self.prefix) == 0:
                return False
            self.prefix.evict()
            self.stats.evictions += 1
        return True

    def _admit_one(self, req: Request) -> bool:
        need = len(req.prompt) + req.max_tokens + (self.rows if self.round else 0)
        hit = None
        if self.prefix is not None and len(req.prompt) > 1:
            self.stats.prefix_queries += 1
            # at least one prompt token must be computed so the call has a row to emit from
            hit = self.prefix.lookup(req.prompt, len(req.prompt) - 1)
        for attempt in range(2):
            try:
                if hit is not None:
                    length, ckpt = hit
                    lease, copies = self.pool.restore(ckpt, length, need)
                    self.eng.rt.run_copies(copies)
                    if lease.slot >= 0 and copies["slot"] is None:
                        self.eng.rt.zero_slot(lease.slot)
                    req.seq = Sequence(lease=lease, length=length, sampling=req.sampling, tokens=list(req.prompt[:length]))
                    req.fed = req.cached = length
                    self.stats.prefix_hits += 1
                    self.stats.prefix_hit_tokens += length
                else:
                    req.seq = self.eng.open(need, req.sampling)
                if self.pooled is not None and len(req.prompt) > 1:
                    have = req.seq.length
                    got = self.pooled.fetch(req.prompt, have, list(req.seq.lease.pages), len(req.prompt) - 1)
                    if got > have:
                        req.seq.length = got
                        req.seq.tokens = list(req.prompt[:got])
                        req.fed = req.cached = got
                        self.stats.pooled_hit_tokens += got - have
                return True
            except _native.Denied as e:
                why = e.args[1] if len(e.args) > 1 else "busy"
                if why != "busy" or attempt == 1:
                    self.stats.denied += 1
                    return False
                shared = (hit[0] // self.pool.unit) if hit is not None else 0
                if not self._make_room(self.pool.pages_for(need) - shared, True):
                    self.stats.denied += 1
                    return False
        return False

    def _admit(self) -> None:
        while self.waiting and len(self.running) < self.max_seqs:
            if not self._admit_one(self.waiting[0]):
                break
            self.running.append(self.waiting.popleft())

    # ---- keeping prefixes ----
    def _keep(self, req: Request) -> None:
        """A finished request leaves its tokens' state behind for the next turn of the conversation."""
        seq = req.seq
        req.seq = None
        if seq is None:
            return
        if self.prefix is None or seq.length < 1:
            self.eng.close(seq)
            return
        tokens = seq.tokens[:seq.length]
        stateful = seq.lease.slot >= 0
        # pure KV: keep whole pages only (usable at any page boundary, nothing to copy);
        # stateful: the state is "exactly after these tokens", kept at the exact end by retiring the lease
        length = seq.length if stateful else (seq.length // self.pool.unit) * self.pool.unit
        if length == 0:
            self.eng.close(seq)
            return
        if self.pooled is not None and not stateful:
            self.pooled.put(tokens[:length], list(seq.lease.pages))
        ckpt = self.pool.retire(seq.lease, length)
        self.prefix.insert(tokens, ckpt, stateful, length)

    def _snapshot(self, req: Request) -> None:
        """Keep the states of a running request at its turn boundary: whole pages join the shared chain, the half page
        and the state slot are copied to the checkpoint (`Pool.checkpoint`); the request goes on with its lease. A
        later prompt that shares the history restores from here — a checkpoint that holds a slot is usable at its
        exact length only, so without this a stateful model would hit the cache only at the very end of a sequence."""
        try:
            ckpt, copies = self.pool.checkpoint(req.seq.lease, req.fed)
        except _native.Denied:
            return                                  # no room for the copy: go on without a snapshot
        self.eng.rt.run_copies(copies)
        self.prefix.insert(req.prompt[:req.fed], ckpt, True, req.fed)

    def _finish(self, req: Request, why: str, keep: bool = True) -> None:
        req.finished = why
        self.running.remove(req)
        if self.on_finish is not None and req.seq is not None:
            self.on_finish(req)
        if keep:
            self._keep(req)
        elif req.seq is not None:
            self.eng.close(req.seq)
            req.seq = None
        self.done.append(req)

    # ---- one step ----
    def _target(self, r: Request) -> int:
        """Prompt tokens the ragged program is fed: all of them, or all but the last when it emits nothing."""
        return len(r.prompt) - (0 if self.prefill_emits else 1)

    def step(self) -> list[tuple[Request, list[int]]]:
        """Run one step (one call; several when the ragged program takes fewer sequences than the step holds);
        returns (request, new tokens) for every request that produced tokens."""
        plan = self.plan()
        if plan is None:
            return []
        for pre in plan.get("pre", []):
            pre["toks"] = self.eng.step(pre["batch"], read=self._emits(pre["kinds"]))
        return self.finish(plan, self.eng.step(plan["batch"], pad=plan["pad"], round=plan["round"], read=self._emits(plan["kinds"])))

    def _emits(self, kinds) -> bool:
        """Whether any token of this call is wanted: a decode row, or a chunk that completes its prompt. A call of
        unfinished chunks only is issued without reading anything back, so the next chunk (or a pipeline's next item)
        follows it without a host round trip."""
        return any(kind != "prefill" or (self.prefill_emits and r.fed + n >= self._target(r)) for r, kind, n in kinds)

    def plan(self) -> dict | None:
        """Admit, then decide this step's call: {batch, kinds, pad, round}. None when there is nothing to run.
        A tier that runs several schedulers in lockstep plans each, issues all calls at once, then finishes each."""
        t0 = time.monotonic()
        self._admit()
        if not self.running:
            return None
        batch, kinds = [], []
        budget = self.chunk
        decoding = [r for r in self.running if r.fed >= self._target(r)]
        prefilling = [r for r in self.running if r.fed < self._target(r)]
        rows_decode = self.rows if self.round else 1
        if not self.split:
            budget -= len(decoding) * rows_decode
        pre: list[dict] = []
        for r in prefilling:                       # prefill first: oldest request gets the budget
            if budget <= 0:
                break
            n = min(budget, self._target(r) - r.fed)
            h = r.history_tokens
            if h is not None and r.seq.lease.slot >= 0 and r.fed < h < len(r.prompt):
                n = min(n, h - r.fed)      # a chunk ends at the turn boundary, where the per-sequence state is snapshotted
            if self.split:
                # calls of their own, as many sequences each as the ragged program takes
                if not pre or len(pre[-1]["batch"]) >= self.ragged_groups or \
                        sum(k[2] for k in pre[-1]["kinds"]) + n > self.eng.rows_max:
                    pre.append({"batch": [], "kinds": []})
                pre[-1]["batch"].append((r.seq, r.prompt[r.fed:r.fed + n]))
                pre[-1]["kinds"].append((r, "prefill", n))
            else:
                batch.append((r.seq, r.prompt[r.fed:r.fed + n]))
                kinds.append((r, "prefill", n))
            budget -= n
        use_round = self.round is not None and not batch and bool(decoding)     # a round is a fixed-shape call of its own
        for r in decoding:
            last = r.out[-1] if r.out else r.prompt[-1]       # a prefill that emits nothing leaves the last prompt token to the step
            batch.append((r.seq, [last] * (self.rows if use_round else 1)))
            kinds.append((r, "decode", 1))
        if not batch and pre:
            last_pre = pre.pop()                   # nothing decodes yet: the last ragged call is the step's main call
            batch, kinds = last_pre["batch"], last_pre["kinds"]
        if not batch:
            return None
        pad = 0
        if not any(k[1] == "prefill" for k in kinds):
            # fixed-shape call: pad to a bucket with dead rows so captured graphs are reused
            want = bucket_for(len(batch), self.max_seqs)
            pad = want - len(batch)
        return {"batch": batch, "kinds": kinds, "pad": pad, "round": use_round, "t0": t0, "pre": pre}

    def finish(self, plan: dict, toks) -> list[tuple[Request, list[int]]]:
        """Account for the tokens the planned call emitted."""
        kinds, use_round, t0 = list(plan["kinds"]), plan["round"], plan["t0"]
        toks = list(toks or [[]] * len(kinds))
        for pre in reversed(plan.get("pre", [])):          # the ragged calls that ran before the main one
            kinds = list(pre["kinds"]) + kinds
            toks = list(pre.get("toks") or [[]] * len(pre["kinds"])) + toks
        now = time.monotonic()
        emitted = []
        for (r, kind, n), got in zip(kinds, toks):
            if kind == "prefill":
                r.fed += n
                self.stats.prefill_tokens += n
                if r.fed < self._target(r):
                    if self.prefix is not None and r.history_tokens == r.fed and r.seq.lease.slot >= 0:
                        self._snapshot(r)          # a stateful model's state exactly after the previous turns
                    continue                       # the chunk's emitted token is not the prompt's next token yet
                if not self.prefill_emits:
                    continue                       # the first step feeds the prompt's last token and emits
                new = got[:1]
            else:
                new = got
                self.stats.decode_tokens += len(new)
                if use_round:
                    self.stats.proposed += self.rows - 1
                    self.stats.accepted += max(0, len(new) - 1)
            if r.first_token_at is None and new:
                r.first_token_at = now
            taken, why = [], None
            for t in new:
                r.out.append(int(t))
                r.token_times.append(now)
                taken.append(int(t))
                if int(t) in r.stop_ids:
                    why = "stop"
                    break
                if len(r.out) >= r.max_tokens:
                    why = "length"
                    break
            keepable = True
            if use_round and kind == "decode" and r.seq is not None:
                # A round fed `rows` positions holding [last, d1 .. d(rows-1)]; the engine recorded placeholders. Only the
                # positions of the tokens taken stay (paged KV slot = position: no copy), and the history must name what
                # those positions really hold, [last] + taken[:-1], before anything is kept under it as a prefix key.
                old_len = r.seq.length - self.rows
                last = r.seq.tokens[old_len]
                r.seq.length = old_len + len(taken)
                r.seq.tokens[old_len:] = [last] + taken[:-1]
                # a per-sequence recurrent state was advanced by the kernels over every accepted position: when the
                # request stops short of them, the slot is ahead of `length` and cannot be kept as a checkpoint
                keepable = not (r.seq.lease.slot >= 0 and len(taken) < len(new))
            if why is not None:
                self._finish(r, why, keep=keepable)
            emitted.append((r, taken))
        self.stats.steps += 1
        self.stats.step_seconds += time.monotonic() - t0
        self._maybe_log()
        return emitted

    def run_until_idle(self, max_steps: int = 1 << 30) -> None:
        n = 0
        while not self.idle() and n < max_steps:
            self.step()
            n += 1

    def _maybe_log(self) -> None:
        now = time.monotonic()
        if now - self._last_stats < self._stats_every:
            return
        s = self.stats
        dt = now - self._last_stats
        steps = s.steps - self._last_counts[0]
        toks = s.decode_tokens - self._last_counts[1]
        p = self.pool
        log.info("stats running=%d waiting=%d kv=%.1f%% steps=%d step_ms=%.2f tok_s=%.1f accept=%.1f%% prefix_hits=%d evictions=%d",
                 len(self.running), len(self.waiting), 100.0 * (p.total_pages - p.free_pages) / max(1, p.total_pages), steps,
                 1e3 * s.step_seconds / max(1, s.steps), toks / dt, 100.0 * s.accepted / max(1, s.proposed), s.prefix_hits, s.evictions)
        self._last_stats = now
        self._last_counts = (s.steps, s.decode_tokens)
