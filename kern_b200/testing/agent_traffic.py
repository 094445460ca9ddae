"""Agent-style traffic and its replay against a scheduler.

A session is a long shared prefix (a system prompt plus tool descriptions: one of a few `families`, so sessions of a
family share their first tokens) followed by turns; every turn's request is the whole conversation so far — the prefix,
the earlier suffixes and the earlier answers — plus a new suffix, so most of a request's prompt has been seen before
(by the session's previous turn, and its prefix by other sessions). A closed loop keeps `sessions` conversations going:
when a turn's answer is complete the session's next turn is submitted, until every session has had its turns.

    generate(...)   the sessions: prefix, per-turn suffix and answer budget, all from one seed (splitmix64)
    replay(...)     drive a `Scheduler` with them; returns requests served, output tokens per second, TTFT / ITL
                    percentiles and the share of prompt tokens that came out of the prefix cache

Reference shape: crates/kern-run/examples/agentx_replay.rs (a recorded agent trace replayed against the engine),
docs/serve.md:213-216 (prefix-cache effect), docs/vllm-rsi-example.md:233-239 (the metric set).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

from .abtest import Rng


@dataclass
class Turn:
    suffix: list[int]
    max_tokens: int


@dataclass
class Session:
    id: int
    family: int
    prefix: list[int]
    turns: list[Turn]
    history: list[int] = field(default_factory=list)     # the conversation so far (prefix + suffixes + answers)
    at: int = 0                                          # next turn


def generate(seed: int, sessions: int, turns: int, prefix: tuple[int, int], suffix: tuple[int, int], output: tuple[int, int],
             vocab: int, families: int = 4, shared: float = 0.5) -> list[Session]:
    """`prefix`, `suffix`, `output`: (low, high) token counts, uniform. The first `shared` part of a session's prefix is
    its family's (identical across the family's sessions), the rest its own."""
    rng = Rng(seed)
    span = lambda lo_hi: lo_hi[0] + rng.below(max(1, lo_hi[1] - lo_hi[0] + 1))
    tok = lambda n: [1 + rng.below(vocab - 1) for _ in range(n)]
    fam = [tok(prefix[1]) for _ in range(families)]
    out = []
    for i in range(sessions):
        f = i % families
        n = span(prefix)
        k = int(n * shared)
        out.append(Session(id=i, family=f, prefix=fam[f][:k] + tok(n - k),
                           turns=[Turn(tok(span(suffix)), span(output)) for _ in range(turns)]))
    return out


def _pct(xs: list[float], q: float) -> float | None:
    if not xs:
        return None
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(q * len(xs)))]


def replay(sched, sessions: list[Session], concurrent: int | None = None, deadline_s: float = 600.0, clock=time.monotonic) -> dict:
    """Closed loop: at most `concurrent` sessions have a request in flight; a finished turn's answer joins the
    session's history and its next turn is submitted at once. Returns the figures of the whole run."""
    from ..serve.scheduler import Request

    waiting = list(sessions)
    live: dict[str, Session] = {}
    reqs: dict[str, Request] = {}
    concurrent = concurrent or len(sessions)
    served, out_tokens, prompt_tokens, cached_tokens = 0, 0, 0, 0
    ttft, itl = [], []
    t0 = clock()

    def submit(s: Session) -> None:
        turn = s.turns[s.at]
        if not s.history:
            s.history = list(s.prefix)
        boundary = len(s.history)                          # the turn boundary a stateful model snapshots at
        prompt = s.history + turn.suffix
        r = Request(id=f"s{s.id}.t{s.at}", prompt=prompt, max_tokens=turn.max_tokens, history_tokens=boundary)
        r.arrival = clock()
        live[r.id], reqs[r.id] = s, r
        sched.submit(r)

    while (waiting or live) and clock() - t0 < deadline_s:
        while waiting and len(live) < concurrent:
            submit(waiting.pop(0))
        for r, _ in sched.step():
            if r.finished is None or r.id not in live:
                continue
            s = live.pop(r.id)
            served += 1
            out_tokens += len(r.out)
            prompt_tokens += len(r.prompt)
            cached_tokens += r.cached
            if r.first_token_at is not None:
                ttft.append(r.first_token_at - r.arrival)
            itl += [b - a for a, b in zip(r.token_times, r.token_times[1:])]
            s.history = r.prompt + r.out
            s.at += 1
            if s.at < len(s.turns):
                waiting.insert(0, s)                       # the session's next turn goes first: its context is warm
    wall = clock() - t0
    return {"requests_served": served, "sessions": len(sessions), "wall_s": wall, "output_tokens": out_tokens,
            "output_tok_s": out_tokens / wall if wall > 0 else 0.0, "prompt_tokens": prompt_tokens,
            "prefix_cache_share": cached_tokens / prompt_tokens if prompt_tokens else 0.0,
            "ttft_ms_p50": None if not ttft else 1e3 * _pct(ttft, 0.5), "ttft_ms_p90": None if not ttft else 1e3 * _pct(ttft, 0.9),
            "itl_ms_p50": None if not itl else 1e3 * _pct(itl, 0.5), "itl_ms_p90": None if not itl else 1e3 * _pct(itl, 0.9),
            "unfinished": len(live) + sum(1 for s in waiting if s.at < len(s.turns))}
