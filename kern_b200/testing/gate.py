"""The serving gate: named scenarios that every model target must pass, each an exact statement — a request served
in a batch, in chunks, after a prefix hit, under pool pressure or next to an aborted neighbour produces the tokens the
same request produces alone.

    python -m kern_b200 gate --model toy --cpu            # one line per scenario; exit 0 only if all pass
    python -m kern_b200 gate --model tiny-hybrid --only repeat_hit,turn2

`make_engine(tokens)` returns a fresh engine (runtime + pool) with the given token capacity; greedy sampling throughout,
so a difference is a bug and not noise (on bf16 models near-ties may flip between batch shapes: a scenario then reports
the first differing position and how close the two logits were is left to `kern test`).
Reference: tools/e2e/e2e.py (scenarios `conc1_equals_run`, `rows1_equals_run`, `repeat_hit`, `turn2_*`, `concurrent`,
`abort` by a client that hangs up mid-stream, `slot_pressure`, `kept_nothing`, `spec_acceptance` / `rows1_vs_spec`),
tools/e2e/README.md.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from ..serve.scheduler import Request, Scheduler


@dataclass
class Result:
    name: str
    ok: bool
    detail: str = ""

    def line(self) -> str:
        return f"{'PASS' if self.ok else 'FAIL'} {self.name}" + (f"  {self.detail}" if self.detail else "")


class Gate:
    def __init__(self, make_engine, vocab: int, page: int, capacity: int, seed: int = 0, out_tokens: int = 6):
        self.make, self.vocab, self.page, self.capacity, self.n = make_engine, vocab, page, capacity, out_tokens
        self.rng = np.random.default_rng(seed)
        self._alone: dict[tuple, list[int]] = {}

    # ---- helpers ----
    def prompt(self, n: int) -> list[int]:
        return self.rng.integers(1, self.vocab, n).tolist()

    def alone(self, prompt: list[int], n: int | None = None) -> list[int]:
        key = (tuple(prompt), n or self.n)
        if key not in self._alone:
            self._alone[key] = self.make(self.capacity).generate(prompt, n or self.n)
        return self._alone[key]

    def serve(self, sched: Scheduler, reqs: list[Request], steps: int = 2000) -> None:
        for r in reqs:
            sched.submit(r)
        sched.run_until_idle(steps)

    @staticmethod
    def differ(got: list[int], want: list[int]) -> str:
        for i, (a, b) in enumerate(zip(got, want)):
            if a != b:
                return f"token {i}: {a} != {b}"
        return f"lengths {len(got)} != {len(want)}" if len(got) != len(want) else ""

    # ---- scenarios ----
    def conc1_equals_run(self) -> Result:
        """One request through the scheduler equals the plain generation loop."""
        p = self.prompt(2 * self.page + 5)
        r = Request(id="a", prompt=p, max_tokens=self.n)
        self.serve(Scheduler(self.make(self.capacity)), [r])
        d = self.differ(r.out, self.alone(p))
        return Result("conc1_equals_run", not d and r.finished == "length", d)

    def rows1_equals_run(self) -> Result:
        """The prompt fed one row per call equals the prompt fed whole."""
        p = self.prompt(self.page + 3)
        r = Request(id="a", prompt=p, max_tokens=self.n)
        self.serve(Scheduler(self.make(self.capacity), chunk=1), [r])
        d = self.differ(r.out, self.alone(p))
        return Result("rows1_equals_run", not d, d)

    def repeat_hit(self) -> Result:
        """The same prompt again: whole pages come from the prefix cache and the tokens do not change."""
        p = self.prompt(2 * self.page + 8)
        s = Scheduler(self.make(self.capacity))
        # a turn boundary inside the prompt: where a model with per-sequence state snapshots it (a checkpoint that
        # holds a state slot is usable at its exact length only)
        a = Request(id="a", prompt=p, max_tokens=self.n, history_tokens=2 * self.page)
        b = Request(id="b", prompt=p, max_tokens=self.n, history_tokens=2 * self.page)
        self.serve(s, [a])
        self.serve(s, [b])
        d = self.differ(a.out, self.alone(p)) or self.differ(b.out, self.alone(p))
        ok = not d and b.cached >= self.page and s.stats.prefix_hits >= 1
        return Result("repeat_hit", ok, d or f"cached {b.cached} of {len(p)}")

    def turn2(self) -> Result:
        """A second turn (first prompt + its answer + more): the shared prefix is reused, the tokens equal a cold run."""
        p = self.prompt(2 * self.page + 8)
        s = Scheduler(self.make(self.capacity))
        a = Request(id="a", prompt=p, max_tokens=self.n)
        self.serve(s, [a])
        p2 = p + a.out + self.prompt(7)
        c = Request(id="c", prompt=p2, max_tokens=self.n, history_tokens=len(p) + len(a.out))
        self.serve(s, [c])
        d = self.differ(c.out, self.alone(p2))
        return Result("turn2", not d and c.cached >= self.page, d or f"cached {c.cached} of {len(p2)}")

    def concurrent(self) -> Result:
        """Several requests of mixed lengths in flight, chunked prefill mixed with decode rows."""
        prompts = [self.prompt(n) for n in (5, self.page, self.page + 1, 2 * self.page - 2, 3)]
        reqs = [Request(id=f"r{i}", prompt=p, max_tokens=self.n) for i, p in enumerate(prompts)]
        self.serve(Scheduler(self.make(self.capacity), chunk=self.page + self.page // 2), reqs)
        for r, p in zip(reqs, prompts):
            d = self.differ(r.out, self.alone(p))
            if d:
                return Result("concurrent", False, f"{r.id}: {d}")
        return Result("concurrent", True, f"{len(reqs)} requests")

    def abort(self) -> Result:
        """Aborting one of two running requests returns its pages and leaves the other's tokens alone."""
        s = Scheduler(self.make(self.capacity), prefix_cache=False)
        pa, pb = self.prompt(self.page + 4), self.prompt(self.page + 9)
        a, b = Request(id="a", prompt=pa, max_tokens=self.n + 6), Request(id="b", prompt=pb, max_tokens=self.n)
        s.submit(a)
        s.submit(b)
        for _ in range(3):
            s.step()
        gone = s.abort("a")
        s.run_until_idle(2000)
        d = self.differ(b.out, self.alone(pb))
        ok = gone and a.finished == "abort" and not d and s.pool.free_pages == s.pool.total_pages
        return Result("abort", ok, d or f"free {s.pool.free_pages} of {s.pool.total_pages}")

    def slot_pressure(self) -> Result:
        """A pool too small for every request at once: requests wait or evict cached prefixes, all finish, tokens exact."""
        need = 2 * self.page + self.n + 2
        tokens = self.page * (2 * -(-need // self.page) + 1)           # room for two requests and a page to spare
        s = Scheduler(self.make(tokens))
        prompts = [self.prompt(2 * self.page - 3 + i) for i in range(5)]
        reqs = [Request(id=f"r{i}", prompt=p, max_tokens=self.n) for i, p in enumerate(prompts)]
        self.serve(s, reqs, steps=5000)
        for r, p in zip(reqs, prompts):
            if r.finished != "length":
                return Result("slot_pressure", False, f"{r.id} finished {r.finished}")
            d = self.differ(r.out, self.alone(p))
            if d:
                return Result("slot_pressure", False, f"{r.id}: {d}")
        return Result("slot_pressure", True, f"{len(reqs)} requests through {tokens // self.page} pages, {s.stats.evictions} evictions")

    def kept_nothing(self) -> Result:
        """After a mix of sessions, aborts and cache hits, letting go of every cached prefix leaves the pool as it
        started: every page and slot free (nothing leaked by a finished, aborted or evicted request)."""
        s = Scheduler(self.make(self.capacity))
        prompts = [self.prompt(self.page + 2 + 3 * i) for i in range(4)]
        reqs = [Request(id=f"r{i}", prompt=p, max_tokens=self.n) for i, p in enumerate(prompts)]
        for r in reqs:
            s.submit(r)
        for _ in range(2):
            s.step()
        s.abort("r1")
        s.run_until_idle(3000)
        again = Request(id="again", prompt=prompts[0], max_tokens=self.n)        # a hit on what r0 left behind
        self.serve(s, [again])
        total_pages, free_before = s.pool.total_pages, s.pool.free_pages
        if s.prefix is not None:
            while len(s.prefix):                                                 # whatever the cache still keeps goes
                s.prefix.evict()
        pad = int(getattr(s.eng, "pad_pages", 0))                                 # the engine's own page for padding rows
        ok = s.idle() and s.pool.free_pages == total_pages - pad
        return Result("kept_nothing", ok, f"free {s.pool.free_pages} of {total_pages} ({pad} held for padding rows; "
                                          f"before letting the cache go: {free_before})")

    def http_hang_up(self) -> Result:
        """A client that streams a few chunks and closes its connection: the request is aborted, its pages come back,
        and a request that shared the batch finishes with the tokens it has alone."""
        import http.client
        import json
        import time

        from ..serve.server import Server

        s = Scheduler(self.make(self.capacity), prefix_cache=False)
        srv = Server(s, model_name="gate", port=0).start()
        try:
            pa, pb = self.prompt(self.page + 4), self.prompt(self.page + 9)
            conn = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=60)
            conn.request("POST", "/v1/completions", json.dumps({"prompt": pa, "max_tokens": 6 * self.n, "stream": True, "ignore_eos": True}),
                         {"Content-Type": "application/json"})
            resp = conn.getresponse()
            got = 0
            while got < 2:                                   # two streamed chunks, then the client leaves
                line = resp.readline()
                if not line:
                    break
                got += line.startswith(b"data: {")
            resp.close()
            conn.close()
            other = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=60)
            other.request("POST", "/v1/completions", json.dumps({"prompt": pb, "max_tokens": self.n, "return_token_ids": True, "ignore_eos": True}),
                          {"Content-Type": "application/json"})
            body = json.loads(other.getresponse().read())
            other.close()
            d = self.differ(body["choices"][0]["token_ids"], self.alone(pb))
            deadline = time.monotonic() + 20
            while time.monotonic() < deadline and not (s.idle() and s.pool.free_pages == s.pool.total_pages):
                time.sleep(0.02)
            pad = int(getattr(s.eng, "pad_pages", 0))
            gone = any(r.id != body["id"] and r.finished == "abort" for r in s.done)      # the hung-up request was aborted, not served out
            ok = got == 2 and not d and gone and s.idle() and s.pool.free_pages == s.pool.total_pages - pad
            return Result("http_hang_up", ok, d or f"chunks read {got}, aborted {gone}, free {s.pool.free_pages} of {s.pool.total_pages} after the client left")
        finally:
            srv.stop()

    def spec_acceptance(self) -> Result:
        """A package with speculative rounds: the tokens of a round-by-round run equal the one-row-per-step run's
        (`rows1_vs_spec`), and a burst of concurrent requests keeps the acceptance rate of a single one within bounds."""
        eng = self.make(self.capacity)
        rounds = [f for f in eng.forwards if f["rows"] != "var" and f["rows"] > 1]
        if not rounds:
            return Result("spec_acceptance", True, "no round program in this package (skipped)")
        p = self.prompt(self.page + 6)
        s1 = Scheduler(eng)
        a = Request(id="a", prompt=p, max_tokens=4 * self.n)
        self.serve(s1, [a])
        base = s1.stats.accepted / max(1, s1.stats.proposed)
        plain = Scheduler(self.make(self.capacity), rows=1)
        b = Request(id="b", prompt=p, max_tokens=4 * self.n)
        self.serve(plain, [b])
        d = self.differ(a.out, b.out)
        s2 = Scheduler(self.make(self.capacity))
        burst = [Request(id=f"c{i}", prompt=self.prompt(self.page + i), max_tokens=4 * self.n) for i in range(3)] + \
                [Request(id="same", prompt=p, max_tokens=4 * self.n)]
        self.serve(s2, burst, steps=5000)
        rate = s2.stats.accepted / max(1, s2.stats.proposed)
        d = d or self.differ(burst[-1].out, a.out)
        ok = not d and s1.stats.proposed > 0 and all(r.finished == "length" for r in burst)
        return Result("spec_acceptance", ok, d or f"acceptance {base:.2f} alone, {rate:.2f} in a burst of {len(burst)}")

    SCENARIOS = ("conc1_equals_run", "rows1_equals_run", "repeat_hit", "turn2", "concurrent", "abort", "slot_pressure",
                 "kept_nothing", "http_hang_up", "spec_acceptance")

    def run(self, only: list[str] | None = None) -> list[Result]:
        out = []
        for name in self.SCENARIOS:
            if only and name not in only:
                continue
            try:
                out.append(getattr(self, name)())
            except Exception as e:          # a scenario that cannot even run is a failure with its reason
                out.append(Result(name, False, f"{type(e).__name__}: {e}"))
        return out
