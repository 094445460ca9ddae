"""A prefill tier's front: the head that prefills runs on a thread of its own, apart from the loop that answers clients.

The head waits on its device for as long as a step takes (a long prompt's chunk is tens of milliseconds). A head that
were also the loop the HTTP driver calls would hold every token of the process behind that wait — the decode tier's among
them — and clients would get them in bursts a step apart. So:

    head thread    owns the prefill scheduler and is the one writer to the decode tier: Reserve, the hand-over (push,
                   then Start), Abort. It takes Calls (submit / a message the decode tier sent about seats / abort /
                   gone) and writes Notes, in order, into the front's one channel.
    front (step)   reads the decode tier's connection: Tokens are applied at once, every other message goes to the head
                   as a Call. It applies the head's Notes as they come. `Clients` keeps who answers each client: the
                   head from submission until it finishes, rejects or hands the request over; the front after.

A hand-over's Notes — the first token, then Decode — are written before the head sends Start, so in the one channel a
request's decode tokens always come after them. A client that leaves is the front's to see: a decoding request is
retired at once and the head frees its seats (Call abort); the head is told once of any other (Call gone) and retires it
at its next touch.
Reference counterpart: crates/kern-serve/src/front.rs:1-30 (who answers a client), :47-135 (Note, Call, Write), :135-260
(Clients), pd/relay.rs.
"""
from __future__ import annotations

import logging
import queue
import threading
import time

from . import pd, wire
from .pd_serve import _drain
from .scheduler import Request, Scheduler

log = logging.getLogger("kern.serve")

WAIT = 0.001      # how long a step waits for a note before handing the driver back


class Clients:
    """Who answers each open request, as a pure state machine: Notes and decode Tokens in, Writes out.

    Notes (from the head, in order): ("admit", id, cached) | ("reject", id, why) | ("emit", id, tok) |
    ("finish", id, why) | ("decode", id). Decode tokens: `tokens(id, tok, last)`.
    Writes (for whoever holds the client's stream): ("token", id, tok) | ("finish", id, why).
    Calls (for the head): ("abort", id) for a decoding request whose client left or that stopped on a token only the
    front saw; ("gone", id) once for any other whose client left."""

    def __init__(self):
        self.state: dict[str, str] = {}          # id -> "head" | "decoding"
        self.told_gone: set[str] = set()

    def submit(self, rid: str) -> None:
        if rid in self.state:
            raise ValueError(f"request {rid} is already open")
        self.state[rid] = "head"

    def open(self) -> int:
        return len(self.state)

    def decoding(self) -> int:
        return sum(1 for s in self.state.values() if s == "decoding")

    def note(self, n: tuple) -> list[tuple]:
        kind, rid = n[0], n[1]
        st = self.state.get(rid)
        if st is None:
            return []                              # retired already (the client left, or a finish came first)
        if st != "head":
            raise RuntimeError(f"note {kind} for request {rid}, which the head handed over")
        if kind == "admit":
            return []
        if kind == "reject":
            self._retire(rid)
            return [("finish", rid, "abort")]
        if kind == "emit":
            return [("token", rid, n[2])]
        if kind == "finish":
            self._retire(rid)
            return [("finish", rid, n[2])]
        if kind == "decode":
            self.state[rid] = "decoding"
            return []
        raise ValueError(f"unknown note {kind!r}")

    def tokens(self, rid: str, tok: int, last: bool, why: str = "length") -> list[tuple]:
        """One token of a decode step. Tokens of a request that is not decoding (retired here first) are dropped."""
        if self.state.get(rid) != "decoding":
            return []
        out = [("token", rid, tok)]
        if last:
            self._retire(rid)
            out.append(("finish", rid, why))
        return out

    def sweep(self, left) -> tuple[list[tuple], list[tuple]]:
        """`left(id)`: whether the request's client is gone. -> (writes, calls for the head)."""
        writes, calls = [], []
        for rid, st in list(self.state.items()):
            if not left(rid):
                continue
            if st == "decoding":
                self._retire(rid)
                writes.append(("finish", rid, "abort"))
                calls.append(("abort", rid))
            elif rid not in self.told_gone:
                self.told_gone.add(rid)
                calls.append(("gone", rid))
        return writes, calls

    def _retire(self, rid: str) -> None:
        self.state.pop(rid, None)
        self.told_gone.discard(rid)


class Front:
    """The scheduler-like face of a prefill tier with a decode tier behind it (submit / step / idle / abort / metrics /
    stats), with the prefill scheduler on a head thread. Built by `pd_serve.connect_tiers(front=True)`."""

    def __init__(self, sched: Scheduler, rt, sock, mapped, mirrors=None, dealer=None):
        self.sched, self.rt, self.sock, self.mapped = sched, rt, sock, mapped
        self.mirrors, self.dealer = mirrors, dealer
        self.hand = pd.Handoffs(sched.pool.unit)          # the head's
        self.clients = Clients()                          # the front's
        self.users: dict[str, Request] = {}               # every open request, by id (the front's)
        self.left: set[str] = set()                       # clients that went away (abort was called)
        self.notes: queue.Queue = queue.Queue()           # head -> front (decode tokens are applied by the front itself)
        self.calls: queue.Queue = queue.Queue()           # front -> head
        self.stats, self.pool = sched.stats, sched.pool
        self.done: list[Request] = []
        self.decode_load: dict = {}
        self.failed: str | None = None
        self._halt = threading.Event()
        # the head's own books
        self._asking: dict[str, Request] = {}
        self._prefilling: dict[str, Request] = {}
        self._handed: set[str] = set()
        sched.on_finish = self._hand_over
        self.head = threading.Thread(target=self._head_main, daemon=True, name="kern-prefill-head")
        self.head.start()

    # ---- the front: the scheduler interface, on the driver's thread ----
    def submit(self, req: Request) -> None:
        need = len(req.prompt) + req.max_tokens
        if self.pool.pages_for(need) > self.pool.total_pages:
            req.finished = "abort"
            self.done.append(req)
            raise ValueError(f"request {req.id} needs {need} tokens, more than the prefill pool holds")
        self.clients.submit(req.id)
        self.users[req.id] = req
        self.calls.put(("submit", req))

    def abort(self, req_id: str) -> bool:
        if req_id not in self.users:
            return False
        self.left.add(req_id)
        return True

    def idle(self) -> bool:
        return self.clients.open() == 0

    def metrics(self) -> dict:
        m = self.sched.metrics()
        m["pd"] = {"open": self.clients.open(), "decoding": self.clients.decoding(), "decode_tier": self.decode_load}
        return m

    def _apply(self, writes: list[tuple], emitted: list, now: float) -> None:
        for w in writes:
            user = self.users.get(w[1])
            if user is None:
                continue
            if w[0] == "token":
                if user.first_token_at is None:
                    user.first_token_at = now
                user.out.append(int(w[2]))
                user.token_times.append(now)
                emitted.append((user, [int(w[2])]))
            else:
                user.finished = w[2]
                self.users.pop(w[1], None)
                self.left.discard(w[1])
                self.done.append(user)
                if w[2] == "abort" or not user.out:
                    emitted.append((user, []))

    def step(self) -> list[tuple[Request, list[int]]]:
        if self.failed:
            raise RuntimeError(f"the prefill head failed: {self.failed}")
        emitted: list = []
        # The decode tier's frames are read first and applied last: a hand-over's notes were in the channel before its
        # Start left, so every note that precedes a token read here is drained below before the token is applied.
        msgs = _drain(self.sock, 0.0)
        if msgs is None:
            raise ConnectionError("the decode tier closed its connection")
        got = False
        while True:
            try:
                n = self.notes.get(timeout=0.0 if (got or msgs) else WAIT)
            except queue.Empty:
                break
            got = True
            if n[0] == "admit":
                user = self.users.get(n[1])
                if user is not None:
                    user.cached = n[2]
            self._apply(self.clients.note(n), emitted, time.monotonic())
        now = time.monotonic()
        for m in msgs:
            if "tokens" in m:
                self.decode_load = m["tokens"].get("load", self.decode_load)
                for rid, tok, last in m["tokens"]["step"]:
                    user = self.users.get(rid)
                    why = "stop" if user is not None and tok in user.stop_ids else "length"
                    self._apply(self.clients.tokens(rid, int(tok), bool(last), why), emitted, now)
                    if last:
                        self.calls.put(("retired", rid))          # the decode tier let the seat go by itself
            else:
                self.calls.put(("d", m))
        if self.left:
            writes, calls = self.clients.sweep(lambda rid: rid in self.left)
            self._apply(writes, emitted, time.monotonic())
            for c in calls:
                self.calls.put(c)
        return emitted

    def run_until_idle(self, max_steps: int = 1 << 30) -> None:
        for _ in range(max_steps):
            if self.idle():
                return
            self.step()

    def close(self) -> None:
        self._halt.set()
        self.calls.put(("quit",))
        self.head.join(10)
        try:
            wire.send(self.sock, {"quit": True})
        except OSError:
            pass
        self.sock.close()

    # ---- the head: its own thread, the one writer to the decode tier ----
    def _hand_over(self, inner: Request) -> None:
        user = self._prefilling.get(inner.id)
        if user is None or inner.finished == "abort" or not inner.out:
            return
        first = inner.out[0]
        if user.max_tokens <= 1 or first in user.stop_ids:
            msg = self.hand.abort(inner.id)                # the first token ends it: the seat goes back unused
            if msg is not None:
                wire.send(self.sock, msg)
            return
        length = inner.seq.length
        if self.mirrors is not None:
            h = self.hand.items[inner.id]
            lease = inner.seq.lease
            if self.dealer is not None:
                self.dealer(self.rt, self.mirrors, list(lease.pages), h.seats, length)
            else:
                self.mirrors.push(pd.group_moves(list(lease.pages), h.seats, length, self.pool.unit, lease.slot, by_position=True))
            h.state = "pushing"
        else:
            for plan in self.hand.prefilled(inner.id, inner.seq.lease, length):
                self.rt.push(self.mapped, plan)
        self.rt.synchronize()                              # the pages are in the decode tier's pool before Start leaves
        # the first token and the hand-over are in the channel before the decode tier can answer the Start
        self.notes.put(("admit", inner.id, inner.cached))
        self.notes.put(("emit", inner.id, first))
        self.notes.put(("decode", inner.id))
        self._handed.add(inner.id)
        smp = user.sampling if getattr(user.sampling, "temperature", 0.0) else None
        wire.send(self.sock, self.hand.pushed(inner.id, first, length, user.max_tokens - 1, tokens=list(user.prompt),
                                              sampling=smp, stop_ids=tuple(user.stop_ids)))

    def _drop(self, rid: str) -> None:
        """The head lets go of a request wherever it holds it, and of its seat on the decode tier."""
        self._asking.pop(rid, None)
        if self._prefilling.pop(rid, None) is not None:
            self.sched.abort(rid)
        self._handed.discard(rid)
        msg = self.hand.abort(rid)
        if msg is not None:
            wire.send(self.sock, msg)

    def _call(self, c: tuple) -> None:
        if c[0] == "submit":
            req = c[1]
            self._asking[req.id] = req
            wire.send(self.sock, self.hand.ask(req.id, len(req.prompt) + req.max_tokens))
        elif c[0] == "d":
            for kind, rid, val in self.hand.told(c[1]):
                if kind == "granted":
                    user = self._asking.pop(rid, None)
                    if user is None:                       # gone while it waited: give the seat back
                        wire.send(self.sock, {"abort": {"req": rid}})
                        continue
                    self._prefilling[rid] = user
                    self.sched.submit(Request(id=rid, prompt=list(user.prompt), max_tokens=1, sampling=user.sampling,
                                              history_tokens=user.history_tokens, arrival=user.arrival))
                elif kind == "refused":
                    self._asking.pop(rid, None)
                    self._handed.discard(rid)
                    log.warning("request %s refused by the decode tier: %s", rid, val)
                    self.notes.put(("reject", rid, val))
        elif c[0] == "abort":            # a decoding request the front retired: free its seats
            self._handed.discard(c[1])
            msg = self.hand.abort(c[1])
            if msg is not None:
                wire.send(self.sock, msg)
        elif c[0] == "retired":          # finished on the decode tier: nothing to send, forget it
            self._handed.discard(c[1])
            self.hand.items.pop(c[1], None)
        elif c[0] == "gone":             # its client left before the hand-over
            if c[1] in self._handed:
                return                   # handed over in the meantime: the front's sweep sees it as decoding next
            self._drop(c[1])
            self.notes.put(("finish", c[1], "abort"))

    def _head_main(self) -> None:
        try:
            while not self._halt.is_set():
                busy = not self.sched.idle()
                try:
                    c = self.calls.get(timeout=0.0 if busy else 0.02)
                    while True:
                        if c[0] == "quit":
                            return
                        self._call(c)
                        c = self.calls.get_nowait()
                except queue.Empty:
                    pass
                if self.sched.idle():
                    continue
                for inner, toks in self.sched.step():
                    user = self._prefilling.get(inner.id)
                    if user is None or not toks:
                        continue
                    if inner.finished is None:
                        continue
                    self._prefilling.pop(inner.id, None)
                    if inner.id in self._handed:
                        continue                              # its notes went out with the hand-over
                    first = toks[0]
                    self.notes.put(("admit", inner.id, inner.cached))
                    self.notes.put(("emit", inner.id, first))
                    self.notes.put(("finish", inner.id, "stop" if first in user.stop_ids else "length"))
        except Exception as e:      # noqa: BLE001 - the front's next step raises it where the server can see it
            log.exception("the prefill head failed")
            self.failed = f"{type(e).__name__}: {e}"
