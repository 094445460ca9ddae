"""Prefill/decode disaggregation as a deployment: the state machines of `pd.py` carried by `wire` frames.

    prefill tier (this process)                                decode tier (a process of its own, its own GPU)
    PrefillTier: scheduler-like face for the HTTP front        decode_loop: pd.Decoder over its engine
      submit   -> Reserve ------------------------------------>  grant seats (pages + slot) | Busy (queued) | Refuse
      granted  -> the prompt joins the prefill scheduler
      first token -> push pages and slot into the seats
                     (device copies into the mapped pools), Start ->  decode steps
      tokens of every decode step  <----------------------------  Tokens{[req, tok, last]}

A decode tier may be a group that deals every sequence's positions over its members (decode context parallelism, a
`models/dense_dcp.py` member manifest behind `ranks.GroupEngine(by_position=True)`): the Hello then lists every member's
handles and sizes, a grant holds one seat per member, and the hand-over deals the prompt's rows — position p to member
p mod w at local position p // w — by `pd.group_moves` + `pd.Mirrors` (token-contiguous states), or by the model's own
`dealer` where a page is not token-contiguous (the dense KV pages: `dense_dcp.dealer`, the deal kernel writing into the
members' mapped pools).

The decode tier says Hello once with its pools' geometry and export handles; the prefill tier checks that its own
manifest covers them (`pd.cover`) and maps them (`Runtime.map_pool`). The prefill scheduler keeps its prefix cache: a
finished prompt's pages stay behind as on one GPU. A request whose first token ends it never reaches the decode tier
(its seat is given back). The decode process exits when the connection closes.
Reference counterpart: crates/kern-serve/src/pd/handoff.rs:41-282, pd/decoder.rs:27-239, pd/relay.rs:20-103 (the tiers as
processes), crates/kern-serve/src/lib.rs:317-404 (deployment by flags).
"""
from __future__ import annotations

import logging
import select
import time

from . import pd, wire
from .scheduler import Request, Scheduler

log = logging.getLogger("kern.serve")


def _drain(sock, wait: float) -> list[dict] | None:
    """Every frame that is there (waiting up to `wait` seconds for the first); None when the peer closed."""
    out = []
    while True:
        ready, _, _ = select.select([sock], [], [], wait if not out else 0.0)
        if not ready:
            return out
        msg = wire.recv(sock)
        if msg is None:
            return None if not out else out
        out.append(msg)


def hello_of(rt, doc: dict, max_seq_tokens: int, handles=None) -> dict:
    """What the decode tier says first. `handles`: its pools' export handles (left out when both tiers live in one
    process and the prefill tier is handed the pools directly)."""
    msg = pd.pools_message(doc, rt.page_unit, 1, max_seq_tokens)
    if handles is not None:
        msg["handles"] = handles
    return {"hello": msg}


def decode_loop(sock, engine, max_seqs: int | None = None, stop_ids: tuple = (), idle_wait: float = 0.2) -> int:
    """The decode tier's process loop: messages in, one decode call over every started sequence, messages out. Returns
    the number of decode calls. Ends when the prefill tier closes the connection or says quit."""
    dec = pd.Decoder(engine, max_seqs=max_seqs, stop_ids=stop_ids)
    calls = 0
    while True:
        live = any(s.started for s in dec.seats.values())
        try:
            msgs = _drain(sock, 0.0 if live else idle_wait)
        except (ConnectionError, OSError):
            msgs = None
        if msgs is None:
            break
        out = []
        quit_ = False
        for m in msgs:
            if "quit" in m:
                quit_ = True
                continue
            out += dec.handle(m)
        if quit_:
            break
        step = dec.step()
        calls += bool(step)
        try:
            for m in out + step:
                wire.send(sock, m)
        except (ConnectionError, OSError):        # the prefill tier went away in the middle of a step
            break
    for seat in list(dec.seats.values()):          # whatever was in flight when the front went away
        engine.close(seat.seq)
    return calls


class PrefillTier:
    """The prefill tier's face towards the HTTP front (submit / step / idle / abort / metrics / stats): requests wait
    for a seat on the decode tier, are prefilled by the local scheduler, handed over with their first token, and
    receive the decode tier's tokens."""

    def __init__(self, sched: Scheduler, rt, sock, mapped, poll_wait: float = 0.002, mirrors=None, dealer=None):
        self.sched, self.rt, self.sock, self.mapped = sched, rt, sock, mapped
        self.mirrors, self.dealer = mirrors, dealer      # a decode group that deals positions over its members
        self.hand = pd.Handoffs(sched.pool.unit)
        self.asking: dict[str, Request] = {}       # Reserve sent, no seat yet
        self.prefilling: dict[str, Request] = {}   # in the local scheduler (by the user's request id)
        self.decoding: dict[str, Request] = {}     # handed over
        self.done: list[Request] = []
        self.stats = sched.stats
        self.pool = sched.pool
        self.poll_wait = poll_wait
        self.lost = False
        self.decode_load: dict = {}
        sched.on_finish = self._hand_over

    # ---- the scheduler interface ----
    def submit(self, req: Request) -> None:
        need = len(req.prompt) + req.max_tokens
        if self.pool.pages_for(need) > self.pool.total_pages:
            req.finished = "abort"
            self.done.append(req)
            raise ValueError(f"request {req.id} needs {need} tokens, more than the prefill pool holds")
        self.asking[req.id] = req
        wire.send(self.sock, self.hand.ask(req.id, need))

    def abort(self, req_id: str) -> bool:
        for box in (self.asking, self.decoding):
            r = box.pop(req_id, None)
            if r is not None:
                msg = self.hand.abort(req_id)
                if msg is not None:
                    wire.send(self.sock, msg)
                r.finished = "abort"
                self.done.append(r)
                return True
        r = self.prefilling.pop(req_id, None)
        if r is not None:
            self.sched.abort(req_id)
            msg = self.hand.abort(req_id)
            if msg is not None:
                wire.send(self.sock, msg)
            r.finished = "abort"
            self.done.append(r)
            return True
        return False

    def idle(self) -> bool:
        return not (self.asking or self.prefilling or self.decoding)

    def metrics(self) -> dict:
        m = self.sched.metrics()
        m["num_waiting_reqs"] += len(self.asking)
        m["pd"] = {"waiting_for_seat": len(self.asking), "prefilling": len(self.prefilling), "decoding": len(self.decoding),
                   "decode_tier": self.decode_load}
        return m

    # ---- one step ----
    def _hand_over(self, inner: Request) -> None:
        """The local scheduler is done with a prompt (its first token is out, its lease still held): push its pages and
        slot into the seats and start it on the decode tier."""
        user = self.prefilling.get(inner.id)
        if user is None or inner.finished == "abort" or not inner.out:
            return
        first = inner.out[0]
        if user.max_tokens <= 1 or first in user.stop_ids:
            msg = self.hand.abort(inner.id)            # the first token ends it: the seat goes back unused
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
        self.rt.synchronize()                          # the pages are in the decode tier's pool before Start leaves
        smp = user.sampling if getattr(user.sampling, "temperature", 0.0) else None
        wire.send(self.sock, self.hand.pushed(inner.id, first, length, user.max_tokens - 1, tokens=list(user.prompt),
                                              sampling=smp, stop_ids=tuple(user.stop_ids)))

    def _take(self, user: Request, toks: list[int], now: float) -> None:
        if user.first_token_at is None and toks:
            user.first_token_at = now
        for t in toks:
            user.out.append(int(t))
            user.token_times.append(now)

    def step(self) -> list[tuple[Request, list[int]]]:
        emitted = []
        busy_here = not self.sched.idle()
        msgs = _drain(self.sock, 0.0 if busy_here else self.poll_wait)
        if msgs is None:
            self.lost = True
            raise ConnectionError("the decode tier closed its connection")
        now = time.monotonic()
        for m in msgs:
            if "tokens" in m:
                self.decode_load = m["tokens"].get("load", self.decode_load)
            for kind, req, val in self.hand.told(m):
                if kind == "granted":
                    user = self.asking.pop(req, None)
                    if user is None:                   # aborted while it waited: give the seat back
                        wire.send(self.sock, {"abort": {"req": req}})
                        continue
                    self.prefilling[req] = user
                    self.sched.submit(Request(id=req, prompt=list(user.prompt), max_tokens=1, sampling=user.sampling,
                                              history_tokens=user.history_tokens, arrival=user.arrival))
                elif kind == "refused":
                    user = self.asking.pop(req, None) or self.decoding.pop(req, None)
                    if user is not None:
                        log.warning("request %s refused by the decode tier: %s", req, val)
                        user.finished = "abort"
                        self.done.append(user)
                        emitted.append((user, []))
                elif kind == "tokens":
                    user = self.decoding.get(req)
                    if user is None:
                        continue
                    tok, last = val
                    self._take(user, [tok], now)
                    if last:
                        user.finished = "stop" if tok in user.stop_ids else "length"
                        self.decoding.pop(req)
                        self.done.append(user)
                    emitted.append((user, [int(tok)]))
        if busy_here:
            for inner, toks in self.sched.step():
                user = self.prefilling.get(inner.id)
                if user is None or not toks:
                    continue
                user.cached, user.fed = inner.cached, inner.fed
                self._take(user, toks[:1], time.monotonic())
                if inner.finished is not None:
                    self.prefilling.pop(inner.id)
                    first = toks[0]
                    if user.max_tokens <= 1 or first in user.stop_ids:
                        user.finished = "stop" if first in user.stop_ids else "length"
                        self.done.append(user)
                    else:
                        self.decoding[inner.id] = user
                emitted.append((user, toks[:1]))
        return emitted

    def run_until_idle(self, max_steps: int = 1 << 30) -> None:
        for _ in range(max_steps):
            if self.idle():
                return
            self.step()

    def close(self) -> None:
        try:
            wire.send(self.sock, {"quit": True})
        except OSError:
            pass
        self.sock.close()


def connect_tiers(sched: Scheduler, rt, doc: dict, sock, pools=None, timeout: float = 600.0, dealer=None, front: bool = False):
    """Read the decode tier's Hello from `sock`, check that this tier's manifest covers its pools, map them (or take
    `pools`, the decode runtime's exported states, when both tiers share a process) and return the prefill tier:
    `PrefillTier` (one loop steps the scheduler and relays tokens), or with `front` a `front.Front` (the scheduler on a
    head thread, tokens relayed as they come)."""
    ready, _, _ = select.select([sock], [], [], timeout)
    if not ready:
        raise TimeoutError("the decode tier did not say hello")
    msg = wire.recv(sock)
    if msg is None or "hello" not in msg:
        raise ConnectionError(f"expected the decode tier's hello, got {msg!r}")
    hello = msg["hello"]
    why = pd.cover(doc, rt.page_unit, hello)
    if why:
        raise ValueError("the prefill manifest does not cover the decode tier's pools: " + "; ".join(why))
    if front:                               # the prefill scheduler on a head thread of its own (`front.py`)
        from .front import Front as Tier
    else:
        Tier = PrefillTier
    if "members" in hello:                  # a decode group: every member's pools, mapped once
        mirrors = pd.Mirrors(rt, [m["handles"] for m in hello["members"]], [m["sizes"] for m in hello["members"]])
        return Tier(sched, rt, sock, None, mirrors=mirrors, dealer=dealer)
    mapped = rt.map_pool(pools if pools is not None else hello["handles"])
    return Tier(sched, rt, sock, mapped)
