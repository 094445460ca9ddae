"""Prefill/decode disaggregation as pure state machines.

A prefill (P) head asks a decode (D) tier for seats before it prefills a request, pushes the request's pages and
state slot into those seats when the prompt is done, and hands over with the first token; the D tier decodes and
streams tokens back. Nothing here touches a GPU or a socket: every class takes messages and returns messages (or
copy plans), so the protocol is tested on the CPU and any transport carries it (`wire` frames in production).

    D -> P   Pools{states, page, max_seq_tokens, ranks}                      once, on connect
    P -> D   Reserve{req, tokens} | Start{req, first, len, max_tokens, sampling} | Abort{req}
    D -> P   Grant{req, seats:[{rank, pages, slot}], load} | Busy{req} | Room{} | Refuse{req, why}
             | Tokens{step:[[req, tok, last]], load}
    P        Push{req, pages:[[src, dst]...] per rank, slot:[src, dst] | None, len}   (its own copy plan)

Reference counterpart: crates/kern-serve/src/pd/mod.rs:74-329 (messages, cover, moves), pd/handoff.rs:41-282,
pd/decoder.rs:27-239, pd/tiers.rs:20-157, pd/relay.rs:20-103.
"""
from __future__ import annotations

import random
from collections import deque
from dataclasses import dataclass, field

from .. import _native, fills


# ---- shape check and copy plan ---------------------------------------------------------------------------
def pools_message(doc: dict, unit: int, ranks: int, max_seq_tokens: int) -> dict:
    """What a D tier says about itself: every state's geometry, so P can check its own manifest covers it."""
    return {"pools": {"states": {n: {k: v for k, v in s.items() if k in ("bytes_per_token", "bytes_per_seq", "bytes")}
                                 for n, s in doc["states"].items()},
                      "page": unit, "ranks": ranks, "max_seq_tokens": max_seq_tokens}}


def cover(p_doc: dict, p_unit: int, pools: dict) -> list[str]:
    """Why P's states cannot be pushed into D's pools (empty list: they can). Both sides must hold the same states
    with the same bytes per token / per sequence, and D's page must be a whole number of P's pages or vice versa."""
    d = pools["pools"]
    errs = []
    for name, s in p_doc["states"].items():
        t = d["states"].get(name)
        if t is None:
            errs.append(f"decode tier has no state `{name}`")
            continue
        for k in ("bytes_per_token", "bytes_per_seq"):
            if s.get(k, 0) != t.get(k, 0):
                errs.append(f"state `{name}`: {k} {s.get(k, 0)} here, {t.get(k, 0)} on the decode tier")
    for name in d["states"]:
        if name not in p_doc["states"]:
            errs.append(f"decode tier state `{name}` is not produced here")
    if d["page"] != p_unit:
        errs.append(f"page of {p_unit} tokens here, {d['page']} on the decode tier")
    return errs


def moves(src_pages: list[int], seat: dict, length: int, unit: int, src_slot: int = -1) -> dict:
    """The copies that put the first `length` tokens of a lease into a seat: whole pages pair up in order, the
    state slot (if any) goes to the seat's slot."""
    n = -(-length // unit)
    if n > len(src_pages) or n > len(seat["pages"]):
        raise ValueError(f"{length} tokens need {n} pages; the lease has {len(src_pages)}, the seat {len(seat['pages'])}")
    return {"pages": [[src_pages[i], seat["pages"][i]] for i in range(n)],
            "slot": [src_slot, seat["slot"]] if src_slot >= 0 and seat.get("slot", -1) >= 0 else None}


def group_moves(src_pages: list[int], seats: list[dict], length: int, unit: int, src_slot: int = -1, *,
                by_position: bool = False, splits: dict | None = None, d_unit: int | None = None) -> list[dict]:
    """The copies of one request into the seats of a decode *group* (one seat per rank), a move per (state kind, rank):

    * ``by_position`` (decode context parallelism): rank m of w holds positions p = m (mod w) at local position p // w,
      so its paged states take the dealt rows — ``{"kind": "rows", "rank": m, "runs": [...]}`` with the runs of
      `kern_pool.deal` over this lease's pages and the seat's pages; every rank takes the whole state slot.
    * otherwise (tensor parallel by heads): paged states are sharded by the manifests themselves (each rank's pool holds
      its heads of every position; the prefill side is built with the same sharding, or pushes whole pages when the
      bytes per token agree), and a per-sequence state named in ``splits`` — ``{state: [(rows, width), ...]}``, the
      generator's knowledge of what a line of the slot holds — goes by parts:
      ``{"kind": "part", "rank": m, "state": name, "from": slot, "into": slot, "segments": [...], "of": w, "part": m}``.
    Whole pages / whole slots are ``{"kind": "pages", ...}`` / ``{"kind": "slot", ...}`` as in `moves`.
    Reference: crates/kern-serve/src/pd/mod.rs:225-329 (Move::Rows / Part / Slot)."""
    w = len(seats)
    out: list[dict] = []
    for m, seat in enumerate(seats):
        if by_position:
            runs = _native.deal(list(src_pages), unit, list(seat["pages"]), d_unit or unit, w, m, length)
            out.append({"kind": "rows", "rank": m, "runs": [list(r) for r in runs]})
        else:
            n = -(-length // unit)
            if n > len(src_pages) or n > len(seat["pages"]):
                raise ValueError(f"{length} tokens need {n} pages; the lease has {len(src_pages)}, rank {m}'s seat {len(seat['pages'])}")
            out.append({"kind": "pages", "rank": m, "pages": [[src_pages[i], seat["pages"][i]] for i in range(n)]})
        if src_slot >= 0 and seat.get("slot", -1) >= 0:
            parted = set()
            for name, segments in (splits or {}).items():
                out.append({"kind": "part", "rank": m, "state": name, "from": src_slot, "into": seat["slot"],
                            "segments": [list(x) for x in segments], "of": w, "part": m})
                parted.add(name)
            out.append({"kind": "slot", "rank": m, "slot": [src_slot, seat["slot"]], "except": sorted(parted)})
    return out


class Mirrors:
    """A prefill runtime's view of a decode group: every rank's pools mapped once (they are fixed from the rank's load
    for as long as it serves), and the moves of `group_moves` run into them as copies on the prefill runtime's stream,
    behind the call that wrote the prompt's last rows. `sizes[rank][state]` are the mapped states' bytes (each rank
    says them with its handles), against which every strided copy is checked before it is issued.
    Reference: crates/kern-serve/src/pd/mirror.rs:17-61."""

    def __init__(self, rt, handles: list[dict], sizes: list[dict]):
        self.rt = rt
        self.mapped = [rt.map_pool(h) for h in handles]
        self.sizes = sizes

    def push(self, plan: list[dict]) -> int:
        """Issue every move; returns how many device copies were enqueued."""
        rt, doc, n = self.rt, self.rt.doc, 0
        for mv in plan:
            to, size = self.mapped[mv["rank"]], self.sizes[mv["rank"]]
            if mv["kind"] == "rows":
                for name, s in doc["states"].items():
                    if s.get("bytes_per_token") and name in to:
                        n += rt.push_rows(name, to[name], size[name], mv["runs"], s["bytes_per_token"])
            elif mv["kind"] == "pages":
                rt.push(to, {"pages": mv["pages"], "slot": None})
                n += len(mv["pages"])
            elif mv["kind"] == "part":
                n += rt.push_slot_part(mv["state"], to[mv["state"]], size[mv["state"]], mv["from"], mv["into"],
                                       [tuple(x) for x in mv["segments"]], mv["of"], mv["part"])
            elif mv["kind"] == "slot":
                for name, s in doc["states"].items():
                    if s.get("bytes_per_seq") and name in to and name not in mv.get("except", ()):
                        rt.push_state_unit(name, to[name], mv["slot"][0], mv["slot"][1])
                        n += 1
            else:
                raise ValueError(f"unknown move {mv['kind']!r}")
        return n


# ---- D side ------------------------------------------------------------------------------------------------
@dataclass
class _Seat:
    req: str
    seq: object                      # engine Sequence (lease inside)
    started: bool = False
    max_tokens: int = 0
    produced: int = 0
    last: int = 0
    stop_ids: tuple = ()


class Decoder:
    """The decode tier's head: grants seats, starts sequences whose state has been pushed, steps them."""

    def __init__(self, engine, max_seqs: int | None = None, stop_ids: tuple = ()):
        self.eng = engine
        self.pool = engine.pool
        self.max_seqs = max_seqs or engine.groups_max
        self.seats: dict[str, _Seat] = {}
        self.waiting: deque[dict] = deque()      # Reserve asks answered Busy, in order
        self.stop_ids = tuple(stop_ids)
        self.told_busy = False

    def load(self) -> dict:
        p = self.pool
        return {"seqs": len(self.seats), "free_pages": p.free_pages, "total_pages": p.total_pages}

    def _grant(self, ask: dict) -> dict | None:
        if len(self.seats) >= self.max_seqs:
            return None
        from ..engine import Sequence
        try:
            lease = self.pool.lease(ask["tokens"])
        except _native.Denied as e:
            why = e.args[1] if len(e.args) > 1 else "busy"
            if why != "busy":
                return {"refuse": {"req": ask["req"], "why": why}}
            return None
        members = getattr(lease, "members", [lease])
        self.seats[ask["req"]] = _Seat(req=ask["req"], seq=Sequence(lease=lease))
        return {"grant": {"req": ask["req"], "load": self.load(),
                          "seats": [{"rank": i, "pages": list(m.pages), "slot": m.slot} for i, m in enumerate(members)]}}

    def handle(self, msg: dict) -> list[dict]:
        """One message from P -> the replies to send."""
        if "reserve" in msg:
            ask = msg["reserve"]
            if self.pool.pages_for(ask["tokens"]) > self.pool.total_pages:
                return [{"refuse": {"req": ask["req"], "why": "exceeds_pool"}}]
            got = self._grant(ask)
            if got is None:
                self.waiting.append(ask)
                self.told_busy = True
                return [{"busy": {"req": ask["req"]}}]
            return [got]
        if "start" in msg:
            st = msg["start"]
            seat = self.seats.get(st["req"])
            if seat is None:
                return [{"refuse": {"req": st["req"], "why": "unknown request"}}]
            seat.started, seat.last, seat.max_tokens = True, int(st["first"]), int(st["max_tokens"])
            seat.seq.length = int(st["len"])
            seat.seq.tokens = list(st.get("tokens", []))
            seat.stop_ids = tuple(st.get("stop_ids", self.stop_ids))
            smp = st.get("sampling")
            if smp:
                seat.seq.sampling = fills.Sampling(**smp)
            return []
        if "abort" in msg:
            return self._release(msg["abort"]["req"])
        raise ValueError(f"unknown message {sorted(msg)}")

    def _release(self, req: str) -> list[dict]:
        seat = self.seats.pop(req, None)
        if seat is not None:
            self.eng.close(seat.seq)
        # an ask that was answered Busy and is still queued dies with its request: granted later, its seat would belong
        # to nobody (the prefill side has already forgotten the request)
        if any(a["req"] == req for a in self.waiting):
            self.waiting = deque(a for a in self.waiting if a["req"] != req)
        out = []
        while self.waiting:                       # whoever waited longest gets the room first
            got = self._grant(self.waiting[0])
            if got is None:
                break
            self.waiting.popleft()
            out.append(got)
        if self.told_busy and not self.waiting:
            self.told_busy = False
            out.append({"room": {}})
        return out

    def step(self) -> list[dict]:
        """One decode call over every started sequence -> [Tokens{...}] plus grants freed by finished ones."""
        live = [s for s in self.seats.values() if s.started]
        if not live:
            return []
        toks = self.eng.step([(s.seq, [s.last]) for s in live])
        step, after = [], []
        for s, got in zip(live, toks):
            t = int(got[0])
            s.produced += 1
            s.last = t
            last = t in s.stop_ids or s.produced >= s.max_tokens
            step.append([s.req, t, last])
            if last:
                after += self._release(s.req)
        return [{"tokens": {"step": step, "load": self.load()}}] + after


# ---- P side ------------------------------------------------------------------------------------------------
@dataclass
class _Handoff:
    req: str
    tokens: int
    state: str = "asked"              # asked -> granted -> pushed -> started | refused
    seats: list = field(default_factory=list)
    tier: int = 0


class Handoffs:
    """P's side of every request in flight towards a D tier."""

    def __init__(self, unit: int):
        self.unit = unit
        self.items: dict[str, _Handoff] = {}
        self.busy_tiers: set[int] = set()

    def ask(self, req: str, tokens: int, tier: int = 0) -> dict:
        self.items[req] = _Handoff(req=req, tokens=tokens, tier=tier)
        return {"reserve": {"req": req, "tokens": tokens}}

    def told(self, msg: dict, tier: int = 0) -> list[tuple[str, str, object]]:
        """One message from D -> events for the prefill scheduler:
        ("granted", req, seats) | ("refused", req, why) | ("tokens", req, (tok, last)) | ("room", tier, None)."""
        ev = []
        if "grant" in msg:
            g = msg["grant"]
            h = self.items.get(g["req"])
            if h is not None:
                h.state, h.seats = "granted", g["seats"]
                ev.append(("granted", h.req, g["seats"]))
        elif "busy" in msg:
            self.busy_tiers.add(tier)
        elif "room" in msg:
            self.busy_tiers.discard(tier)
            ev.append(("room", tier, None))
        elif "refuse" in msg:
            r = msg["refuse"]
            h = self.items.pop(r["req"], None)
            if h is not None:
                ev.append(("refused", r["req"], r["why"]))
        elif "tokens" in msg:
            for req, tok, last in msg["tokens"]["step"]:
                ev.append(("tokens", req, (tok, last)))
                if last:
                    self.items.pop(req, None)
        return ev

    def ready(self, req: str) -> bool:
        h = self.items.get(req)
        return h is not None and h.state == "granted"

    def prefilled(self, req: str, lease, length: int) -> list[dict]:
        """The prompt is in P's states: the push plan for every member rank (rank i's lease -> seat i)."""
        h = self.items[req]
        if h.state != "granted":
            raise RuntimeError(f"request {req} prefilled before a seat was granted (state {h.state})")
        members = getattr(lease, "members", [lease])
        if len(members) != len(h.seats):
            raise RuntimeError(f"request {req}: {len(members)} prefill ranks, {len(h.seats)} decode seats")
        plans = [{"req": req, "rank": i, "len": length, **moves(list(m.pages), h.seats[i], length, self.unit, m.slot)}
                 for i, m in enumerate(members)]
        h.state = "pushing"
        return plans

    def pushed(self, req: str, first: int, length: int, max_tokens: int, tokens: list[int] | None = None,
               sampling: fills.Sampling | None = None, stop_ids: tuple = ()) -> dict:
        h = self.items[req]
        h.state = "started"
        msg = {"req": req, "first": int(first), "len": int(length), "max_tokens": int(max_tokens), "stop_ids": list(stop_ids),
               "tokens": list(tokens or [])}
        if sampling is not None:
            msg["sampling"] = sampling.__dict__
        return {"start": msg}

    def abort(self, req: str) -> dict | None:
        if self.items.pop(req, None) is None:
            return None
        return {"abort": {"req": req}}


class Tiers:
    """Several D tiers behind one P: pick by the power of two choices on the load each last reported."""

    def __init__(self, n: int, seed: int = 0):
        self.loads = [{"seqs": 0, "free_pages": 1 << 30, "total_pages": 1 << 30} for _ in range(n)]
        self.rng = random.Random(seed)

    def report(self, tier: int, load: dict) -> None:
        self.loads[tier] = load

    def score(self, tier: int) -> float:
        l = self.loads[tier]
        return l["seqs"] + 1.0 - l["free_pages"] / max(1, l["total_pages"])

    def pick(self, busy: set[int] = frozenset()) -> int | None:
        open_ = [t for t in range(len(self.loads)) if t not in busy]
        if not open_:
            return None
        if len(open_) == 1:
            return open_[0]
        a, b = self.rng.sample(open_, 2)
        return a if self.score(a) <= self.score(b) else b


class Relay:
    """Streams a D tier's tokens to whoever waits on the request on the P side (the HTTP front)."""

    def __init__(self):
        self.sinks: dict[str, object] = {}

    def watch(self, req: str, sink) -> None:
        self.sinks[req] = sink

    def deliver(self, events: list[tuple[str, str, object]]) -> None:
        for kind, req, val in events:
            sink = self.sinks.get(req)
            if sink is None:
                continue
            if kind == "tokens":
                tok, last = val
                sink(tok, last)
                if last:
                    self.sinks.pop(req, None)
            elif kind == "refused":
                sink(None, True)
                self.sinks.pop(req, None)
