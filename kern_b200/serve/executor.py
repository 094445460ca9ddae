"""Process-per-GPU rank executors and the head's fan-out.

A rank process owns one runtime and no scheduler. It connects to the head, says ``Hello{rank,pages,slots,offer}``,
gets back ``Table{peers:{group:[offer...]}}`` (every member's exported handles, in member order), maps its peers,
runs the ``once`` programs, and then serves ``Order{acts,item}`` -> ``Answer{tokens,counts,landed,error}`` until
the head closes. The head sends every rank its order in parallel and gathers the answers.
Reference counterpart: crates/kern-serve/src/executor.rs:69-122 (handshake), :150-165 (join),
:263-296 (rank loop), :299-376 (Executor), :412-450 (Executors::run).
"""
from __future__ import annotations

import logging
import threading

import numpy as np

from ..parallel.group import members_of
from . import wire

log = logging.getLogger("kern.serve")
_NP = {"i32": np.int32, "i64": np.int64, "f32": np.float32, "u8": np.uint8}


class Executor:
    """Rank side: runs acts and items against one runtime."""

    def __init__(self, rt):
        self.rt = rt
        self.p = rt.protocol
        self._fills = {f["name"]: f for f in (self.p["fills"] if self.p else [])}

    def act(self, a: dict):
        if "zero" in a:
            self.rt.zero_slot(int(a["zero"]))
        elif "copy" in a:
            c = a["copy"]
            self.rt.run_copies({"pages": [tuple(x) for x in c.get("pages", [])],
                                "slot": tuple(c["slot"]) if c.get("slot") else None})
        elif "write" in a:          # rows of an input outside the protocol (a landing, a mask)
            w = a["write"]
            self.rt.write(w["name"], np.asarray(w["values"], _NP[w["dtype"]]), w.get("offset", 0))
        else:
            raise ValueError(f"unknown act {sorted(a)}")
        return None

    def run(self, order: dict) -> dict:
        landed = [x for x in (self.act(a) for a in order.get("acts", [])) if x is not None]
        ans = {"tokens": [], "counts": [], "landed": landed, "error": 0}
        item = order.get("item")
        if item:
            for name, (dtype, values) in item["rows"].items():
                self.rt.write(name, np.asarray(values, _NP[dtype]))
            self.rt.issue(item["program"], item["vars"])
            emits, count, groups = item.get("emits"), item.get("count"), item.get("groups", 0)
            if emits and item.get("read", True):
                w = self._fills[emits]["width"]
                toks = np.asarray(self.rt.read(emits, groups * w)).reshape(groups, w)
                ans["tokens"] = toks.tolist()
                if count:
                    ans["counts"] = np.asarray(self.rt.read(count, groups)).tolist()
            else:
                self.rt.synchronize()
            for f in self._fills.values():
                if f["fill"] == "error":
                    ans["error"] = int(np.asarray(self.rt.read(f["name"], 1))[0])
        return ans


def serve_rank(head: tuple[str, int], rank: int, world: int, make_runtime, watch=None, export_pools: bool = False) -> None:
    """A rank process's whole life. ``make_runtime() -> runtime`` builds and loads this rank's runtime (its
    place in every group is ``parallel.group.topology(groups, rank, world)``). ``export_pools``: the Hello also carries
    a handle and the size of every state of this rank's pools, for a prefill tier that pushes into them."""
    sock = wire.connect(head)
    try:
        rt = make_runtime()
    except Exception as e:       # tell the head why instead of leaving it waiting for a Hello
        log.exception("rank %d could not start", rank)
        wire.send(sock, {"hello": {"rank": rank, "failed": f"{type(e).__name__}: {e}"}})
        sock.close()
        return
    offer = rt.offer() if hasattr(rt, "offer") else {}
    hello = {"rank": rank, "pages": rt.pages, "slots": rt.slots, "unit": rt.page_unit, "offer": offer}
    if export_pools:
        hello["pools"] = {"handles": rt.export_states(), "sizes": rt.state_bytes()}
    wire.send(sock, {"hello": hello})
    table = wire.recv(sock)
    if table is None:
        return
    for group, offers in table["table"]["peers"].items():
        if len(offers) > 1:
            rt.connect(group, offers)
    rt.once()
    rt.synchronize()
    wire.send(sock, {"joined": rank})
    ex = Executor(rt)
    log.info("rank ready rank=%d pages=%d slots=%d", rank, rt.pages, rt.slots)
    while True:
        try:
            order = wire.recv(sock)
        except (ConnectionError, OSError):      # the head went away: same as a clean close
            return
        if order is None:
            return
        try:
            answer = ex.run(order)
        except Exception as e:     # the head decides what a failed step means; the rank stays in its loop
            log.exception("order failed rank=%d", rank)
            answer = {"tokens": [], "counts": [], "landed": [], "error": -1, "why": f"{type(e).__name__}: {e}"}
        try:
            wire.send(sock, answer)
        except (ConnectionError, OSError):
            return


class Executors:
    """Head side: the connections to every rank, in rank order."""

    def __init__(self, lsock, world: int, groups: dict[str, int], watch=None, timeout: float = 600.0):
        self.world, self.groups = world, groups
        socks, hellos = [None] * world, [None] * world
        lsock.settimeout(timeout)
        for _ in range(world):
            s = wire.accept(lsock)
            s.settimeout(timeout)
            m = wire.recv(s)
            if m is None or "hello" not in m:
                raise ConnectionError("a rank closed its connection before its Hello")
            h = m["hello"]
            if "failed" in h:
                raise RuntimeError(f"rank {h['rank']} could not start: {h['failed']}")
            s.settimeout(None)
            socks[h["rank"]], hellos[h["rank"]] = s, h
        self.socks, self.hellos = socks, hellos
        for q in range(world):
            peers = {g: [hellos[r]["offer"] for r in members_of(groups, g, q, world)] for g in groups}
            wire.send(socks[q], {"table": {"peers": peers}})
        for q in range(world):
            j = wire.recv(socks[q])
            if j is None or j.get("joined") != q:
                raise ConnectionError(f"rank {q} did not join")
        self.watch = watch
        if watch:
            for q, s in enumerate(socks):
                watch.add(s, f"rank {q}")

    @property
    def pages(self) -> list[int]:
        return [h["pages"] for h in self.hellos]

    @property
    def slots(self) -> list[int]:
        return [h["slots"] for h in self.hellos]

    def run(self, orders: list[dict | None]) -> list[dict | None]:
        """Send every rank its order at once, then gather; a rank with no order (None) is left alone."""
        for q, o in enumerate(orders):
            if o is not None:
                wire.send(self.socks[q], o)
        out: list[dict | None] = [None] * self.world
        for q, o in enumerate(orders):
            if o is not None:
                a = wire.recv(self.socks[q])
                if a is None:
                    raise ConnectionError(f"rank {q} closed its connection")
                if a.get("error", 0) != 0:
                    raise RuntimeError(f"rank {q}: step failed (error {a['error']}) {a.get('why', '')}")
                out[q] = a
        return out

    def close(self) -> None:
        for s in self.socks:
            if self.watch:
                self.watch.remove(s)
            try:
                s.close()
            except OSError:
                pass


def spawn_threads(world: int, make_runtime_for_rank, groups: dict[str, int], timeout: float = 120.0):
    """In-process ranks on threads (CPU executor, tests): returns (Executors, threads)."""
    lsock = wire.listen()
    addr = lsock.getsockname()
    threads = [threading.Thread(target=serve_rank, args=(addr, q, world, make_runtime_for_rank(q)), daemon=True)
               for q in range(world)]
    for t in threads:
        t.start()
    try:
        ex = Executors(lsock, world, groups, timeout=timeout)
    finally:
        lsock.close()
    return ex, threads
