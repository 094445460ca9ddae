"""Pipeline-parallel prefill that pipelines: a process per stage, several items (prompt chunks, steps) in flight.

Every rank of the pipeline's process group loads one stage manifest of `Manifest.cut` on its own GPU. The head (stage 0)
turns requests into *items* — (program, vars, input columns) — and announces each on the control group; every stage
runs the items in order:

    receive item k's crossing buffers from the stage before      (NCCL p2p on the receive stream, into landing k % 2)
    land them in the buffers the stage computes in               (compute stream, after the receive's event)
    run the stage's part of the program                          (compute stream = the runtime's stream)
    copy what crosses the next cut into send twin k % 2          (compute stream)
    send it to the next stage                                    (NCCL p2p on the send stream, after the copy's event)

The three streams are ordered by events only: while item k computes, item k + 1's buffers are already arriving and
item k - 1's are leaving, and the host is never in the device's path. With `LANDINGS` = 2 twins per crossing buffer a
stage is held back only when the next one is two items behind (the NCCL send cannot complete before the matching
receive is posted, and the receive waits for its landing to be free): that is the whole back-pressure. The last stage
reports each item's tokens to the head on the control group; the head keeps at most `ahead` items unreported. A
neighbour that delivers or takes nothing for `timeout` seconds (60 by default) ends the wait with an error naming it.

The same code runs on CPU ranks (gloo, host-memory runtimes): streams and events become no-ops and the waits block
the host, which is what the CPU tests use.
Reference counterpart: crates/kern-serve/src/pp/mod.rs:31-47 (landings), :72 (TIMEOUT), :225-389 (edges),
pp/stage.rs:41-192 (a stage's loop), pp/head.rs:941-1129 (chunks through the stages), pp/pack.rs:65-120. The
reference pushes with its own copy kernels and device gates; here the transport is NCCL send/recv on side streams.
"""
from __future__ import annotations

import json
import logging
import time
from dataclasses import dataclass, field

import numpy as np
import torch
import torch.distributed as dist

from .. import _native, fills
from . import pp as pp_cut

LANDINGS = 2
TIMEOUT = 60.0
log = logging.getLogger("kern.serve")
_NP = {"i32": np.int32, "i64": np.int64, "f32": np.float32}


class StageTimeout(RuntimeError):
    pass


@dataclass
class Item:
    """One call of one program, as the head announces it."""
    k: int
    program: str
    vars: dict
    columns: dict                      # input name -> [dtype, values]
    emits: str | None = None
    count: str | None = None
    groups: int = 0
    real: int = 0
    width: int = 1
    stop: bool = False

    def to_wire(self) -> str:
        return json.dumps({"k": self.k, "program": self.program, "vars": self.vars, "columns": self.columns, "emits": self.emits,
                           "count": self.count, "groups": self.groups, "real": self.real, "width": self.width, "stop": self.stop})

    @staticmethod
    def from_wire(s: str) -> "Item":
        return Item(**json.loads(s))


class _Streams:
    """Compute / receive / send streams and events on a GPU; no-ops on CPU ranks."""

    def __init__(self, rt, device: torch.device):
        self.cuda = device.type == "cuda"
        if self.cuda:
            self.compute = torch.cuda.ExternalStream(rt.stream, device=device)
            self.recv = torch.cuda.Stream(device=device)
            self.send = torch.cuda.Stream(device=device)

    def event(self):
        return torch.cuda.Event() if self.cuda else None

    def on(self, stream):
        import contextlib

        return torch.cuda.stream(stream) if self.cuda else contextlib.nullcontext()


def crossing_names(prev_doc: dict, doc: dict) -> list[str]:
    """Buffers that travel from the stage before into this one: its exported inputs that the previous stage writes."""
    outs = {n for n, x in prev_doc["buffers"].items() if x["kind"] in ("output", "inout") and not x.get("fill")}
    return [n for n, x in doc["buffers"].items() if x.get("export") and n in outs]


class Stage:
    def __init__(self, rt, docs: list[dict], rank: int, data_pg=None, ctrl_pg=None, timeout: float = TIMEOUT):
        self.rt, self.docs, self.rank, self.world = rt, docs, rank, len(docs)
        self.doc = docs[rank]
        self.data_pg, self.ctrl_pg, self.timeout = data_pg, ctrl_pg, timeout
        probe = rt.tensor(next(iter(self.doc["buffers"])))
        self.device = probe.device
        self.st = _Streams(rt, self.device)
        self.vmax = {k: v["max"] for k, v in self.doc["vars"].items()}
        self.arrive = crossing_names(docs[rank - 1], self.doc) if rank > 0 else []
        self.leave = crossing_names(self.doc, docs[rank + 1]) if rank + 1 < self.world else []
        flat = lambda n: rt.tensor(n).view(-1).view(torch.uint8)
        self.bufs = {n: flat(n) for n in set(self.arrive + self.leave)}
        twin = lambda n: [torch.empty_like(self.bufs[n]) for _ in range(LANDINGS)]
        self.landing = {n: twin(n) for n in self.arrive}
        self.outgoing = {n: twin(n) for n in self.leave}
        self.landing_free = [self.st.event() for _ in range(LANDINGS)]      # recorded when a landing has been copied out
        self.arrived = [self.st.event() for _ in range(LANDINGS)]
        self.ready = [self.st.event() for _ in range(LANDINGS)]             # a send twin holds item k's outputs
        self.sent = [self.st.event() for _ in range(LANDINGS)]
        self.sends: list = [[] for _ in range(LANDINGS)]                   # outstanding send handles per twin (CPU ranks wait on them)
        self.timeline: list[tuple[int, int, int, int]] = []                # (item, rows, issued_us, done_us) of every item run here
        self._stamps: list = []                                            # GPU: items whose end event has not happened yet
        self._t0 = None                                                    # GPU: (event, host microseconds) the ends are measured from
        self.items = 0
        self.moved_bytes = 0

    # ---- helpers ----
    def _bytes(self, doc: dict, name: str, vars_: dict) -> int:
        vmax = {k: v["max"] for k, v in doc["vars"].items()}
        return pp_cut._bytes_for(doc["buffers"][name], vars_, vmax)

    def _wait(self, work, what: str) -> None:
        """Block the host on a CPU rank's transfer (a GPU rank orders its streams by events instead)."""
        try:
            if not work.wait(timeout=_timedelta(self.timeout)):
                raise StageTimeout(what)
        except RuntimeError as e:
            if "imeout" in str(e) or "timed out" in str(e):
                raise StageTimeout(f"{what}: nothing for {self.timeout:.0f} s") from e
            raise

    # ---- one item ----
    def run(self, item: Item):
        rt, st, j = self.rt, self.st, item.k % LANDINGS
        issued_us = time.perf_counter_ns() // 1000
        bufs = self.doc["buffers"]
        for name, (dtype, vals) in item.columns.items():
            if name in bufs and bufs[name]["kind"] == "input":
                rt.write(name, np.ascontiguousarray(np.asarray(vals, dtype=_NP[dtype])))
        vars_ = {k: v for k, v in item.vars.items() if k in self.doc["vars"]}
        if self.arrive:
            sizes = {n: self._bytes(self.doc, n, item.vars) for n in self.arrive}
            if st.cuda:
                with st.on(st.recv):
                    if self.items >= LANDINGS:
                        st.recv.wait_event(self.landing_free[j])              # item k - 2 has been copied out of this landing
                    works = [dist.irecv(self.landing[n][j][:sizes[n]], src=self._peer(self.rank - 1), group=self.data_pg) for n in self.arrive]
                    for w in works:
                        w.wait()                                             # the receive stream waits, not the host
                    self.arrived[j].record(st.recv)
                st.compute.wait_event(self.arrived[j])
                with st.on(st.compute):
                    for n in self.arrive:
                        self.bufs[n][:sizes[n]].copy_(self.landing[n][j][:sizes[n]], non_blocking=True)
                    self.landing_free[j].record(st.compute)
            else:
                works = [dist.irecv(self.landing[n][j][:sizes[n]], src=self._peer(self.rank - 1), group=self.data_pg) for n in self.arrive]
                for n, w in zip(self.arrive, works):
                    self._wait(w, f"stage {self.rank}: item {item.k} from stage {self.rank - 1}")
                    self.bufs[n][:sizes[n]].copy_(self.landing[n][j][:sizes[n]])
            self.moved_bytes += sum(sizes.values())
        rt.issue(item.program, vars_)
        if self.leave:
            sizes = {n: self._bytes(self.docs[self.rank + 1], n, item.vars) for n in self.leave}
            if st.cuda:
                with st.on(st.compute):
                    if self.items >= LANDINGS:
                        st.compute.wait_event(self.sent[j])                  # item k - 2 has left this twin
                    for n in self.leave:
                        self.outgoing[n][j][:sizes[n]].copy_(self.bufs[n][:sizes[n]], non_blocking=True)
                    self.ready[j].record(st.compute)
                with st.on(st.send):
                    st.send.wait_event(self.ready[j])
                    works = [dist.isend(self.outgoing[n][j][:sizes[n]], dst=self._peer(self.rank + 1), group=self.data_pg) for n in self.leave]
                    for w in works:
                        w.wait()
                    self.sent[j].record(st.send)
            else:
                for w in self.sends[j]:
                    self._wait(w, f"stage {self.rank}: stage {self.rank + 1} has not taken item {item.k - LANDINGS}")
                for n in self.leave:
                    self.outgoing[n][j][:sizes[n]].copy_(self.bufs[n][:sizes[n]])
                self.sends[j] = [dist.isend(self.outgoing[n][j][:sizes[n]], dst=self._peer(self.rank + 1), group=self.data_pg) for n in self.leave]
        self.items += 1
        self._stamp(item, issued_us)
        if self.rank == self.world - 1 and item.emits is not None:
            return self._tokens_later(item) if st.cuda else self._tokens(item)
        return None

    def _stamp(self, item: Item, issued_us: int) -> None:
        """One `pp item` line per item: when this stage issued it and when it left the device (its kernels and the copy
        into the send twin), on this process's clock. On a GPU the end is an event resolved later, when it has
        happened, so the stage never waits for its own stamp. `serve/pp_timeline.py` reads the lines of all stages."""
        rows = int(item.vars.get("tokens", item.vars.get("rows", item.groups)) or 0)
        if self.st.cuda:
            if self._t0 is None:
                self._t0 = (torch.cuda.Event(enable_timing=True), time.perf_counter_ns() // 1000)
                self._t0[0].record(self.st.compute)
                self._t0[0].synchronize()
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(self.st.compute)
            self._stamps.append((item.k, rows, issued_us, ev))
            while self._stamps and self._stamps[0][3].query():
                k, r, iu, e = self._stamps.pop(0)
                self._emit(k, r, iu, self._t0[1] + int(self._t0[0].elapsed_time(e) * 1e3))
        else:
            self._emit(item.k, rows, issued_us, time.perf_counter_ns() // 1000)

    def _emit(self, k: int, rows: int, issued_us: int, done_us: int) -> None:
        self.timeline.append((k, rows, issued_us, max(done_us, issued_us)))
        log.debug("pp item stage=%d item=%d rows=%d issued_us=%d done_us=%d", self.rank, k, rows, issued_us, max(done_us, issued_us))

    def flush_stamps(self) -> None:
        """Resolve the stamps still pending (after a synchronize: at the end of a run)."""
        while self._stamps:
            k, r, iu, e = self._stamps.pop(0)
            e.synchronize()
            self._emit(k, r, iu, self._t0[1] + int(self._t0[0].elapsed_time(e) * 1e3))

    def _tokens_later(self, item: Item):
        """GPU: copy the item's outputs to pinned memory behind its kernels and hand back something to wait on — the
        host goes on to the next item at once (a read that waited here would hold the whole pipeline to one item)."""
        n = item.groups * item.width
        slot = self._pinned[item.k % len(self._pinned)] if getattr(self, "_pinned", None) else None
        if slot is None:
            self._pinned = [{} for _ in range(8)]
            slot = self._pinned[item.k % 8]
        with self.st.on(self.st.compute):
            out = {}
            for name in [item.emits] + ([item.count] if item.count else []):
                src = self.rt.tensor(name).view(-1)
                dst = slot.get(name)
                if dst is None or dst.numel() < src.numel():
                    dst = slot[name] = torch.empty(src.numel(), dtype=src.dtype, pin_memory=True)
                m = n if name == item.emits else item.groups
                dst[:m].copy_(src[:m], non_blocking=True)
                out[name] = dst
            ev = torch.cuda.Event()
            ev.record(self.st.compute)
        return _Pending(item, ev, out)

    def finish(self, pending) -> list:
        """Wait (with the deadline) for a pending read and decode it."""
        if not isinstance(pending, _Pending):
            return pending
        deadline = time.monotonic() + self.timeout
        while not pending.event.query():
            if time.monotonic() > deadline:
                raise StageTimeout(f"stage {self.rank}: item {pending.item.k} did not finish within {self.timeout:.0f} s")
            time.sleep(0.0002)
        item = pending.item
        toks = pending.out[item.emits][: item.groups * item.width].numpy().reshape(item.groups, item.width)
        if item.count is not None:
            cnt = pending.out[item.count][: item.groups].numpy()
            return [toks[i, : int(cnt[i])].tolist() for i in range(item.real)]
        return [toks[i, :1].tolist() for i in range(item.real)]

    def _peer(self, stage: int) -> int:
        return dist.get_global_rank(self.data_pg, stage) if self.data_pg is not None else stage

    def _tokens(self, item: Item):
        self._sync(f"stage {self.rank}: item {item.k} did not finish")
        toks = np.asarray(self.rt.read(item.emits, item.groups * item.width)).reshape(item.groups, item.width)
        if item.count is not None:
            cnt = np.asarray(self.rt.read(item.count, item.groups))
            return [toks[i, : int(cnt[i])].tolist() for i in range(item.real)]
        return [toks[i, :1].tolist() for i in range(item.real)]

    def _sync(self, what: str) -> None:
        """Wait for the compute stream with a deadline (a GPU rank polls an event; a CPU rank has nothing in flight)."""
        if not self.st.cuda:
            return
        ev = torch.cuda.Event()
        ev.record(self.st.compute)
        deadline = time.monotonic() + self.timeout
        while not ev.query():
            if time.monotonic() > deadline:
                raise StageTimeout(f"{what} within {self.timeout:.0f} s")
            time.sleep(0.0002)

    def drain(self) -> None:
        for tw in self.sends:
            for w in tw:
                self._wait(w, f"stage {self.rank}: the last items were not taken by stage {self.rank + 1}")
        self.sends = [[] for _ in range(LANDINGS)]
        if self.st.cuda:
            self._sync(f"stage {self.rank}: drain")
            self.st.send.synchronize()
            self.st.recv.synchronize()
            self.flush_stamps()                 # the items' end stamps that were still pending


@dataclass
class _Pending:
    item: Item
    event: object
    out: dict


def _timedelta(seconds: float):
    import datetime

    return datetime.timedelta(seconds=seconds)


# ---- the control plane: the head announces items, the last stage reports tokens ---------------------------------------
class Pipeline:
    """One pipeline over the ranks of `pg` (default: the world). Stage 0 is the head: it owns the pool and packs items;
    every rank calls `serve()` except the head, which drives `prefill` / `step` and finally `stop()`."""

    def __init__(self, rt, docs: list[dict], whole_protocol: dict, data_pg=None, ctrl_pg=None, report_pg=None, ahead: int = 4,
                 timeout: float = TIMEOUT, unit: int | None = None, pages: int | None = None, slots: int | None = None):
        """`ctrl_pg`: a host-side (gloo) group of every stage, for the head's announcements. `report_pg`: a host-side
        group of the head and the last stage only; the head listens on it from a thread of its own, so the last
        stage's reports never wait for the head's main thread (which may itself be waiting in an announcement)."""
        self.rank = dist.get_rank(data_pg)
        self.world = len(docs)
        self.stage = Stage(rt, docs, self.rank, data_pg, ctrl_pg, timeout)
        self.p = whole_protocol
        self.ctrl_pg, self.report_pg, self.ahead, self.timeout = ctrl_pg, report_pg, ahead, timeout
        self.k = 0
        self.reported = 0
        self.results: dict[int, list] = {}
        self._inbox = None
        if self.rank == 0 and self.world > 1:
            import queue
            import threading

            self._inbox = queue.Queue()
            threading.Thread(target=self._watch, daemon=True, name="kern-pp-reports").start()
        if self.rank == 0:
            # one pool at the head: page and slot ids mean the same on every stage (same geometry everywhere)
            self.unit = unit or rt.page_unit
            row_pages = min((t["width"] * t["stride"] // self.unit for t in whole_protocol["page_tables"]), default=0)
            self.pool = _native.Pool(self.unit, pages if pages is not None else rt.pages, slots if slots is not None else rt.slots, row_pages)

    # -- wire: length-prefixed JSON over point-to-point host messages (a stage that has stopped cannot block the others) --
    def _send_json(self, text: str, stage: int) -> None:
        raw = torch.frombuffer(bytearray(text.encode()), dtype=torch.uint8)
        dst = self._ctrl_rank(stage)
        for t in (torch.tensor([raw.numel()], dtype=torch.int64), raw):
            w = dist.isend(t, dst=dst, group=self.ctrl_pg)
            try:
                done = w.wait(timeout=_timedelta(self.timeout))
            except RuntimeError as e:
                raise StageTimeout(f"head: stage {stage} took no announcement for {self.timeout:.0f} s") from e
            if done is False:
                raise StageTimeout(f"head: stage {stage} took no announcement for {self.timeout:.0f} s")

    def _recv_json(self, stage: int) -> str:
        src = self._ctrl_rank(stage)
        n = torch.zeros(1, dtype=torch.int64)
        dist.recv(n, src=src, group=self.ctrl_pg)
        raw = torch.empty(int(n.item()), dtype=torch.uint8)
        dist.recv(raw, src=src, group=self.ctrl_pg)
        return bytes(raw.numpy()).decode()

    def _announce(self, item: Item) -> None:
        text = item.to_wire()
        for stage in range(1, self.world):
            self._send_json(text, stage)

    def _hear(self) -> Item:
        return Item.from_wire(self._recv_json(0))

    def _ctrl_rank(self, stage: int) -> int:
        return dist.get_global_rank(self.ctrl_pg, stage) if self.ctrl_pg is not None else stage

    def _report(self, item: Item, toks) -> None:
        """Last stage -> head: the item's number and its tokens (an empty list when it emits nothing)."""
        if self.world == 1:
            self.results[item.k] = toks
            return
        head = dist.get_global_rank(self.report_pg, 0) if self.report_pg is not None else 0
        dist.send_object_list([json.dumps({"k": item.k, "tokens": toks})], dst=head, group=self.report_pg)

    def _watch(self) -> None:
        """Head, on its own thread: take the last stage's reports as they come."""
        last = dist.get_global_rank(self.report_pg, 1) if self.report_pg is not None else self.world - 1
        while True:
            box = [None]
            try:
                dist.recv_object_list(box, src=last, group=self.report_pg)
            except Exception as e:      # noqa: BLE001  (the group went away: the pipeline is shutting down or broken)
                self._inbox.put({"k": -2, "error": repr(e)})
                return
            r = json.loads(box[0])
            self._inbox.put(r)
            if r["k"] < 0:
                return

    def _collect(self, upto: int) -> None:
        """Head: take reports until item `upto` is in; nothing for `timeout` seconds means a stage has stopped."""
        import queue

        while self.reported <= upto:
            try:
                r = self._inbox.get(timeout=self.timeout)
            except queue.Empty:
                raise StageTimeout(f"head: no report of item {self.reported} from the last stage within {self.timeout:.0f} s") from None
            if r["k"] < 0:
                raise StageTimeout(f"head: the report channel closed ({r.get('error', 'stop')})")
            self.results[r["k"]] = r["tokens"]
            self.reported = r["k"] + 1

    # -- every stage but the head --
    def serve(self) -> int:
        """Run announced items until the head says stop; returns how many. Announcements arrive on a listener thread
        and (on the last stage) reports leave on a reporter thread, so the loop below only ever issues device work."""
        import queue
        import threading

        items: queue.Queue = queue.Queue()
        outbox: queue.Queue = queue.Queue()
        failure: list = []

        def listen():
            try:
                while True:
                    it = self._hear()
                    items.put(it)
                    if it.stop:
                        return
            except Exception as e:      # noqa: BLE001
                failure.append(e)
                items.put(Item(k=-1, program="", vars={}, columns={}, stop=True))

        def report():
            try:
                while True:
                    got = outbox.get()
                    if got is None:
                        return
                    item, pending = got
                    self._report(item, self.stage.finish(pending) if pending is not None else [])
            except Exception as e:      # noqa: BLE001
                failure.append(e)

        threading.Thread(target=listen, daemon=True, name="kern-pp-listen").start()
        last = self.rank == self.world - 1
        reporter = None
        if last:
            reporter = threading.Thread(target=report, daemon=True, name="kern-pp-report")
            reporter.start()
        n = 0
        while True:
            item = items.get()
            if failure:
                raise failure[0]
            if item.stop:
                self.stage.drain()
                if last:
                    outbox.put(None)
                    reporter.join(timeout=self.timeout)
                    if failure:
                        raise failure[0]
                    self._report(Item(k=-1, program="", vars={}, columns={}), [])        # lets the head's listener go
                return n
            pending = self.stage.run(item)
            if last:
                outbox.put((item, pending))
            n += 1

    # -- the head --
    def submit(self, batch, pad: int = 0, round: bool = False) -> int:
        """Announce one call over `[(sequence, new tokens)]` and run the head's part; returns the item number."""
        entries = [fills.Entry(length=s.length, new=new, pages=s.lease.pages, slot=s.lease.slot,
                               slots=s.lease.slots_of(s.length, s.length + len(new)), sampling=s.sampling) for s, new in batch]
        call = fills.build(self.p, self.unit, entries, pad, round=round)
        fw = call.forward
        ef = next((f for f in self.p["fills"] if f["name"] == fw["emits"]), None) if fw["emits"] else None
        item = Item(k=self.k, program=call.program, vars=call.vars,
                    columns={n: [dt, np.asarray(col).tolist()] for n, (dt, col) in call.columns.items()},
                    emits=fw["emits"], count=fw["count"], groups=call.groups, real=call.real, width=ef["width"] if ef else 1)
        if self.k - self.reported >= self.ahead and self.world > 1:
            self._collect(self.k - self.ahead)                     # at most `ahead` items unreported
        if self.world > 1:
            self._announce(item)
        toks = self.stage.run(item)
        if self.world == 1:
            self._report(item, self.stage.finish(toks) if toks is not None else [])
            self.reported = self.k + 1
        for s, new in batch:
            s.length += len(new)
            s.tokens.extend(new)
        self.k += 1
        return item.k

    def tokens(self, k: int):
        """The tokens item `k` emitted (waits for the last stage's report)."""
        if self.world > 1:
            self._collect(k)
        return self.results.pop(k)

    def open(self, tokens_capacity: int, sampling=None):
        from ..engine import Sequence

        lease = self.pool.lease(tokens_capacity)
        return Sequence(lease=lease, sampling=sampling or fills.Sampling())

    def prefill(self, seq, prompt: list[int], chunk: int) -> list[int]:
        """A prompt through the pipeline in chunks, all of them in flight at once (up to `ahead`); the last chunk's token."""
        last = None
        for i in range(0, len(prompt), chunk):
            last = self.submit([(seq, prompt[i:i + chunk])])
        return self.tokens(last)[0]

    def stop(self) -> None:
        if self.world > 1:
            if self.reported < self.k:
                self._collect(self.k - 1)
            self._announce(Item(k=self.k, program="", vars={}, columns={}, stop=True))
        self.stage.drain()


class HeadEngine:
    """The engine interface (open / close / step, `.pool`, bounds) over a `Pipeline`, for the scheduler that runs in the
    head's process: a step is one announced item; a step whose tokens nobody wants (`read=False`: unfinished prompt
    chunks) is not waited for, so a long prompt's chunks follow one another through the stages.
    Prefix checkpoints copy pages on every stage's own pool: not carried over the pipeline, so the scheduler above runs
    with `prefix_cache=False`."""

    class _NoCopies:
        def run_copies(self, copies: dict) -> None:
            if copies.get("pages") or copies.get("slot") is not None:
                raise NotImplementedError("page copies are not carried over a pipeline: run its scheduler with prefix_cache=False")

        def zero_slot(self, slot: int) -> None:
            raise NotImplementedError("per-sequence state slots are not zeroed over a pipeline yet")

    def __init__(self, pipe: Pipeline):
        self.pipe, self.p, self.pool, self.unit = pipe, pipe.p, pipe.pool, pipe.unit
        self.rt = self._NoCopies()
        self.rows_max, self.groups_max = self.p["rows"]["max"], self.p["groups"]["max"]
        self.forwards, self.page_tables = self.p["forwards"], self.p["page_tables"]
        self.steps = 0

    def open(self, tokens_capacity: int, sampling=None):
        return self.pipe.open(tokens_capacity, sampling)

    def close(self, seq) -> None:
        seq.lease.release()

    def step(self, batch, eager: bool = False, read: bool = True, timed: bool = False, pad: int = 0, round: bool = False):
        if not batch or sum(len(t) for _, t in batch) == 0:
            return []
        k = self.pipe.submit(batch, pad=pad, round=round)
        self.steps += 1
        if not read:
            return None
        toks = self.pipe.tokens(k)
        for old in [x for x in self.pipe.results if x < k]:       # reports of calls nobody read
            del self.pipe.results[old]
        return toks[: len(batch)] if toks is not None else None
