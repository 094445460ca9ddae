"""Pipeline parallelism over a cut manifest: every stage is a runtime of its own (its layers' weights and states on
its own GPU), a call walks the stages in order and the workspaces that are live across a cut travel from one stage's
outputs into the next stage's exported inputs. The head owns the one pool and the one prefix cache: page and slot
ids mean the same thing on every stage, because every stage is given the same geometry.

`PipelineEngine` has the engine interface (open / close / step, `.pool`, `.rt.run_copies / zero_slot`), so the same
scheduler, server and tiers run on top of it. Stages may be host-memory runtimes (tests), GPU runtimes in this
process (one per device; the transfer is a device-to-device copy), or rank processes behind executors.
Reference counterpart: crates/kern-serve/src/pp/mod.rs:84-141 (jobs), pp/stage.rs:41-192 (a stage's loop),
pp/head.rs:941-1049 (chunks through the stages), crates/kern-manifest/src/cut.rs:79-282 (the cut itself).
"""
from __future__ import annotations

import json

import numpy as np

from .. import _native, fills


def layer_cuts(doc: dict, stages: int, program: str | None = None) -> list[int]:
    """Call indices that split a decoder's program into `stages` runs of whole layers (labels `l<i>.`)."""
    progs = [p for p in doc["programs"].values() if p.get("batch")]
    calls = (doc["programs"][program] if program else progs[0])["calls"]
    first = {}
    for i, c in enumerate(calls):
        lbl = c.get("label", "")
        if lbl.startswith("l") and "." in lbl and lbl[1:lbl.index(".")].isdigit():
            first.setdefault(int(lbl[1:lbl.index(".")]), i)
    layers = len(first)
    if stages < 2 or stages > layers:
        raise ValueError(f"{layers} layers cannot make {stages} stages")
    return [first[(layers * s) // stages] for s in range(1, stages)]


def cut(doc: dict, at: list[int]) -> list[dict]:
    m, errs = _native.verify(json.dumps(doc))
    if m is None:
        raise ValueError("manifest does not verify:\n  - " + "\n  - ".join(errs))
    return [json.loads(s.to_json()) for s in m.cut(at)]


def _bytes_for(buf: dict, vars_: dict, vmax: dict) -> int:
    es = {"bf16": 2, "f16": 2, "f32": 4, "i32": 4, "u32": 4, "i64": 8, "u64": 8, "u8": 1, "i8": 1}[buf["dtype"]]
    n = es
    for i, d in enumerate(buf["shape"]):
        # only the leading var dim shrinks with the call; inner var dims keep their max so rows stay in place
        n *= (vars_.get(d, vmax[d]) if i == 0 else vmax[d]) if isinstance(d, str) else d
    return n


class PipelineEngine:
    class _AllStages:
        def __init__(self, stages):
            self.stages = stages

        def run_copies(self, copies: dict) -> None:
            for rt in self.stages:
                rt.run_copies(copies)

        def zero_slot(self, slot: int) -> None:
            for rt in self.stages:
                rt.zero_slot(slot)

    def __init__(self, stages: list, protocol: dict, transfer=None):
        """`stages`: runtimes of the cut's stage manifests, in order, same page/slot geometry.
        `protocol`: the whole (uncut) manifest's projection. `transfer(src_rt, dst_rt, name, nbytes)` moves a
        crossing buffer; the default reads it to the host and writes it (host-memory runtimes)."""
        self.stages, self.p = stages, protocol
        # a stage without paged states reports a page of one token: the pipeline's page is the stages' largest
        self.unit = max(rt.page_unit for rt in stages)
        pages = min(rt.pages for rt in stages if rt.page_unit == self.unit)
        slots = min(rt.slots for rt in stages)
        row_pages = min((t["width"] * t["stride"] // self.unit for t in protocol["page_tables"]), default=0)
        self.pool = _native.Pool(self.unit, pages, slots, row_pages)
        self.rt = self._AllStages(stages)
        self.rows_max, self.groups_max = protocol["rows"]["max"], protocol["groups"]["max"]
        self.forwards, self.page_tables = protocol["forwards"], protocol["page_tables"]
        self.transfer = transfer or self._host_transfer
        self.crossing = []          # per boundary: names the next stage takes from this one
        for a, b in zip(stages, stages[1:]):
            outs = {n for n, x in a.doc["buffers"].items() if x["kind"] in ("output", "inout") and not x.get("fill")}
            self.crossing.append([n for n, x in b.doc["buffers"].items() if x.get("export") and n in outs])
        self.steps = 0
        self.moved_bytes = 0

    @staticmethod
    def _host_transfer(src, dst, name, nbytes) -> None:
        es = src.buffers[name].element_size()
        dst.buffers[name][: nbytes // es] = src.buffers[name][: nbytes // es]

    def open(self, tokens_capacity: int, sampling=None):
        from ..engine import Sequence

        lease = self.pool.lease(tokens_capacity)
        if lease.slot >= 0:
            self.rt.zero_slot(lease.slot)
        return Sequence(lease=lease, sampling=sampling or fills.Sampling())

    def close(self, seq) -> None:
        seq.lease.release()

    def step(self, batch, eager: bool = False, read: bool = True, timed: bool = False, pad: int = 0, round: bool = False):
        if not batch or sum(len(t) for _, t in batch) == 0:
            return []
        entries = [fills.Entry(length=s.length, new=new, pages=s.lease.pages, slot=s.lease.slot,
                               slots=s.lease.slots_of(s.length, s.length + len(new)), sampling=s.sampling) for s, new in batch]
        call = fills.build(self.p, self.unit, entries, pad, round=round)
        for si, rt in enumerate(self.stages):
            bufs = rt.doc["buffers"]
            for name, (dtype, col) in call.columns.items():
                if name in bufs and bufs[name]["kind"] == "input":
                    rt.write(name, np.ascontiguousarray(col.astype({"i32": np.int32, "i64": np.int64, "f32": np.float32}[dtype])))
            if si > 0:
                prev = self.stages[si - 1]
                vmax = {k: v["max"] for k, v in rt.doc["vars"].items()}
                for name in self.crossing[si - 1]:
                    n = _bytes_for(bufs[name], call.vars, vmax)
                    self.transfer(prev, rt, name, n)
                    self.moved_bytes += n
            rt.issue(call.program, {k: v for k, v in call.vars.items() if k in rt.doc["vars"]})
        for s, new in batch:
            s.length += len(new)
            s.tokens.extend(new)
        self.steps += 1
        fw = call.forward
        if not read or fw["emits"] is None:
            return None
        last = self.stages[-1]
        ef = next(f for f in self.p["fills"] if f["name"] == fw["emits"])
        w = ef["width"]
        toks = np.asarray(last.read(ef["name"], call.groups * w)).reshape(call.groups, w)
        if fw["count"] is not None:
            cnt = np.asarray(last.read(fw["count"], call.groups))
            return [toks[i, : int(cnt[i])].tolist() for i in range(call.real)]
        return [toks[i, :1].tolist() for i in range(call.real)]


def device_transfer(src, dst, name: str, nbytes: int) -> None:
    """Crossing buffer between two GPU runtimes of this process: a device-to-device copy ordered after the producing
    stage's stream and before the consuming stage's next call."""
    import torch

    src.synchronize()
    s, d = src.tensor(name).view(-1).view(torch.uint8), dst.tensor(name).view(-1).view(torch.uint8)
    d[:nbytes].copy_(s[:nbytes], non_blocking=True)
    torch.cuda.synchronize(d.device)
