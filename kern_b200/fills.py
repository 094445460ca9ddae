"""Pure construction of one call's inputs from the manifest's protocol projection.

``build(protocol, unit, batch, pad)`` turns "these sequences each get these new tokens" into the host columns
of every fill and table the protocol names, the var assignment and the forward program to run. It touches no
runtime: the local engine writes the columns to its own device, a serving head ships them to rank processes.
Reference counterpart: crates/kern-run/src/lib.rs:111-258 (``fills``, table rows).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


@dataclass
class Sampling:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    seed: int = 0


@dataclass
class Entry:
    """One sequence of a call: where it stands, what it is fed, where its memory is."""
    length: int                       # positions already in the states
    new: list[int]                    # tokens fed by this call
    pages: list[int]                  # page ids of its lease, in order
    slot: int = -1                    # per-sequence state slot (-1: none)
    slots: np.ndarray | None = None   # KV slot of every new row (from the lease)
    sampling: Sampling = field(default_factory=Sampling)


@dataclass
class Call:
    program: str
    forward: dict
    vars: dict[str, int]
    columns: dict[str, tuple[str, np.ndarray]]     # input name -> (dtype, flat values)
    groups: int
    real: int


def forward_for(protocol: dict, groups: int, rows_each: list[int], round: bool = False) -> dict:
    """The forward program for a call of this shape. A speculative round (a fixed-shape forward of several rows per
    sequence that reports a `count`) is taken only when the caller asks for one: a prefill chunk that happens to be as
    long as a round is still a prefill chunk."""
    r0 = rows_each[0]
    if all(r == r0 for r in rows_each):
        for f in protocol["forwards"]:
            if f["rows"] == r0 and groups <= f["groups"] and (round or r0 == 1 or f["count"] is None):
                return f
    for f in protocol["forwards"]:
        if f["rows"] == "var" and groups <= f["groups"]:
            return f
    raise ValueError(f"no program takes {groups} sequences of rows {sorted(set(rows_each))}")


def build(p: dict, unit: int, batch: list[Entry], pad: int = 0, page_map=None, round: bool = False,
          pad_entry: Entry | None = None) -> Call:
    """``pad`` extra sequences of the first one's row count bring a fixed-shape call up to a bucket; their outputs are
    dropped. With ``pad_entry`` (a page and a state slot no sequence owns) they are ordinary rows that write there:
    token 0 at positions 0.., the pad page's slots, a context of their own rows — the package format's convention
    (crates/kern-serve/src/ranks.rs:301-355, scheduler.rs:35-38), which kernels written for it rely on. Without one
    they are dead rows: slot -1 (nothing appended), context 0 (nothing attended), which this package's own kernels skip.
    ``page_map(entry) -> pages`` lets a head substitute one member rank's page ids (default: ``entry.pages``)."""
    real = len(batch)
    rows_each = [len(e.new) for e in batch] + [len(batch[0].new)] * pad
    b = real + pad
    total = sum(rows_each)
    rows_max, groups_max = p["rows"]["max"], p["groups"]["max"]
    if total > rows_max or b > groups_max:
        raise ValueError(f"call of {b} sequences / {total} rows exceeds the manifest's {groups_max} / {rows_max}")
    fw = forward_for(p, b, rows_each, round)
    tok = np.zeros(total, np.int64)
    pos = np.zeros(total, np.int64)
    slot = np.full(total, -1, np.int64)
    seq_len = np.zeros(b, np.int64)
    cu = np.zeros(b + 1, np.int64)
    at = 0
    for i, e in enumerate(batch):
        n = len(e.new)
        tok[at:at + n] = e.new
        pos[at:at + n] = np.arange(e.length, e.length + n)
        if e.slots is not None:
            slot[at:at + n] = e.slots
        seq_len[i] = e.length + n
        at += n
        cu[i + 1] = at
    for i in range(real, b):
        n = rows_each[i]
        if pad_entry is not None:
            pos[at:at + n] = np.arange(n)
            if pad_entry.slots is not None:
                slot[at:at + n] = pad_entry.slots[:n]
            seq_len[i] = n
        at += n
        cu[i + 1] = at
    fills: dict[str, list] = {}
    for f in p["fills"]:
        fills.setdefault(f["fill"], []).append(f)
    cols: dict[str, tuple[str, np.ndarray]] = {}
    for f in fills.get("token", []):
        cols[f["name"]] = (f["dtype"], np.array([e.new[0] for e in batch] + [0] * pad, np.int64) if f["axis"] == "groups" else tok)
    for kind, col in (("position", pos), ("slot", slot), ("seq_len", seq_len), ("valid", np.ones(total, np.int64))):
        for f in fills.get(kind, []):
            cols[f["name"]] = (f["dtype"], col)
    for f in fills.get("cu_seqlens", []):
        cols[f["name"]] = (f["dtype"], cu)
    if "temperature" in fills:
        sm = [e.sampling for e in batch] + [Sampling()] * pad
        for kind, vals in (("temperature", [x.temperature for x in sm]), ("top_k", [x.top_k for x in sm]),
                           ("top_p", [x.top_p for x in sm]), ("min_p", [x.min_p for x in sm]), ("seed", [x.seed for x in sm])):
            f = fills[kind][0]
            cols[f["name"]] = (f["dtype"], np.array(vals))
    for t in p["page_tables"]:
        w = t["width"]
        per = t["stride"] // unit           # pool pages per table entry
        rows = np.zeros((b, w), np.int32)
        for i, e in enumerate(batch):
            pg = page_map(e) if page_map else e.pages
            ids = pg[::per] if per > 1 else pg
            m = min(len(ids), w)
            rows[i, :m] = np.asarray(ids[:m], np.int32) // per if per > 1 else ids[:m]
        if pad_entry is not None and b > real:
            pg = page_map(pad_entry) if page_map else pad_entry.pages
            ids = pg[::per] if per > 1 else pg
            m = min(len(ids), w)
            rows[real:, :m] = np.asarray(ids[:m], np.int32) // per if per > 1 else ids[:m]
        cols[t["name"]] = ("i32", rows.reshape(-1))
    for t in p.get("line_tables", []):
        # [lines, groups(, w)]: line 0 of a sequence is its own state slot; the rest stay null (0)
        rows = np.zeros((t["lines"], b, t["width"]), np.int32)
        for i, e in enumerate(batch):
            rows[0, i, 0] = max(0, e.slot)
        if pad_entry is not None:
            rows[0, real:, 0] = max(0, pad_entry.slot)
        cols[t["name"]] = ("i32", rows.reshape(-1))
    vars_ = {p["rows"]["var"]: total, p["groups"]["var"]: b}
    if p.get("ranks"):
        vars_[p["ranks"]["var"]] = total
    if p.get("context"):
        vars_[p["context"]["var"]] = int(seq_len.max())
    return Call(program=fw["name"], forward=fw, vars=vars_, columns=cols, groups=b, real=real)
