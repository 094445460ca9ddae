"""The batch driver: turns "these sequences each get these new tokens" into one runtime call.

It knows no buffer, program or var name: everything it writes or reads is found through the manifest's
protocol projection (fills, page tables, forwards), exactly as the reference's drivers do
(crates/kern-run/src/lib.rs:111-258 ``fills`` / table rows; :421-555 ``Caller``).

One step = (1) build each fill's column for the call in pinned host memory, (2) copy them to the
device on the runtime's stream, (3) issue the forward program whose row shape matches (a captured
graph for fixed-shape programs), (4) read the tokens the call emits back to the host.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from . import _native, fills

_NP = {"i32": np.int32, "i64": np.int64, "f32": np.float32}
_TT = {"i32": torch.int32, "i64": torch.int64, "f32": torch.float32}


Sampling = fills.Sampling


@dataclass
class Sequence:
    """One sequence's place in the pool: its lease and how many positions it has filled."""
    lease: object
    length: int = 0                      # positions already in the states
    sampling: Sampling = field(default_factory=Sampling)
    tokens: list[int] = field(default_factory=list)   # everything fed or produced so far (for prefix keys)


class Engine:
    def __init__(self, rt, pool: "_native.Pool | None" = None):
        self.rt = rt
        self.probe = None      # a testing.probe.Probe: steps run call range by call range and dump activations
        p = rt.protocol
        if p is None:
            raise ValueError("the manifest has no serving protocol (no program declares a `batch`)")
        self.p = p
        self.rows_max, self.groups_max = p["rows"]["max"], p["groups"]["max"]
        self.fills = {}
        for f in p["fills"]:
            self.fills.setdefault(f["fill"], []).append(f)
        self.page_tables = p["page_tables"]
        self.unit = rt.page_unit
        row_pages = min((t["width"] * t["stride"] // self.unit for t in self.page_tables), default=0)
        self.pool = pool or _native.Pool(self.unit, rt.pages, rt.slots, row_pages)
        self.forwards = p["forwards"]
        self._pinned: dict[str, torch.Tensor] = {}
        self._out: dict[str, torch.Tensor] = {}
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.steps = 0
        self._pad: Sequence | None = None     # a page (and a state slot) no sequence owns, leased on the first padded call
        self._pad_denied = False

    # ---- sequences ----
    def open(self, tokens_capacity: int, sampling: Sampling | None = None) -> Sequence:
        """Lease room for a sequence that will hold up to ``tokens_capacity`` positions."""
        lease = self.pool.lease(tokens_capacity)
        if lease.slot >= 0:
            self.rt.zero_slot(lease.slot)
        return Sequence(lease=lease, sampling=sampling or Sampling())

    def close(self, seq: Sequence) -> None:
        seq.lease.release()

    @property
    def pad_pages(self) -> int:
        """Pages held by the pad lease (0 until a call was padded)."""
        return len(self._pad.lease.pages) if self._pad is not None else 0

    def _pad_entry(self, rows: int):
        """The entry padding rows write to: a lease of its own, taken once. When the pool has no page to spare the
        call falls back to dead rows (slot -1, context 0), which only this package's own kernels are built to skip."""
        if self._pad is None and not self._pad_denied:
            widest = max([f["rows"] for f in self.forwards if f["rows"] != "var"] + [rows])
            try:
                self._pad = self.open(widest)
            except _native.Denied:
                self._pad_denied = True
        if self._pad is None:
            return None
        l = self._pad.lease
        return fills.Entry(length=0, new=[0] * rows, pages=l.pages, slot=l.slot, slots=l.slots_of(0, rows))

    # ---- one call ----
    def _buf(self, name: str, dtype: str, n: int) -> torch.Tensor:
        t = self._pinned.get(name)
        if t is None or t.numel() < n:
            t = torch.empty(max(n, 16), dtype=_TT[dtype], pin_memory=torch.cuda.is_available())
            self._pinned[name] = t
        return t

    def _write(self, name: str, dtype: str, values: np.ndarray) -> None:
        t = self._buf(name, dtype, len(values))
        t.numpy()[: len(values)] = values
        self.rt.write(name, t[: len(values)])
        self.h2d_bytes += len(values) * t.element_size()

    def forward_for(self, groups: int, rows_each: list[int], round: bool = False):
        return fills.forward_for(self.p, groups, rows_each, round)

    def step(self, batch: list[tuple[Sequence, list[int]]], eager: bool = False, read: bool = True, timed: bool = False,
             pad: int = 0, round: bool = False):
        """Feed each sequence its new tokens; returns, per sequence, the tokens the call emitted for it
        (one for a plain step, up to ``count`` for a speculative round), or None when ``read`` is off
        or the program emits nothing. ``pad`` dead sequences bring a fixed-shape call up to a bucket; ``round`` asks for
        the speculative-round program (every sequence is fed the round's row count)."""
        real = len(batch)
        if real == 0 or sum(len(t) for _, t in batch) == 0:
            return []
        entries = [fills.Entry(length=s.length, new=new, pages=s.lease.pages, slot=s.lease.slot,
                               slots=s.lease.slots_of(s.length, s.length + len(new)), sampling=s.sampling)
                   for s, new in batch]
        call = fills.build(self.p, self.unit, entries, pad, round=round,
                           pad_entry=self._pad_entry(len(batch[0][1])) if pad > 0 else None)
        for name, (dtype, col) in call.columns.items():
            self._write(name, dtype, col)
        fw, vars_, b = call.forward, call.vars, call.groups
        if timed:     # cost by call, eagerly, with an event between calls
            self.last_times = self.rt.issue_timed(fw["name"], vars_)
            launches = sum(t[3] for t in self.last_times)
        elif self.probe is not None:     # call range by call range, dumping what the asked-for calls wrote
            launches = self.probe.run(self.rt, fw["name"], vars_, f"step{self.steps:04d}")
        else:
            launches = self.rt.issue(fw["name"], vars_, eager)
        for s, new in batch:
            s.length += len(new)
            s.tokens.extend(new)
        self.steps += 1
        self.last_launches = launches
        if not read or fw["emits"] is None:
            return None
        return self.read_tokens(fw, b)[:real]

    def read_tokens(self, fw, b: int):
        ef = next(f for f in self.p["fills"] if f["name"] == fw["emits"])
        w = ef["width"]
        out = self._out.get(ef["name"])
        if out is None or out.numel() < b * w:
            out = torch.empty(max(self.groups_max * w, 16), dtype=_TT[ef["dtype"]], pin_memory=torch.cuda.is_available())
            self._out[ef["name"]] = out
        self.rt.read(ef["name"], out=out[: b * w])
        self.d2h_bytes += b * w * out.element_size()
        toks = out[: b * w].numpy().reshape(b, w)
        if fw["count"] is not None:
            cf = next(f for f in self.p["fills"] if f["name"] == fw["count"])
            cnt = self.rt.read(cf["name"], b)
            self.d2h_bytes += b * cnt.itemsize
            return [toks[i, : int(cnt[i])].tolist() for i in range(b)]
        return [toks[i, :1].tolist() for i in range(b)]

    # ---- whole-sequence helpers (the single-sequence `Caller`) ----
    def generate(self, prompt: list[int], steps: int, chunk: int | None = None, sampling: Sampling | None = None) -> list[int]:
        """bs = 1: chunked prefill, then `steps` tokens one decode call each."""
        chunk = chunk or self.rows_max
        seq = self.open(len(prompt) + steps, sampling)
        try:
            out = None
            for i in range(0, len(prompt), chunk):
                out = self.step([(seq, prompt[i:i + chunk])])
            toks = [out[0][0]]
            while len(toks) < steps:
                toks.append(self.step([(seq, [toks[-1]])])[0][0])
            return toks
        finally:
            self.close(seq)
