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

from . import _native

_NP = {"i32": np.int32, "i64": np.int64, "f32": np.float32}
_TT = {"i32": torch.int32, "i64": torch.int64, "f32": torch.float32}


@dataclass
class Sampling:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    seed: int = 0


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

    # ---- sequences ----
    def open(self, tokens_capacity: int, sampling: Sampling | None = None) -> Sequence:
        """Lease room for a sequence that will hold up to ``tokens_capacity`` positions."""
        lease = self.pool.lease(tokens_capacity)
        if lease.slot >= 0:
            self.rt.zero_slot(lease.slot)
        return Sequence(lease=lease, sampling=sampling or Sampling())

    def close(self, seq: Sequence) -> None:
        seq.lease.release()

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

    def forward_for(self, groups: int, rows_each: list[int]):
        r0 = rows_each[0]
        if all(r == r0 for r in rows_each):
            for f in self.forwards:
                if f["rows"] == r0 and groups <= f["groups"]:
                    return f
        for f in self.forwards:
            if f["rows"] == "var" and groups <= f["groups"]:
                return f
        raise ValueError(f"no program takes {groups} sequences of rows {sorted(set(rows_each))}")

    def step(self, batch: list[tuple[Sequence, list[int]]], eager: bool = False, read: bool = True, timed: bool = False,
             pad: int = 0):
        """Feed each sequence its new tokens; returns, per sequence, the tokens the call emitted for it
        (one for a plain step, up to ``count`` for a speculative round), or None when ``read`` is off
        or the program emits nothing."""
        real = len(batch)
        rows_each = [len(t) for _, t in batch]
        if real == 0 or sum(rows_each) == 0:
            return []
        # `pad` dead sequences of the same row count bring a fixed-shape call up to a bucket: token 0 at
        # position 0, slot -1 (nothing appended), context 0 (nothing attended); their outputs are dropped
        rows_each += [rows_each[0]] * pad
        b = real + pad
        total = sum(rows_each)
        if total > self.rows_max or b > self.groups_max:
            raise ValueError(f"call of {b} sequences / {total} rows exceeds the manifest's {self.groups_max} / {self.rows_max}")
        fw = self.forward_for(b, rows_each)
        tok = np.empty(total, np.int64)
        pos = np.empty(total, np.int64)
        slot = np.empty(total, np.int64)
        seq_len = np.empty(b, np.int64)
        cu = np.zeros(b + 1, np.int64)
        at = 0
        for i, (s, new) in enumerate(batch):
            n = len(new)
            tok[at:at + n] = new
            pos[at:at + n] = np.arange(s.length, s.length + n)
            slot[at:at + n] = s.lease.slots_of(s.length, s.length + n)
            seq_len[i] = s.length + n
            at += n
            cu[i + 1] = at
        for i in range(real, b):
            n = rows_each[i]
            tok[at:at + n], pos[at:at + n], slot[at:at + n], seq_len[i] = 0, 0, -1, 0
            at += n
            cu[i + 1] = at
        longest = int(seq_len.max())
        for f in self.fills.get("token", []):
            if f["axis"] == "groups":
                self._write(f["name"], f["dtype"], np.array([t[0] for _, t in batch] + [0] * pad, np.int64))
            else:
                self._write(f["name"], f["dtype"], tok)
        cols = {"position": pos, "slot": slot, "seq_len": seq_len, "valid": np.ones(total, np.int64)}
        for kind, col in cols.items():
            for f in self.fills.get(kind, []):
                self._write(f["name"], f["dtype"], col)
        for f in self.fills.get("cu_seqlens", []):
            self._write(f["name"], f["dtype"], cu)
        if "temperature" in self.fills:
            sm = [s.sampling for s, _ in batch] + [Sampling()] * pad
            for kind, vals in (("temperature", [x.temperature for x in sm]), ("top_k", [x.top_k for x in sm]),
                               ("top_p", [x.top_p for x in sm]), ("min_p", [x.min_p for x in sm]), ("seed", [x.seed for x in sm])):
                f = self.fills[kind][0]
                self._write(f["name"], f["dtype"], np.array(vals))
        for t in self.page_tables:
            w = t["width"]
            per = t["stride"] // self.unit           # pool pages per table entry
            rows = np.zeros((b, w), np.int32)
            for i, (s, _) in enumerate(batch):
                pg = s.lease.pages
                ids = pg[::per] if per > 1 else pg
                m = min(len(ids), w)
                rows[i, :m] = np.asarray(ids[:m], np.int32) // per if per > 1 else ids[:m]
            self._write(t["name"], "i32", rows.reshape(-1))
        for t in self.p.get("line_tables", []):
            # [lines, groups(, w)]: line 0 of a sequence is its own state slot; the rest stay null (0)
            rows = np.zeros((t["lines"], b, t["width"]), np.int32)
            for i, (s, _) in enumerate(batch):
                rows[0, i, 0] = max(0, s.lease.slot)
            self._write(t["name"], "i32", rows.reshape(-1))
        vars_ = {self.p["rows"]["var"]: total, self.p["groups"]["var"]: b}
        if self.p.get("ranks"):
            vars_[self.p["ranks"]["var"]] = total
        if self.p.get("context"):
            vars_[self.p["context"]["var"]] = longest
        if timed:     # cost by call, eagerly, with an event between calls
            self.last_times = self.rt.issue_timed(fw["name"], vars_)
            launches = sum(t[3] for t in self.last_times)
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
