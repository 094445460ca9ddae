"""Activation probes: the buffers a run's calls wrote, for comparing a manifest against an implementation outside
this engine.

A program is run call range by call range, cut after every call whose label equals or ends with one of the asked-for
labels, so nothing executes twice and the buffer that call wrote is read before the next range overwrites it. Each
probe lands in the directory as `<tag>.<label>.<buffer>.pt` (a CPU tensor of the buffer's live rows) and is listed in
`index.json` with its dtype and shape.
Reference: crates/kern-run/src/probe.rs:1-60 (`kern run --probe-dir`).
"""
from __future__ import annotations

import json
from pathlib import Path

import torch


class Probe:
    def __init__(self, directory, labels: str | list[str]):
        self.dir = Path(directory)
        self.dir.mkdir(parents=True, exist_ok=True)
        self.labels = [l for l in (labels.split(",") if isinstance(labels, str) else labels) if l]
        self.index: list[dict] = []

    def wants(self, label: str) -> bool:
        return any(label == l or label.endswith(l) for l in self.labels)

    @staticmethod
    def _written(doc: dict, call: dict) -> list[str]:
        """Names of the buffers a call writes (its `out` / `inout` buffer params), in param order."""
        out = []
        for a, pt in zip(call["args"], doc["ops"][call["op"]]["params"]):
            if isinstance(a, dict) and "buf" in a and pt.split()[0] in ("out", "inout"):
                out.append(a["buf"])
        return out

    def run(self, rt, program: str, vars: dict[str, int], tag: str) -> int:
        doc = rt.doc
        calls = doc["programs"][program]["calls"]
        proto = rt.protocol or {}
        rows = vars.get((proto.get("rows") or {}).get("var"), 0)
        lo, n = 0, 0
        for i, c in enumerate(calls):
            label = c.get("label") or ""
            if not label or not self.wants(label):
                continue
            n += rt.issue_range(program, vars, lo, i + 1)
            lo = i + 1
            if hasattr(rt, "synchronize"):
                rt.synchronize()
            for name in self._written(doc, c):
                t = rt.tensor(name)
                shape = doc["buffers"][name]["shape"]
                if rows and len(shape) >= 1 and not isinstance(shape[0], int):
                    t = t.view(-1)[: rows * (t.numel() // max(1, t.shape[0]))].view(rows, -1) if t.dim() >= 1 and t.shape[0] >= rows else t
                cpu = t.detach().to("cpu").clone()
                f = f"{tag}.{label}.{name}.pt"
                torch.save(cpu, self.dir / f)
                self.index.append({"file": f, "program": program, "call": i, "label": label, "buffer": name,
                                   "dtype": str(cpu.dtype).replace("torch.", ""), "shape": list(cpu.shape)})
        if lo < len(calls):
            n += rt.issue_range(program, vars, lo, len(calls))
        (self.dir / "index.json").write_text(json.dumps(self.index, indent=1))
        return n
