"""e2e-logits: record what an engine answers to a fixed set of questions (tokens, the top of every step's
distribution, the engine's own run-to-run noise) and judge a second engine — another manifest, another runtime,
another host framework — against the recording, teacher-forced along the recorded tokens.

Recording = one Parquet file: source, question, prompt, output, top_ids, top_logprobs, noise.
Judgment per question: token agreement along the forced path, the largest and mean KL(recorded || candidate)
over the recorded top entries, against a limit scaled by the recording's own noise.
Reference counterpart: crates/kern-test/src/e2e.rs:56-200 (Question, Recording, Plan, kl, Judgment).
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path

import numpy as np

TOP = 20


@dataclass
class Question:
    id: str
    prompt: list[int]
    max_tokens: int = 16


def plan(seed: int, count: int, vocab: int, lengths=(8, 64), max_tokens: int = 16) -> list[Question]:
    """A seeded set of questions over the token domain (prompts of mixed length)."""
    from .abtest import Rng

    rng = Rng(seed)
    out = []
    for i in range(count):
        n = lengths[0] + rng.below(max(1, lengths[1] - lengths[0] + 1))
        out.append(Question(id=f"q{i}", prompt=[1 + rng.below(max(1, vocab - 1)) for _ in range(n)], max_tokens=max_tokens))
    return out


def top_of(row: np.ndarray, top: int = TOP):
    """(ids, log-probabilities) of the `top` most likely tokens of a logits row; ties by lower id."""
    x = row.astype(np.float64)
    lse = x.max() + math.log(np.exp(x - x.max()).sum())
    order = np.lexsort((np.arange(len(x)), -x))[:top]
    return order.astype(np.int64).tolist(), (x[order] - lse).tolist()


def kl_top(ids: list[int], logp: list[float], row: np.ndarray) -> float:
    """KL(recorded || candidate) restricted to the recorded top entries, the rest lumped into one bucket."""
    x = row.astype(np.float64)
    lse = x.max() + math.log(np.exp(x - x.max()).sum())
    p = np.exp(np.asarray(logp))
    q = np.exp(x[np.asarray(ids)] - lse)
    kl = float((p * (np.log(p + 1e-300) - np.log(q + 1e-300))).sum())
    pr, qr = max(0.0, 1.0 - p.sum()), max(0.0, 1.0 - q.sum())
    if pr > 1e-12:
        kl += pr * (math.log(pr) - math.log(max(qr, 1e-300)))
    return max(0.0, kl)


@dataclass
class Recording:
    source: str
    rows: list[dict] = field(default_factory=list)      # question, prompt, output, top_ids, top_logprobs, noise
    noise_mean: float = 0.0                              # mean KL of the engine against itself over every replayed position

    def save(self, path: str | Path) -> None:
        import pyarrow as pa
        import pyarrow.parquet as pq

        t = pa.table({"source": [self.source] * len(self.rows), "question": [r["question"] for r in self.rows],
                      "prompt": [r["prompt"] for r in self.rows], "output": [r["output"] for r in self.rows],
                      "top_ids": [r["top_ids"] for r in self.rows], "top_logprobs": [r["top_logprobs"] for r in self.rows],
                      "noise": [r["noise"] for r in self.rows], "noise_mean": [float(self.noise_mean)] * len(self.rows)})
        pq.write_table(t, str(path), compression="zstd")

    @classmethod
    def load(cls, path: str | Path) -> "Recording":
        import pyarrow.parquet as pq

        d = pq.ParquetFile(str(path)).read().to_pydict()
        rows = [{k: d[k][i] for k in ("question", "prompt", "output", "top_ids", "top_logprobs", "noise")}
                for i in range(len(d["question"]))]
        return cls(source=d["source"][0] if d["source"] else "", rows=rows,
                   noise_mean=float(d["noise_mean"][0]) if d.get("noise_mean") else 0.0)


def record(side, questions: list[Question], source: str, chunk: int = 256, top: int = TOP, batch: int = 4) -> Recording:
    """`side`: an EngineSide (free_run / forced_run / batched_forced_run). The noise of a question is the largest KL
    between the recorded distribution and what the same engine gives along the same tokens again — alone, with the
    decode steps of `batch` questions run as one call, and in batches half that size: what the engine's own batch
    shapes move a distribution by (0 for an engine whose arithmetic does not depend on the batch)."""
    rec = Recording(source=source)
    for q in questions:
        outs, rows, _ = side.free_run([q.prompt], q.max_tokens, chunk)
        again = side.forced_run([q.prompt], outs, chunk)
        tops = [top_of(r, top) for r in rows]
        noise = max((kl_top(ids, lp, r2) for (ids, lp), r2 in zip(tops, again)), default=0.0)
        rec.rows.append({"question": q.id, "prompt": list(q.prompt), "output": [int(t) for t in outs[0]],
                         "top_ids": [t[0] for t in tops], "top_logprobs": [t[1] for t in tops], "noise": noise})
    every: list[float] = []
    if batch > 1 and len(rec.rows) > 1 and hasattr(side, "batched_forced_run"):
        prompts, outs = [r["prompt"] for r in rec.rows], [r["output"] for r in rec.rows]
        for b in sorted({batch, max(1, batch // 2)} - {1}, reverse=True):
            for r, rows in zip(rec.rows, side.batched_forced_run(prompts, outs, chunk, b)):
                kls = [kl_top(ids, lp, row) for ids, lp, row in zip(r["top_ids"], r["top_logprobs"], rows)]
                r["noise"] = max([r["noise"]] + kls)
                every += kls
    rec.noise_mean = float(np.mean(every)) if every else 0.0
    return rec


@dataclass
class Judgment:
    question: str
    agree: int              # forced positions where the candidate's arg-max is the recorded token
    positions: int
    max_kl: float
    mean_kl: float
    limit: float
    verdict: str            # PASS | FAIL
    kls: list = field(default_factory=list)          # per scored position, in order (decode step = index)
    prompt_len: int = 0

    def line(self) -> str:
        return (f"{self.verdict} {self.question}: argmax {self.agree}/{self.positions}, KL max {self.max_kl:.3e} "
                f"mean {self.mean_kl:.3e} (limit {self.limit:.3e})")


def judge(recording: Recording, side, kl_limit: float = 0.01, noise_factor: float = 4.0, chunk: int = 256) -> list[Judgment]:
    out = []
    for r in recording.rows:
        rows = side.forced_run([r["prompt"]], [r["output"]], chunk)
        kls = [kl_top(ids, lp, row) for ids, lp, row in zip(r["top_ids"], r["top_logprobs"], rows)]
        agree = sum(int(int(np.argmax(row)) == tok) for row, tok in zip(rows, r["output"]))
        limit = max(kl_limit, noise_factor * r["noise"])
        mx = max(kls, default=0.0)
        # an arg-max flip alone is not a failure (near-ties flip under any rounding); a flip with KL past the limit is
        ok = mx <= limit
        out.append(Judgment(r["question"], agree, len(rows), mx, float(np.mean(kls)) if kls else 0.0, limit, "PASS" if ok else "FAIL",
                            kls=[float(k) for k in kls], prompt_len=len(r["prompt"])))
    return out


def overall(judgments: list[Judgment], noise_mean: float, mean_floor: float = 1e-4) -> dict:
    """The statistical verdict over every scored position: the candidate's mean KL against the recording's own noise
    (what the baseline's batch shapes move its distributions by, never less than `mean_floor`) plus three standard errors
    of that mean. Also the mean by decode step and by context depth, the two ways an error grows.
    Reference: docs/test.md:112 (mean KL <= noise + 3 standard errors), :141 (by context depth and decode step)."""
    kls = np.array([k for j in judgments for k in j.kls], dtype=np.float64)
    n = int(kls.size)
    mean = float(kls.mean()) if n else 0.0
    se = float(kls.std(ddof=1) / np.sqrt(n)) if n > 1 else 0.0
    noise = max(float(noise_mean), mean_floor)
    ok = mean <= noise + 3.0 * se

    def buckets(key, edges):
        out = {}
        for j in judgments:
            for step, k in enumerate(j.kls):
                v = key(j, step)
                name = next((f"<{e}" for e in edges if v < e), f">={edges[-1]}")
                out.setdefault(name, []).append(k)
        return {name: float(np.mean(v)) for name, v in out.items()}

    return {"pass": bool(ok), "mean_kl": mean, "noise": noise, "se": se, "positions": n,
            "by_decode_step": buckets(lambda j, step: step, (1, 8, 64)),
            "by_context_depth": buckets(lambda j, step: j.prompt_len + step, (64, 1024, 16384)),
            "line": (f"{'PASS' if ok else 'FAIL'}      mean KL {mean:.2e} {'<=' if ok else '>'} noise {noise:.2e} + 3 x {se:.2e} "
                     f"({mean / noise:.2f} x the noise) over {n} scored positions")}


def summary(judgments: list[Judgment], noise_mean: float | None = None) -> tuple[str, int]:
    """One line per question, then (with the recording's `noise_mean`) the means by decode step and context depth and the
    verdict over all positions. Exit code 1 when a question is past its own limit or the overall rule fails."""
    bad = [j for j in judgments if j.verdict != "PASS"]
    text = "\n".join(j.line() for j in judgments)
    text += f"\n{'FAIL' if bad else 'PASS'}: {len(judgments) - len(bad)}/{len(judgments)} questions within the limit"
    code = 1 if bad else 0
    if noise_mean is not None:
        o = overall(judgments, noise_mean)
        fmt = lambda d: "  ".join(f"{k}: {v:.2e}" for k, v in d.items())
        text += f"\nmean KL by decode step    {fmt(o['by_decode_step'])}\nmean KL by context depth  {fmt(o['by_context_depth'])}\n{o['line']}"
        code = code or (0 if o["pass"] else 1)
    return text, code
