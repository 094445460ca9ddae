"""A pipeline's timeline from its stages' `pp item` log lines (`serve/pp_ranks.py`, log level debug).

Every stage logs when it issued each item and when the item left its device (`issued_us`, `done_us`, the stage
process's own clock); the item number is the same on every stage. A stage can start item k once it has issued it, is
done with k - 1 and its upstream is done with k, so per stage and item:

    wait = start - done[k - 1]     idle: nothing issued yet, or the upstream had not delivered
    held = done - start            its own work, plus any wait for the downstream to take the item

and done to done is the stage's period. Stages on different machines have different clocks: `--skew S=us` shifts stage S
and every later one.

    python -m kern_b200.serve.pp_timeline stage*.log [--skew 4=-1200] [--from K] [--to K] [--gantt]

Prints one line per stage (items, median period, median held, median wait, busy share) and, with `--gantt`, a row of
characters per stage over the common time axis (`#` held, `.` waiting). Reference counterpart: tools/pp_timeline.py.
"""
from __future__ import annotations

import argparse
import re
import statistics
from collections import defaultdict

LINE = re.compile(r"pp item stage=(\d+) item=(\d+) rows=(\d+) issued_us=(\d+) done_us=(\d+)")


def parse(texts) -> tuple[dict, dict, dict]:
    """-> (issued[stage][item], done[stage][item], rows[item]) from any iterable of log texts."""
    issued, done, rows = defaultdict(dict), defaultdict(dict), {}
    for text in texts:
        for m in LINE.finditer(text):
            s, k, r, i, t = map(int, m.groups())
            issued[s][k], done[s][k], rows[k] = i, t, r
    return issued, done, rows


def timeline(issued: dict, done: dict, skew: dict[int, int] | None = None, first: int | None = None, last: int | None = None) -> dict:
    """Per stage: the items every stage has, each with (start, done, wait, held); `skew[s]` microseconds are added to
    stage s and every later one."""
    skew = skew or {}
    stages = sorted(done)
    if not stages:
        return {}
    shift = {s: sum(v for at, v in skew.items() if at <= s) for s in stages}
    items = sorted(set.intersection(*(set(done[s]) for s in stages)))
    items = [k for k in items if (first is None or k >= first) and (last is None or k <= last)]
    out = {}
    for si, s in enumerate(stages):
        rows = []
        for n, k in enumerate(items):
            d = done[s][k] + shift[s]
            start = issued[s][k] + shift[s]
            if n > 0:
                start = max(start, done[s][items[n - 1]] + shift[s])
            if si > 0:
                up = stages[si - 1]
                start = max(start, done[up][k] + shift[up])
            start = min(start, d)
            prev = done[s][items[n - 1]] + shift[s] if n > 0 else start
            rows.append({"item": k, "start": start, "done": d, "wait": max(0, start - prev), "held": d - start})
        out[s] = rows
    return out


def summary(tl: dict) -> list[dict]:
    out = []
    for s, rows in sorted(tl.items()):
        if not rows:
            continue
        periods = [b["done"] - a["done"] for a, b in zip(rows, rows[1:])]
        span = rows[-1]["done"] - rows[0]["start"]
        out.append({"stage": s, "items": len(rows), "period_us_p50": statistics.median(periods) if periods else 0,
                    "held_us_p50": statistics.median(r["held"] for r in rows), "wait_us_p50": statistics.median(r["wait"] for r in rows),
                    "busy": round(sum(r["held"] for r in rows) / span, 3) if span > 0 else 1.0})
    return out


def gantt(tl: dict, width: int = 100) -> list[str]:
    """One row of `width` characters per stage over the common axis: `#` while an item is held, `.` otherwise."""
    rows = [r for v in tl.values() for r in v]
    if not rows:
        return []
    t0, t1 = min(r["start"] for r in rows), max(r["done"] for r in rows)
    scale = max(1, t1 - t0) / width
    lines = []
    for s, items in sorted(tl.items()):
        cells = ["."] * width
        for r in items:
            a, b = int((r["start"] - t0) / scale), int((r["done"] - t0) / scale)
            for c in range(max(0, a), min(width, max(a + 1, b))):
                cells[c] = "#"
        lines.append(f"stage {s:2d} |{''.join(cells)}|")
    lines.append(f"          {t0} us .. {t1} us ({(t1 - t0) / 1e3:.1f} ms)")
    return lines


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("logs", nargs="+")
    ap.add_argument("--skew", action="append", default=[], help="S=us: shift stage S and every later one")
    ap.add_argument("--from", dest="first", type=int)
    ap.add_argument("--to", dest="last", type=int)
    ap.add_argument("--gantt", action="store_true")
    a = ap.parse_args(argv)
    skew = {int(k): int(v) for k, v in (x.split("=") for x in a.skew)}
    issued, done, _rows = parse(open(p, errors="replace").read() for p in a.logs)
    tl = timeline(issued, done, skew, a.first, a.last)
    if not tl:
        print("no `pp item` lines (the stages log them at level debug)")
        return 1
    for r in summary(tl):
        print(f"stage {r['stage']}: {r['items']} items, period {r['period_us_p50']:.0f} us, held {r['held_us_p50']:.0f} us, "
              f"wait {r['wait_us_p50']:.0f} us, busy {r['busy']:.2f}")
    if a.gantt:
        print("\n".join(gantt(tl)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
