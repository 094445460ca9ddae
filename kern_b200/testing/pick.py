"""Choosing implementations by range: given each candidate's time at sampled values of a var (rows of a call), the
fewest `when` ranges such that inside every range one candidate is within the noise of the best at each sampled point.
Greedy is optimal here (a range is extended while some candidate still covers all of it; ranges are intervals).
Reference counterpart: crates/kern-run/src/bench/pick.rs:63-114.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class Point:
    value: int                   # the var's value at this sample
    times: dict[str, float]      # candidate -> milliseconds
    noise: float = 0.0           # spread below which two times are the same


def pick(points: list[Point]) -> list[tuple[str, int, int]]:
    """-> [(candidate, min value, max value)] covering the sampled values in order; between samples the boundary sits
    right after the last sample of the earlier range."""
    pts = sorted(points, key=lambda p: p.value)
    out: list[tuple[str, int, int]] = []
    i = 0
    while i < len(pts):
        ok = None                   # candidates within noise of the best at every point of the range so far
        j = i
        while j < len(pts):
            best = min(pts[j].times.values())
            good = {c for c, t in pts[j].times.items() if t <= best + pts[j].noise}
            nxt = good if ok is None else ok & good
            if not nxt:
                break
            ok = nxt
            j += 1
        # among those still standing, the one with the least total time over the range
        name = min(sorted(ok), key=lambda c: sum(p.times[c] for p in pts[i:j]))
        out.append((name, pts[i].value, pts[j - 1].value))
        i = j
    # make the ranges contiguous: a range starts right after the previous one's last sample
    return [(n, (1 if k == 0 else out[k - 1][2] + 1), hi) for k, (n, lo, hi) in enumerate(out)]


def gaps(ranges: list[tuple[str, int, int]], var_max: int) -> list[tuple[int, int]]:
    """Values of the var that no range covers."""
    out, at = [], 1
    for _, lo, hi in ranges:
        if lo > at:
            out.append((at, lo - 1))
        at = hi + 1
    if at <= var_max:
        out.append((at, var_max))
    return out
