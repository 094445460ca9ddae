"""PyTorch statement of the sampler's contract: temperature, then top-k, top-p over the survivors,
min-p; the draw is a pure function of (seed, offset) through splitmix64; temperature <= 0 is greedy
(ties to the lowest index)."""
from __future__ import annotations

import torch

_M = (1 << 64) - 1


def uniform01(seed: int, offset: int) -> float:
    z = (seed + 0x9E3779B97F4A7C15 * (offset + 1)) & _M
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M
    z ^= z >> 31
    return (z >> 40) / 16777216.0


def sample_rows(logits, temperature, top_k, top_p, min_p, seeds, offsets) -> torch.Tensor:
    out = torch.empty(logits.shape[0], dtype=torch.int64)
    for r in range(logits.shape[0]):
        row = torch.nan_to_num(logits[r].float(), nan=float("-inf"))
        t = float(temperature[r])
        if t <= 0:
            out[r] = int((row == row.max()).nonzero()[0, 0])
            continue
        p = torch.softmax(row / t, -1)
        keep = torch.ones_like(p, dtype=torch.bool)
        k = int(top_k[r])
        if 0 < k < p.numel():
            keep &= p >= torch.topk(p, k).values[-1]
        tp = float(top_p[r])
        if tp < 1.0:
            q = torch.where(keep, p, torch.zeros_like(p))
            sv, si = torch.sort(q, descending=True)
            n = int((torch.cumsum(sv, 0) < tp * q.sum()).sum()) + 1
            m = torch.zeros_like(keep)
            m[si[:n]] = True
            keep &= m
        mp = float(min_p[r])
        if mp > 0:
            keep &= p >= mp * p.max()
        q = torch.where(keep, p, torch.zeros_like(p))
        target = uniform01(int(seeds[r]) & _M, int(offsets[r])) * float(q.sum())
        idx = int((torch.cumsum(q, 0) > target).nonzero()[0, 0]) if float(q.sum()) > 0 else int(row.argmax())
        out[r] = idx
    return out
