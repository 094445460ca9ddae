"""Block-draft helpers and the recurrent state's advance after a speculative round: wrappers and PyTorch statements.

Reference counterparts: tools/kernels-src/topk_row.cu:21, gdn_advance.cu:26/:36, dflash_conv.cu:19, dflash_select.cu:26.
"""
from __future__ import annotations

import torch

from .launcher import Kernels, i32, i64, ptr


def topk(logits: torch.Tensor, k: int = 16):
    """Top-k (k <= 16) per row of bf16 logits -> (ids i64 [rows, k], values f32 [rows, k]); ties to the smaller index."""
    assert logits.dtype == torch.bfloat16 and 1 <= k <= 16
    rows, n = logits.shape
    ids = torch.empty(rows, k, dtype=torch.int64, device=logits.device)
    vals = torch.empty(rows, k, dtype=torch.float32, device=logits.device)
    Kernels.get(logits.device).launch("draft", "kern_topk_bf16", (rows,), (256,),
                                      [ptr(logits), ptr(ids), ptr(vals), i32(n), i32(logits.stride(0)), i32(k)])
    return ids, vals


def topk_ref(logits: torch.Tensor, k: int = 16):
    x = logits.float()
    n = x.shape[1]
    # value descending, index ascending: sort on (-value, index)
    order = torch.argsort(-x.double() * (2 * n) + torch.arange(n, device=x.device).double() * 0, dim=1, stable=True)[:, :k]
    return order, torch.gather(x, 1, order)


def mask_row0(src: torch.Tensor, rows_per_seq: int) -> torch.Tensor:
    dst = torch.empty_like(src)
    rows, cols = src.shape
    Kernels.get(src.device).launch("draft", "kern_mask_row0_bf16", (rows,), (128,),
                                   [ptr(dst), ptr(src), i32(rows), i32(rows_per_seq), i32(cols)])
    return dst


def mask_row0_ref(src: torch.Tensor, rows_per_seq: int) -> torch.Tensor:
    out = src.clone()
    out[::rows_per_seq] = float("-inf")
    return out


def conv_shift(lines: torch.Tensor, state: torch.Tensor, accepted: torch.Tensor, line_bytes: int, tok_bytes: int) -> None:
    """lines [seqs, stride] i32; state u8 [lines, line_bytes]; tokens a..a+2 of line lines[s, a] -> 0..2, a = accepted[s] - 1."""
    seqs = lines.shape[0]
    Kernels.get(state.device).launch("draft", "kern_conv_shift", (seqs, (tok_bytes // 16 + 127) // 128), (128,),
                                     [ptr(lines), i32(lines.stride(0)), ptr(state), ptr(accepted), i32(seqs), i64(line_bytes),
                                      i64(tok_bytes)])


def conv_shift_ref(lines, state, accepted, line_bytes: int, tok_bytes: int) -> None:
    flat = state.view(-1)
    for s in range(lines.shape[0]):
        a = int(accepted[s]) - 1
        if a <= 0:
            continue
        ln = int(lines[s, a])
        if ln <= 0:
            continue
        base = ln * line_bytes
        src = flat[base + a * tok_bytes: base + (a + 3) * tok_bytes].clone()
        flat[base: base + 3 * tok_bytes] = src


def dflash_conv(x: torch.Tensor, delta: torch.Tensor, base: torch.Tensor, groups: int, side: int) -> torch.Tensor:
    """In place on x [T, dim] bf16; delta [T, >= 4 groups] bf16 viewed [T, 2 sides, 2 taps, groups]; base [2, 2, dim]."""
    T, dim = x.shape
    Kernels.get(x.device).launch("draft", "kern_dflash_conv_bf16", ((T + 7) // 8, (dim + 255) // 256), (256,),
                                 [ptr(x), ptr(delta), ptr(base), i32(T), i32(dim), i32(groups), i32(delta.stride(0)), i32(side)])
    return x


def dflash_conv_ref(x, delta, base, groups: int, side: int):
    T, dim = x.shape
    bf = lambda t: t.to(torch.bfloat16).float()
    d = delta.float()[:, side * 2 * groups:(side + 1) * 2 * groups].view(T, 2, groups).repeat_interleave(dim // groups, 2)
    b = base.float().view(2, 2, dim)[side]
    c0, c1 = bf(b[0] + d[:, 0]), bf(b[1] + d[:, 1])
    xf = x.float()
    prev = torch.cat([torch.zeros(1, dim, device=x.device), xf[:-1]])
    t1 = bf(c1 * prev)
    t1[torch.arange(T, device=x.device) % 8 == 0] = 0
    return bf(bf(c0 * xf) + t1).to(torch.bfloat16)


def dflash_select(cand, unary, hidden_r, succ, pred, pred_anchor, steps: int, rows_per_seq: int) -> torch.Tensor:
    """cand i64 [rows, 16], unary f32 [rows, 16], hidden_r bf16 [rows, >= rank], succ/pred bf16 [rows, 16, rank],
    pred_anchor bf16 [seqs, rank] -> chosen tokens i64 [seqs, steps]."""
    seqs, rank = pred_anchor.shape
    assert rank % 32 == 0 and rank <= 1024
    out = torch.empty(seqs, steps, dtype=torch.int64, device=cand.device)
    Kernels.get(cand.device).launch("draft", "kern_dflash_select", (seqs,), (rank,),
                                    [ptr(cand), ptr(unary), ptr(hidden_r), ptr(succ), ptr(pred), ptr(pred_anchor), ptr(out),
                                     i32(steps), i32(rank), i32(hidden_r.stride(0)), i32(rows_per_seq)])
    return out


def dflash_select_ref(cand, unary, hidden_r, succ, pred, pred_anchor, steps: int, rows_per_seq: int):
    seqs, rank = pred_anchor.shape
    bf = lambda t: t.to(torch.bfloat16).float()
    out = torch.empty(seqs, steps, dtype=torch.int64, device=cand.device)
    for s in range(seqs):
        prev = 0
        for l in range(steps):
            row = s * rows_per_seq + 1 + l
            pr = pred_anchor[s] if l == 0 else pred[row - 1, prev]
            ph = bf(pr.float() * hidden_r[row, :rank].float())
            score = unary[row] + bf((ph[None, :] * succ[row].float()).sum(-1))
            prev = int(score.argmax())
            out[s, l] = cand[row, prev]
    return out
