"""Speculative-round glue kernels (wrappers) and their host statements."""
from __future__ import annotations

import struct

import torch

from .launcher import Kernels, i32, i64, ptr


def splice(anchor, drafts, ids, block_rows, dstride=0, mask=0):
    k = Kernels.get(anchor.device)
    seqs = anchor.numel()
    k.launch("spec", "kern_spec_splice", (seqs,), (32,),
             [ptr(anchor), ptr(drafts), ptr(ids), i32(seqs), i32(block_rows), i32(dstride), i64(mask)])
    return ids


def rows(base_pos, block_table, block_rows, page_size):
    k = Kernels.get(base_pos.device)
    seqs, w = block_table.shape
    dev = base_pos.device
    pos = torch.empty(seqs * block_rows, dtype=torch.int64, device=dev)
    slots = torch.empty_like(pos)
    lens = torch.empty(seqs, dtype=torch.int32, device=dev)
    k.launch("spec", "kern_spec_rows", (seqs,), (32,),
             [ptr(base_pos), ptr(block_table), ptr(pos), ptr(slots), ptr(lens), i32(seqs), i32(block_rows), i32(w),
              i32(page_size), ptr(k.err_word())])
    return pos, slots, lens


def accept(drafts, verify, block_rows, dstride, line_in=None, seqs_max=0):
    k = Kernels.get(drafts.device)
    seqs = verify.numel() // block_rows
    dev = drafts.device
    count = torch.empty(seqs, dtype=torch.int32, device=dev)
    emitted = torch.empty(seqs, block_rows, dtype=torch.int64, device=dev)
    line_adv = torch.zeros_like(line_in) if line_in is not None else None
    line_rows = line_in.shape[0] if line_in is not None else 0
    k.launch("spec", "kern_spec_accept", (seqs,), (32,),
             [ptr(drafts), ptr(verify), ptr(count), ptr(emitted), ptr(line_in), ptr(line_adv), i32(seqs), i32(block_rows),
              i32(dstride), i32(line_rows), i32(seqs_max)])
    return count, emitted, line_adv


def accept_reference(drafts, verify, block_rows, dstride):
    seqs = verify.numel() // block_rows
    d, v = drafts.view(seqs, dstride).cpu(), verify.view(seqs, block_rows).cpu()
    counts, emitted = [], torch.zeros(seqs, block_rows, dtype=torch.int64)
    for i in range(seqs):
        a = 0
        while a < block_rows - 1 and int(d[i, a]) == int(v[i, a]):
            a += 1
        counts.append(a + 1)
        emitted[i, :a + 1] = v[i, :a + 1]
    return torch.tensor(counts, dtype=torch.int32), emitted
