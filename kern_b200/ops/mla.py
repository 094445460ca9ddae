"""Multi-head latent attention, absorbed decode form: every head attends over one shared paged latent cache whose rows
(576 = 512 compressed + 64 rotary) are keys, and whose first 512 columns are values.

Reference: the reference runs a CuTe-DSL MLA decode kernel for this step (docs/roadmap.md:35); no source there.
"""
from __future__ import annotations

import torch

from .attention import merge_partials
from .launcher import Kernels, f32, i32, ptr

DQK, DV, HEADS_PER_CTA = 576, 512, 16
MATH_WARPS, TILE, STAGES = 8, 64, 2
SMEM = 1024 + STAGES * TILE * DQK * 2 + 16 * (DQK + 8) * 2 + 16 * (TILE + 8) * 2 + 2 * MATH_WARPS * 16 * 4 + 128


def mla_decode(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, seq_lens: torch.Tensor, heads: int,
               scale: float | None = None, splits: int | None = None, out: torch.Tensor | None = None,
               row_seq: torch.Tensor | None = None) -> torch.Tensor:
    """q [seqs, heads * 576] bf16; cache [pages, page_size, 576] bf16; block_table [seqs, max_pages] i32; seq_lens [seqs]
    i32 -> out [seqs, heads * 512] bf16. With `row_seq` [rows] i32 a row of q is not a sequence of its own: it reads
    block-table row row_seq[r] and attends over seq_lens[r] positions (prefill rows: their position + 1). `scale` defaults to 1 / sqrt(192) (the un-absorbed head width: 128 + 64)."""
    k = Kernels.get(q.device)
    seqs = q.shape[0]
    pages, page_size, w = cache.shape
    assert w == DQK and cache.dtype == torch.bfloat16 and q.dtype == torch.bfloat16 and q.shape[1] == heads * DQK
    BOX = 16 if TILE % 32 else None      # rows of a TMA box: never across a page
    assert page_size % (BOX or 1) == 0 and (BOX or page_size % TILE == 0 or TILE % page_size == 0)
    if out is None:
        out = torch.empty(seqs, heads * DV, dtype=torch.bfloat16, device=q.device)
    blocks = -(-heads // HEADS_PER_CTA)
    if splits is None:      # enough CTAs for the machine, never more than one per 64-token tile
        longest = block_table.shape[1] * page_size      # the table's reach: no device read on the launch path
        splits = max(1, min(128, -(-longest // 256), k.sm_count // max(1, seqs * blocks)))      # never more CTAs than SMs
    scale = (192 ** -0.5) if scale is None else scale
    lat = k.tensor_map_2d(cache.view(pages * page_size, DQK), BOX or min(page_size, TILE), 64)
    ws_o = ws_ml = None
    if splits > 1:
        ws_o = torch.empty(seqs * heads * splits * DV, dtype=torch.float32, device=q.device)
        ws_ml = torch.empty(seqs * heads * splits * 2, dtype=torch.float32, device=q.device)
    k.launch("mla_decode", "kern_mla_decode_bf16", (blocks, seqs, splits), (MATH_WARPS * 32 + 32,),
             [lat, ptr(q), ptr(out), ptr(ws_o), ptr(ws_ml), ptr(block_table), ptr(seq_lens), i32(seqs), i32(heads), i32(q.stride(0)),
              i32(out.stride(0)), i32(block_table.shape[1]), i32(page_size), i32(splits), i32(pages), f32(scale * 1.4426950408889634),
              ptr(k.err_word()), ptr(row_seq)], shared_mem=SMEM)
    if splits > 1:
        merge_partials(ws_o, ws_ml, out, seqs, heads, DV, splits)
    return out


def mla_decode_ref(q: torch.Tensor, latent: torch.Tensor, heads: int, scale: float | None = None) -> torch.Tensor:
    """One sequence: q [heads, 576], latent [L, 576] (all positions) -> [heads, 512], fp32."""
    scale = (192 ** -0.5) if scale is None else scale
    s = (q.float() @ latent.float().t()) * scale
    return torch.softmax(s, -1) @ latent.float()[:, :DV]
