"""RoPE + paged KV append, and paged GQA attention (decode / speculative-verify rows / causal chunked
prefill), with PyTorch fp32 reference statements of the same ops.

KV cache of one layer: ``pool[pages, 2, kv_heads, page_size, head_dim]`` bf16 (k then v), slot =
page * page_size + offset. Reference counterparts: tools/kernels-src/attn_prep.cu:152 (prep); the
attention kernels are mined cubins in the reference (no source counterpart).
"""
from __future__ import annotations

import math

import torch

from .launcher import Kernels, f32, i32, i64, ptr

TK = 64


def rope_tables(max_pos: int, rot: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    """f32 ``cos, sin`` tables ``[max_pos, rot/2]`` computed on the device in double precision."""
    k = Kernels.get(device)
    cos = torch.empty(max_pos, rot // 2, dtype=torch.float32, device=device)
    sin = torch.empty_like(cos)
    import struct
    k.launch("attn_prep", "kern_rope_table_f32", (min(1024, (cos.numel() + 255) // 256),), (256,),
             [ptr(cos), ptr(sin), i32(max_pos), i32(rot), struct.pack("<d", float(theta))])
    return cos, sin


def rope_kv_append(qkv: torch.Tensor, pool: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                   cos: torch.Tensor, sin: torch.Tensor, hq: int, hk: int, d: int, rot: int | None = None,
                   q_norm: torch.Tensor | None = None, k_norm: torch.Tensor | None = None,
                   eps: float = 1e-6, norm_plus_one: bool = False, tokens: int | None = None) -> None:
    """Rotate q (in place in ``qkv``) and k, append k/v of every token to ``pool`` at its slot."""
    k = Kernels.get(qkv.device)
    t = qkv.shape[0] if tokens is None else tokens
    pages, two, hk_, page_size, d_ = pool.shape
    assert two == 2 and hk_ == hk and d_ == d and qkv.shape[1] >= (hq + 2 * hk) * d and d % 8 == 0 and qkv.stride(1) == 1
    assert positions.dtype == torch.int64 and slots.dtype == torch.int64
    rot = d if rot is None else rot
    assert cos.shape[1] == rot // 2
    k.launch("attn_prep", "kern_rope_kv_append_bf16", (t,), (128,),
             [ptr(qkv), ptr(pool), ptr(positions), ptr(slots), ptr(cos), ptr(sin), ptr(q_norm),
              ptr(k_norm), i32(t), i32(hq), i32(hk), i32(d), i32(rot), i32(page_size), f32(eps),
              i32(int(norm_plus_one)), i64(pages * page_size), i32(cos.shape[0]), i32(qkv.stride(0)), ptr(k.err_word())],
             shared_mem=4 * d * 4)


def _attn_smem(d: int, prefill: bool = False) -> int:
    stages = 2 if (prefill and d <= 128) else (3 if d >= 256 else 4)
    return 1024 + stages * (2 * TK * d * 2) + 64 * (d + 8) * 2 + 256


def pick_splits(ctas_without_split: int, max_len: int, sms: int, max_splits: int = 32) -> int:
    """Split the KV range only while it adds CTAs up to about one wave and leaves >= 4 tiles each."""
    if ctas_without_split >= sms:
        return 1
    tiles = max(1, (max_len + TK - 1) // TK)
    s = min(max_splits, max(1, sms // max(1, ctas_without_split)), max(1, tiles // 4))
    return max(1, s)


def paged_attention(q: torch.Tensor, pool: torch.Tensor, block_table: torch.Tensor,
                    seq_lens: torch.Tensor, hq: int, *, out: torch.Tensor | None = None,
                    prefill: bool = False, cu_q: torch.Tensor | None = None, rows_per_seq: int = 1,
                    max_rows: int | None = None, seqs: int | None = None, splits: int | None = None,
                    max_len: int | None = None, scale: float | None = None,
                    workspace: tuple[torch.Tensor, torch.Tensor] | None = None,
                    partial: tuple[int, int] | None = None) -> torch.Tensor:
    """Attention of this step's query rows over each sequence's paged context.

    ``partial=(base, total)`` (decode only): write un-normalised partials into slots ``base .. base+splits-1`` of a
    workspace with ``total`` slots per (row, head) and skip the merge — a context-parallel rank's share;
    ``merge_partials`` finishes once every share is in.

    ``q``: 2-D bf16 view whose row t holds the ``hq`` query heads of token t (a column slice of the
    fused qkv buffer works: the row stride is free). ``seq_lens[s]`` counts the context *including*
    this step's rows; rows of sequence s are ``cu_q[s]:cu_q[s+1]`` or ``s*rows_per_seq`` onward.
    ``prefill=True`` picks the row-parallel causal kernel, else the token-parallel decode kernel
    (with split-KV when few CTAs would run). Returns ``out[tokens, hq*d]``.
    """
    k = Kernels.get(q.device)
    pages, _, hk, page_size, d = pool.shape
    assert d in (64, 128, 256), "attention kernels are built for head_dim 64, 128, 256"
    assert page_size >= 8 and (page_size <= TK and TK % page_size == 0 or page_size % TK == 0)
    g = hq // hk
    assert hq % hk == 0 and g <= 16
    n_seqs = block_table.shape[0] if seqs is None else seqs
    if out is None:
        out = torch.empty(q.shape[0], hq * d, dtype=torch.bfloat16, device=q.device)
    if max_rows is None:
        max_rows = rows_per_seq if cu_q is None else q.shape[0]
    toks_per_blk = (64 // g) if prefill else max(1, 16 // g)
    nblk = (max_rows + toks_per_blk - 1) // toks_per_blk
    if max_len is None:
        max_len = block_table.shape[1] * page_size
    if prefill:
        splits = 1
    elif splits is None:
        splits = pick_splits(hk * nblk * n_seqs, max_len, k.sm_count)
    ws_o = ws_ml = None
    total = splits if partial is None else partial[1]
    if partial is not None:
        assert not prefill and workspace is not None and partial[0] + splits <= total < 65536 and partial[0] < 256
    if total > 1:
        if workspace is not None:
            ws_o, ws_ml = workspace
        else:
            ws_o = torch.empty(q.shape[0] * hq * total * d, dtype=torch.float32, device=q.device)
            ws_ml = torch.empty(q.shape[0] * hq * total * 2, dtype=torch.float32, device=q.device)
        assert ws_o.numel() >= q.shape[0] * hq * total * d
    view = pool.view(pages * 2 * hk * page_size, d)
    kv_map = k.tensor_map_2d(view, min(page_size, TK), 64)
    scale = (1.0 / math.sqrt(d)) if scale is None else scale
    entry = f"kern_attn_{'prefill' if prefill else 'decode'}_paged_d{d}"
    grid = (hk * nblk, n_seqs, splits)
    work = count = None
    if prefill and cu_q is not None:
        items = (q.shape[0] + toks_per_blk - 1) // toks_per_blk + n_seqs
        work = torch.empty(2 * items, dtype=torch.int32, device=q.device)
        count = torch.zeros(2, dtype=torch.int32, device=q.device)
        k.launch("attn_paged", "kern_attn_plan", (1,), (256,),
                 [ptr(cu_q), i32(n_seqs), i32(toks_per_blk), i32(max(1, 16 // g)), i32(0), ptr(work), ptr(count),
                  i32(items), ptr(work), ptr(count[1:]), i32(0)])
        grid = (hk, items, 1)
    k.launch("attn_paged", entry, grid, (160,),
             [kv_map, ptr(q), ptr(out), ptr(ws_o), ptr(ws_ml), ptr(block_table), ptr(seq_lens),
              ptr(cu_q), ptr(work), ptr(count), i32(n_seqs), i32(hq), i32(hk), i32(q.stride(0)), i32(out.stride(0)),
              i32(block_table.shape[1]), i32(page_size), i32(rows_per_seq),
              i32(splits if partial is None else splits | (partial[0] << 8) | (total << 16)), i32(pages),
              f32(scale * 1.4426950408889634), ptr(k.err_word())],
             shared_mem=_attn_smem(d, prefill))
    if splits > 1 and partial is None:
        merge_partials(ws_o, ws_ml, out, q.shape[0], hq, d, splits)
    return out


def fmha_smem(d: int, tile: int) -> int:
    """Dynamic shared memory of the tcgen05 prefill kernel: Q and P tiles, a two-stage K/V ring, barriers, alignment room."""
    return (768 if tile == 64 else 1024) + 128 * d * 2 + 128 * tile * 2 + 2 * 2 * (tile * d * 2) + 256


def ragged_attention(q: torch.Tensor, pool: torch.Tensor, block_table: torch.Tensor, seq_lens: torch.Tensor, hq: int,
                     cu_q: torch.Tensor, *, out: torch.Tensor | None = None, seqs: int | None = None,
                     scale: float | None = None, one_launch: bool = True, fmha: bool = False) -> torch.Tensor:
    """A ragged call (prompt chunks and decode rows together) as a model's `attn_prefill` op runs it: the planner
    splits the sequences by their row count into the row-parallel causal kernel's list and the token-parallel kernel's
    list, and either one launch runs both kernels' CTAs side by side (`kern_attn_ragged_paged_d*`, head_dim 64 / 128)
    or two launches run one after the other. `fmha` (head_dim 128, one launch): the prompt rows' CTAs are the tcgen05
    kernel's (`kern_attn_ragged_fmha_d128`, blocks of 128 rows)."""
    k = Kernels.get(q.device)
    pages, _, hk, page_size, d = pool.shape
    g = hq // hk
    assert d in (64, 128) or not one_launch
    n_seqs = block_table.shape[0] if seqs is None else seqs
    if out is None:
        out = torch.empty(q.shape[0], hq * d, dtype=torch.bfloat16, device=q.device)
    assert not fmha or (one_launch and d == 128 and 128 % g == 0)
    tpb, tpd = (128 if fmha else 64) // g, max(1, 16 // g)
    items = (q.shape[0] + tpb - 1) // tpb + n_seqs
    work_p = torch.empty(2 * items, dtype=torch.int32, device=q.device)
    work_d = torch.empty(2 * items, dtype=torch.int32, device=q.device)
    count = torch.zeros(2, dtype=torch.int32, device=q.device)
    k.launch("attn_paged", "kern_attn_plan", (1,), (256,),
             [ptr(cu_q), i32(n_seqs), i32(tpb), i32(tpd), i32(tpd), ptr(work_p), ptr(count), i32(items), ptr(work_d),
              ptr(count[1:]), i32(items)])
    view = pool.view(pages * 2 * hk * page_size, d)
    kv_map = k.tensor_map_2d(view, min(page_size, TK), 64)
    scale = (1.0 / math.sqrt(d)) if scale is None else scale
    common = [i32(hq), i32(hk), i32(q.stride(0)), i32(out.stride(0)), i32(block_table.shape[1]), i32(page_size)]
    if one_launch:
        k.launch("attn_fmha" if fmha else "attn_paged", "kern_attn_ragged_fmha_d128" if fmha else f"kern_attn_ragged_paged_d{d}",
                 (hk, items, 1), (192 if fmha else 160,),
                 [kv_map, ptr(q), ptr(out), ptr(block_table), ptr(seq_lens), ptr(cu_q), ptr(work_p), ptr(count), ptr(work_d),
                  ptr(count[1:])] + common + [i32(pages), f32(scale * 1.4426950408889634), ptr(k.err_word())],
                 shared_mem=fmha_smem(d, 64) if fmha else _attn_smem(d, True))
        return out
    for prefill, work, cnt, gy in ((True, work_p, count, items), (False, work_d, count[1:], n_seqs)):
        k.launch("attn_paged", f"kern_attn_{'prefill' if prefill else 'decode'}_paged_d{d}", (hk, gy, 1), (160,),
                 [kv_map, ptr(q), ptr(out), ptr(None), ptr(None), ptr(block_table), ptr(seq_lens), ptr(cu_q), ptr(work), ptr(cnt),
                  i32(n_seqs)] + common + [i32(1), i32(1), i32(pages), f32(scale * 1.4426950408889634), ptr(k.err_word())],
                 shared_mem=_attn_smem(d, prefill))
    return out


def fmha_prefill(q: torch.Tensor, pool: torch.Tensor, block_table: torch.Tensor, seq_lens: torch.Tensor, hq: int,
                 cu_q: torch.Tensor, *, out: torch.Tensor | None = None, seqs: int | None = None,
                 scale: float | None = None, tile: int = 64) -> torch.Tensor:
    """`tile`: tokens per KV tile, 128 (one CTA per SM) or 64 (two CTAs per SM: one's MMAs under the other's softmax).
    Causal prefill attention of a ragged call on the tcgen05 kernel (csrc/kernels/sm100/attn_fmha.cu): head_dim 128,
    128 query rows per CTA (128 / group tokens x the group's heads), S and O in TMEM. Same operands as
    ``paged_attention(..., prefill=True, cu_q=...)``."""
    k = Kernels.get(q.device)
    pages, _, hk, page_size, d = pool.shape
    assert d == 128, "the tcgen05 prefill kernel is built for head_dim 128"
    assert page_size >= 8 and (page_size <= 64 and 64 % page_size == 0 or page_size % 64 == 0)
    g = hq // hk
    assert hq % hk == 0 and 128 % g == 0
    n_seqs = block_table.shape[0] if seqs is None else seqs
    if out is None:
        out = torch.empty(q.shape[0], hq * d, dtype=torch.bfloat16, device=q.device)
    tpb = 128 // g
    items = (q.shape[0] + tpb - 1) // tpb + n_seqs
    work = torch.empty(2 * items, dtype=torch.int32, device=q.device)
    count = torch.zeros(2, dtype=torch.int32, device=q.device)
    k.launch("attn_paged", "kern_attn_plan", (1,), (256,),
             [ptr(cu_q), i32(n_seqs), i32(tpb), i32(1), i32(0), ptr(work), ptr(count), i32(items), ptr(work), ptr(count[1:]), i32(0)])
    view = pool.view(pages * 2 * hk * page_size, d)
    kv_map = k.tensor_map_2d(view, min(page_size, 64), 64)
    scale = (1.0 / math.sqrt(d)) if scale is None else scale
    assert tile in (64, 128)
    smem = fmha_smem(d, tile)
    k.launch("attn_fmha", "kern_attn_fmha_prefill_d128" + ("_t64" if tile == 64 else ""), (hk, items, 1), (192,),
             [kv_map, ptr(q), ptr(out), ptr(block_table), ptr(seq_lens), ptr(cu_q), ptr(work), ptr(count), i32(hq), i32(hk),
              i32(q.stride(0)), i32(out.stride(0)), i32(block_table.shape[1]), i32(page_size), i32(pages),
              f32(scale * 1.4426950408889634), ptr(k.err_word())], shared_mem=smem)
    return out


def fmha_context(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_q: torch.Tensor, cu_k: torch.Tensor, heads: int, *,
                 out: torch.Tensor | None = None, scale: float | None = None, two_per_sm: bool = True) -> torch.Tensor:
    """Causal context attention over contiguous ragged K / V with a 192-wide q.k and 128-wide values: the prefill of a
    latent-attention layer in its un-absorbed form (csrc/kernels/sm100/attn_fmha.cu, `kern_attn_fmha_ctx_qk192_v128`).
    `q` [q tokens, heads * 192], `k` [kv tokens, heads * 192], `v` [kv tokens, heads * 128], bf16, rows of a sequence
    contiguous (`cu_q`, `cu_k` cumulative counts, int32); query i of a sequence with R rows and L keys sees keys
    0 .. L - R + i. Returns [q tokens, heads * 128]. `two_per_sm`: the one-stage form, two CTAs per SM."""
    kk = Kernels.get(q.device)
    dqk, dv, fn = 192, 128, 64
    assert q.shape[1] == heads * dqk and k.shape[1] == heads * dqk and v.shape[1] == heads * dv
    assert k.is_contiguous() and v.is_contiguous() and q.stride(1) == 1
    n_seqs = cu_q.numel() - 1
    if out is None:
        out = torch.empty(q.shape[0], heads * dv, dtype=torch.bfloat16, device=q.device)
    items = (q.shape[0] + 127) // 128 + n_seqs
    work = torch.empty(2 * items, dtype=torch.int32, device=q.device)
    count = torch.zeros(2, dtype=torch.int32, device=q.device)
    kk.launch("attn_paged", "kern_attn_plan", (1,), (256,),
              [ptr(cu_q), i32(n_seqs), i32(128), i32(1), i32(0), ptr(work), ptr(count), i32(items), ptr(work), ptr(count[1:]), i32(0)])
    k_map = kk.tensor_map_2d(k, fn, 64)
    v_map = kk.tensor_map_2d(v, fn, 64)
    scale = (1.0 / math.sqrt(dqk)) if scale is None else scale
    stages = 1 if two_per_sm else 2
    smem = (768 if two_per_sm else 1024) + 128 * dqk * 2 + 128 * fn * 2 + stages * (fn * dqk * 2 + fn * dv * 2) + 256
    kk.launch("attn_fmha", "kern_attn_fmha_ctx_qk192_v128" + ("_x2" if two_per_sm else ""), (heads, items, 1), (192,),
              [k_map, v_map, ptr(q), ptr(out), ptr(cu_q), ptr(cu_k), ptr(work), ptr(count), i32(q.stride(0)), i32(out.stride(0)),
               f32(scale * 1.4426950408889634), ptr(kk.err_word())], shared_mem=smem)
    return out


def context_reference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_q, cu_k, heads: int, scale: float | None = None) -> torch.Tensor:
    """fp32 statement of `fmha_context`."""
    dqk, dv = q.shape[1] // heads, v.shape[1] // heads
    scale = (1.0 / math.sqrt(dqk)) if scale is None else scale
    out = torch.zeros(q.shape[0], heads * dv, dtype=torch.float32, device=q.device)
    for s in range(len(cu_q) - 1):
        q0, q1, k0, k1 = int(cu_q[s]), int(cu_q[s + 1]), int(cu_k[s]), int(cu_k[s + 1])
        R, L = q1 - q0, k1 - k0
        if R <= 0 or L <= 0:
            continue
        qq = q[q0:q1].float().view(R, heads, dqk)
        kk = k[k0:k1].float().view(L, heads, dqk)
        vv = v[k0:k1].float().view(L, heads, dv)
        sc = torch.einsum("rhd,lhd->hrl", qq, kk) * scale
        limit = torch.arange(L - R, L, device=q.device)
        mask = torch.arange(L, device=q.device)[None, :] <= limit[:, None]
        sc = sc.masked_fill(~mask[None], float("-inf"))
        pr = torch.softmax(sc, -1).nan_to_num(0.0)
        out[q0:q1] = torch.einsum("hrl,lhd->rhd", pr, vv).reshape(R, heads * dv)
    return out


def new_partials(rows: int, hq: int, d: int, total: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    """A workspace of `total` partial slots per (row, head), every slot neutral (m = -inf, l = 0): a rank whose share
    of a sequence is empty leaves its slots as they are."""
    ws_o = torch.zeros(rows * hq * total * d, dtype=torch.float32, device=device)
    ws_ml = torch.zeros(rows * hq * total, 2, dtype=torch.float32, device=device)
    ws_ml[:, 0] = float("-inf")
    return ws_o, ws_ml.view(-1)


def merge_partials(ws_o, ws_ml, out, rows: int, hq: int, d: int, total: int) -> torch.Tensor:
    k = Kernels.get(out.device)
    n = rows * hq
    k.launch("attn_paged", "kern_attn_merge_splits", (n,), (min(256, d),),
             [ptr(ws_o), ptr(ws_ml), ptr(out), i32(n), i32(hq), i32(d), i32(total), i32(out.stride(0))])
    return out


def merge_rank_partials(ws_o, ws_ml, out, rows: int, hq: int, d: int, splits: int, ranks: int) -> torch.Tensor:
    """Merge the all-gathered compact workspaces of a context-parallel group: `ws_o` is [ranks][rows * hq][splits][d],
    `ws_ml` [ranks][rows * hq][splits][2], each rank's part written by a decode launch with ``partial=(0, splits)``."""
    k = Kernels.get(out.device)
    n = rows * hq
    k.launch("attn_paged", "kern_attn_merge_ranks", (n,), (min(256, d),),
             [ptr(ws_o), ptr(ws_ml), ptr(out), i32(n), i32(hq), i32(d), i32(splits), i32(ranks), i32(out.stride(0))])
    return out


def dcp_local_lens(seq_lens: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Positions of each sequence that live on member `rank` of a by-position group of `world`."""
    out = torch.empty_like(seq_lens)
    n = seq_lens.numel()
    Kernels.get(seq_lens.device).launch("attn_paged", "kern_dcp_local_lens", ((n + 255) // 256,), (256,),
                                        [ptr(seq_lens), ptr(out), i32(n), i32(rank), i32(world)])
    return out


def deal_rows(src_kv: torch.Tensor, dst_kv: torch.Tensor, src_table: torch.Tensor, dst_table: torch.Tensor,
              src_lens: torch.Tensor, hk: int, d: int, page_size: int, rank: int, world: int, first_pos: int = 0) -> None:
    """Copy the KV rows of positions p = li * world + rank (p >= first_pos) of every sequence from a pool holding the
    whole context into member `rank`'s pool at local index li. Pools: [page][k|v][kv_head][page_size][d] bf16 (any
    dtype view of the same bytes); `dst_kv` may be another GPU's mapped memory."""
    k = Kernels.get(src_kv.device)
    seqs = src_lens.numel()
    max_local = (int(src_lens.max()) + world - 1) // world
    if max_local <= 0:
        return
    k.launch("attn_paged", "kern_deal_rows_bf16", ((max_local + 3) // 4, seqs), (128,),
             [ptr(src_kv), ptr(dst_kv), ptr(src_table), ptr(dst_table), ptr(src_lens), i32(seqs), i32(src_table.shape[1]),
              i32(dst_table.shape[1]), i32(hk), i32(d), i32(page_size), i32(rank), i32(world), i32(first_pos),
              ptr(k.err_word())])


# ---- PyTorch fp32 references ---------------------------------------------------------------------
def rope_reference(x: torch.Tensor, positions: torch.Tensor, rot: int, theta: float) -> torch.Tensor:
    """x [tokens, heads, d] -> rotate-half RoPE over the first ``rot`` dims, fp32 math."""
    half = rot // 2
    inv = theta ** (-torch.arange(0, half, dtype=torch.float64, device=x.device) * 2.0 / rot)
    ang = positions.double()[:, None] * inv[None, :]
    cos, sin = ang.cos().float()[:, None, :], ang.sin().float()[:, None, :]
    xf = x.float()
    a, b = xf[..., :half], xf[..., half:rot]
    out = xf.clone()
    out[..., :half] = a * cos - b * sin
    out[..., half:rot] = b * cos + a * sin
    return out


def attention_reference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_pos: torch.Tensor,
                        scale: float | None = None) -> torch.Tensor:
    """One sequence: q [R, hq, d], k/v [L, hk, d] (already rotated), q_pos [R] absolute positions.
    Row r attends to keys 0..q_pos[r]. fp32 math; returns [R, hq*d] fp32."""
    r, hq, d = q.shape
    l, hk, _ = k.shape
    g = hq // hk
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    kk = k.float().repeat_interleave(g, dim=1)
    vv = v.float().repeat_interleave(g, dim=1)
    s = torch.einsum("rhd,lhd->hrl", q.float(), kk) * scale
    mask = torch.arange(l, device=q.device)[None, :] <= q_pos[:, None]
    s = s.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(s, -1)
    o = torch.einsum("hrl,lhd->rhd", p, vv)
    return o.reshape(r, hq * d)
