"""A host-memory stand-in for the device: the same manifest executed by PyTorch on the CPU.

``CpuRuntime`` has the interface of :class:`kern_b200.runtime.Runtime` (protocol, write / read, issue,
pool support), allocates every buffer and state as host tensors, and runs each launch through a
Python function with the *same parameter list as the CUDA kernel* it stands in for. It exists so that
the control plane (engine, scheduler, ranks, pipeline, prefill/decode hand-off, fault paths) and whole
manifests run and are tested on machines with no GPU, and it is the executor of the CPU-only toy
decoder configuration. (The reference tests its harness the same way, with a host interpreter keyed by
entry name: crates/kern-test/tests/common/mod.rs:1-130.)
"""
from __future__ import annotations

import json
import math
import struct

import numpy as np
import torch

from . import _native
from .models.common import read_safetensors
from .runtime import _NP, _TORCH, manifest_text

_ES = {k: np.dtype(v).itemsize for k, v in _NP.items()}


def _eval(e, vars_):
    if isinstance(e, int):
        return e
    if isinstance(e, str):
        return vars_[e]
    (k, a), = e.items()
    if k == "ceil_div":
        return -(-_eval(a[0], vars_) // a[1])
    if k == "mul":
        return _eval(a[0], vars_) * a[1]
    if k == "add":
        return _eval(a[0], vars_) + _eval(a[1], vars_)
    if k == "clamp":
        return min(max(_eval(a[0], vars_) - a[1], 0), a[2])
    raise ValueError(f"unknown expression {e}")


# ---- CPU statements of the kernels (same parameter order as the CUDA entries) ------------------------
def _f(t):
    return t.float()


def k_embedding(g, ids, table, out, tokens, hidden, vocab, err):
    n = g[0]
    out.view(-1, hidden)[:n] = table.view(-1, hidden)[ids[:n].long().clamp(0, vocab - 1)]


def k_rms_norm(g, x, w, y, rows, n, xs, ys, eps, plus_one):
    r = g[0]
    xv = _f(torch.as_strided(x, (r, n), (xs, 1)))
    ww = _f(w[:n]) + (1.0 if plus_one else 0.0)
    torch.as_strided(y, (r, n), (ys, 1)).copy_((xv * torch.rsqrt(xv.pow(2).mean(-1, keepdim=True) + eps) * ww).to(y.dtype))


def k_fused_add_rms_norm(g, x, res, w, y, rows, n, eps, plus_one):
    r = g[0]
    s = (_f(x[: r * n]) + _f(res[: r * n])).to(res.dtype)
    res[: r * n] = s
    k_rms_norm(g, res, w, y, rows, n, n, n, eps, plus_one)


def _gemm(epi):
    def run(g, a, w, c, r, m, n, k, ldc, err):
        av = torch.as_strided(a, (m, k), (a_stride(a, k), 1))
        acc = _f(av) @ _f(w[: n * k].view(n, k)).t()
        if epi == "swiglu":
            acc = torch.nn.functional.silu(acc[:, : n // 2]) * acc[:, n // 2:]
        cv = torch.as_strided(c, (m, acc.shape[1]), (ldc, 1))
        if epi == "acc":
            acc = acc + _f(torch.as_strided(r, (m, n), (ldc, 1)))
        cv.copy_(acc.to(c.dtype))
    return run


def _gemv(epi):
    def run(g, a, w, c, r, m, n, k, lda, ldc, err):
        av = torch.as_strided(a, (m, k), (lda, 1), a.storage_offset())
        acc = _f(av) @ _f(w[: n * k].view(n, k)).t()
        if epi == "swiglu":
            acc = torch.nn.functional.silu(acc[:, : n // 2]) * acc[:, n // 2:]
        cv = torch.as_strided(c, (m, acc.shape[1]), (ldc, 1), c.storage_offset())
        if epi == "acc":
            acc = acc + _f(torch.as_strided(r, (m, n), (ldc, 1), r.storage_offset()))
        cv.copy_(acc.to(c.dtype))
    return run


def a_stride(a, k):
    return getattr(a, "_row_stride", k)


def k_rope_append(g, qkv, kv, positions, slots, cos, sin, qn, kn, tokens, hq, hk, d, rot, page, eps, plus_one, kv_slots, max_pos, row_stride, err):
    t = g[0]
    half = rot // 2
    rows = qkv[: t * row_stride].view(t, row_stride)[:, : (hq + 2 * hk) * d].unflatten(1, (hq + 2 * hk, d))
    pos = positions[:t].long().clamp(0, max_pos - 1)
    c, s = cos.view(-1, half)[pos][:, None], sin.view(-1, half)[pos][:, None]
    pool = kv.view(torch.bfloat16).view(-1, 2, hk, page, d)

    def prep(x, w):
        xf = _f(x)
        if isinstance(w, torch.Tensor):
            ww = _f(w[:d]) + (1.0 if plus_one else 0.0)
            xf = _f((xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * ww).to(torch.bfloat16))
        a, b = xf[..., :half], xf[..., half:rot]
        return torch.cat([a * c - b * s, b * c + a * s, xf[..., rot:]], -1).to(torch.bfloat16)

    q = prep(rows[:, :hq], qn)
    k = prep(rows[:, hq:hq + hk], kn)
    v = rows[:, hq + hk:].clone()
    rows[:, :hq] = q
    sl = slots[:t].long()
    ok = sl >= 0
    pg, off = sl[ok] // page, sl[ok] % page
    pool[pg, 0, :, off] = k[ok]
    pool[pg, 1, :, off] = v[ok]


def _attention(prefill):
    def run(g, kv, q, out, ws_o, ws_ml, table, seq_lens, cu_q, work, work_count, seqs, hq, hk, q_stride, out_stride,
            max_pages, page, rows_per_seq, splits, pool_pages, scale_log2, err):
        d = kv._head_dim
        pool = kv.view(torch.bfloat16).view(-1, 2, hk, page, d)
        n_seqs = int(kv._vars_seqs)
        # a work list means a ragged call, whose sequences are split between the two kernels by rows
        small = max(1, 16 // (hq // hk)) if isinstance(work, torch.Tensor) else None
        grp = hq // hk
        scale = scale_log2 / 1.4426950408889634
        tb = table.view(-1, max_pages)
        for s in range(n_seqs):
            L = int(seq_lens[s])
            if isinstance(cu_q, torch.Tensor):
                r0, r1 = int(cu_q[s]), int(cu_q[s + 1])
            else:
                r0, r1 = s * rows_per_seq, (s + 1) * rows_per_seq
            R = r1 - r0
            if R <= 0 or L <= 0:
                continue
            if small is not None and isinstance(cu_q, torch.Tensor) and ((R <= small) == prefill):
                continue
            npg = -(-L // page)
            pages = tb[s, :npg].long()
            kk = _f(pool[pages, 0]).permute(0, 2, 1, 3).reshape(-1, hk, d)[:L]
            vv = _f(pool[pages, 1]).permute(0, 2, 1, 3).reshape(-1, hk, d)[:L]
            qq = _f(torch.as_strided(q, (R, hq, d), (q_stride, d, 1), q.storage_offset() + r0 * q_stride))
            sc = torch.einsum("rhd,lhd->hrl", qq, kk.repeat_interleave(grp, 1)) * scale
            posn = torch.arange(L - R, L)
            mask = torch.arange(L)[None, :] <= posn[:, None]
            sc = sc.masked_fill(~mask[None], float("-inf"))
            if (splits >> 16) and isinstance(ws_o, torch.Tensor):
                # context-parallel partial mode: un-normalised (o, m, l) in the log2 domain into the first of this
                # launch's slots, the other slots neutral; a merge over every member's slots finishes
                nsplit, base, total = splits & 0xff, (splits >> 8) & 0xff, splits >> 16
                s2 = sc * 1.4426950408889634                                      # [hq, R, L]
                m = s2.max(-1).values                                             # [hq, R]
                pr = torch.exp2(s2 - m[..., None])
                l = pr.sum(-1)
                o = torch.einsum("hrl,lhd->rhd", pr, vv.repeat_interleave(grp, 1))   # [R, hq, d]
                wo = ws_o.view(-1, d)
                wml = ws_ml.view(-1, 2)
                for r in range(R):
                    for hh in range(hq):
                        at = ((r0 + r) * hq + hh) * total + base
                        wo[at] = o[r, hh]
                        wml[at, 0], wml[at, 1] = m[hh, r], l[hh, r]
                        for x in range(1, nsplit):
                            wo[at + x] = 0
                            wml[at + x, 0], wml[at + x, 1] = float("-inf"), 0.0
                continue
            o = torch.einsum("hrl,lhd->rhd", torch.softmax(sc, -1), vv.repeat_interleave(grp, 1))
            torch.as_strided(out, (R, hq * d), (out_stride, 1), out.storage_offset() + r0 * out_stride).copy_(o.reshape(R, hq * d).to(out.dtype))
    return run


def k_noop(g, *a):
    return None


def k_last_row(g, src, dst, cu, seqs, row_bytes):
    n = g[0]
    w = row_bytes // src.element_size()
    idx = cu[1:n + 1].long() - 1
    dst.view(-1, w)[:n] = src.view(-1, w)[idx.clamp(min=0)]


def k_argmax_partial(g, logits, pv, pi, rows, vocab, stride):
    r = g[0]
    lv = _f(torch.as_strided(logits, (r, vocab), (stride, 1)))
    lv = torch.nan_to_num(lv, nan=float("-inf"))
    mx = lv.max(-1, keepdim=True).values
    idx = torch.where(lv == mx, torch.arange(vocab)[None], torch.full((1,), vocab)).min(-1).values
    pv.view(-1)[:r] = mx[:, 0]
    pi.view(-1)[:r] = idx.to(pi.dtype)


def k_argmax_final(g, pv, pi, out, rows, parts):
    r = g[0]
    out[:r] = pi.view(-1)[:r].long()


def k_sample(g, logits, probs, out, temperature, top_k, top_p, min_p, seeds, offsets, rows, vocab, stride):
    from .ops.sampling_ref import sample_rows

    r = g[0]
    lv = _f(torch.as_strided(logits, (r, vocab), (stride, 1)))
    out[:r] = sample_rows(lv, temperature[:r], top_k[:r], top_p[:r], min_p[:r], seeds[:r], offsets[:r])


def k_rope_table(g, cos, sin, max_pos, rot, theta_bits):
    theta = struct.unpack("<d", struct.pack("<q", theta_bits))[0]
    half = rot // 2
    inv = theta ** (-torch.arange(0, half, dtype=torch.float64) * 2.0 / rot)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None]
    cos.view(-1)[: max_pos * half] = ang.cos().float().reshape(-1)
    sin.view(-1)[: max_pos * half] = ang.sin().float().reshape(-1)


def k_silu_mul(g, x, out, tokens, d):
    t = g[0]
    xv = _f(x[: t * 2 * d].view(t, 2 * d))
    out[: t * d] = (torch.nn.functional.silu(xv[:, :d]) * xv[:, d:]).reshape(-1).to(out.dtype)


def k_sigmoid_mul(g, x, gate, out, tokens, d, xs, gs):
    t = g[0]
    xv = _f(torch.as_strided(x, (t, d), (xs, 1), x.storage_offset()))
    gv = _f(torch.as_strided(gate, (t, d), (gs, 1), gate.storage_offset()))
    res = (xv * torch.sigmoid(gv)).to(out.dtype)
    out[: t * d] = res.reshape(-1)


def _rows_of(cu, s):
    return (int(cu[s]), int(cu[s + 1])) if isinstance(cu, torch.Tensor) else (s, s + 1)


def _gdn_window(state, line, line_bytes, width, conv_dim):
    return state[line * line_bytes: line * line_bytes + (width - 1) * conv_dim * 2].view(torch.bfloat16).view(width - 1, conv_dim)


def k_gdn_conv(g, x, y, state, lines, cu, w, bias, seqs, rows, conv_dim, width, x_stride, line_bytes, rpc):
    from .ops import gdn as G

    wt = _f(w[: conv_dim * width].view(conv_dim, width))
    for s in range(seqs):
        r0, r1 = _rows_of(cu, s)
        if r1 <= r0:
            continue
        ln = int(lines[s])
        hist = _f(_gdn_window(state, ln, line_bytes, width, conv_dim)) if ln > 0 else torch.zeros(width - 1, conv_dim)
        xs = _f(torch.as_strided(x, (r1 - r0, conv_dim), (x_stride, 1), x.storage_offset() + r0 * x_stride))
        out, _ = G.conv_ref(xs, hist, wt, _f(bias[:conv_dim]) if isinstance(bias, torch.Tensor) else None)
        y[r0 * conv_dim: r1 * conv_dim] = out.to(torch.bfloat16).reshape(-1)


def k_gdn_conv_state(g, x, state, lines, cu, seqs, conv_dim, width, x_stride, line_bytes):
    for s in range(g[0]):
        r0, r1 = _rows_of(cu, s)
        ln = int(lines[s])
        if r1 <= r0 or ln <= 0:
            continue
        win = _gdn_window(state, ln, line_bytes, width, conv_dim)
        xs = torch.as_strided(x, (r1 - r0, conv_dim), (x_stride, 1), x.storage_offset() + r0 * x_stride)
        full = torch.cat([win.clone(), xs], 0)
        win.copy_(full[full.shape[0] - (width - 1):])


def k_gdn_conv_step(g, x, y, state, lines, w, bias, seqs, conv_dim, width, x_stride, line_bytes):
    n = g[0]
    k_gdn_conv((n, 1, 1), x, y, state, lines, 0, w, bias, n, n, conv_dim, width, x_stride, line_bytes, 1)
    k_gdn_conv_state((n, 1, 1), x, state, lines, 0, n, conv_dim, width, x_stride, line_bytes)


def _gdn_rule(dim):
    def run(g, qkv, zba, o_raw, state, lines, cu, A_log, dt_bias, seqs, hk, hv, zba_stride, b_off, a_off, line_bytes, s_off, tb):
        from .ops import gdn as G

        conv_dim = 2 * hk * dim + hv * dim
        for s in range(g[1]):
            r0, r1 = _rows_of(cu, s)
            n = r1 - r0
            if n <= 0:
                continue
            ln = int(lines[s])
            Sb = state[ln * line_bytes + s_off: ln * line_bytes + s_off + hv * dim * dim * 4].view(torch.float32).view(hv, dim, dim)
            S0 = Sb.clone() if ln > 0 else torch.zeros(hv, dim, dim)
            rows = _f(qkv[r0 * conv_dim: r1 * conv_dim].view(n, conv_dim))
            zr = _f(torch.as_strided(zba, (n, a_off + hv), (zba_stride, 1), zba.storage_offset() + r0 * zba_stride))
            q = rows[:, :hk * dim].view(n, hk, dim)
            k = rows[:, hk * dim:2 * hk * dim].view(n, hk, dim)
            v = rows[:, 2 * hk * dim:].view(n, hv, dim)
            o, S1 = G.rule_ref(q, k, v, None, zr[:, b_off:b_off + hv], zr[:, a_off:a_off + hv], S0, A_log[:hv], dt_bias[:hv],
                               None, normalize=False)
            o_raw[r0 * hv * dim: r1 * hv * dim] = o.reshape(-1)
            if ln > 0:
                Sb.copy_(S1)
    return run


def _gdn_step(dim):
    rule = _gdn_rule(dim)

    def run(g, qkv, zba, out, state, lines, A_log, dt_bias, norm_w, seqs, hk, hv, zba_stride, z_off, b_off, a_off,
            line_bytes, s_off, eps):
        n = g[1]
        o_raw = torch.zeros(n * hv * dim, dtype=torch.float32)
        rule((hv, n, 1), qkv, zba, o_raw, state, lines, 0, A_log, dt_bias, seqs, hk, hv, zba_stride, b_off, a_off,
             line_bytes, s_off, 1)
        k_gdn_gate_norm(((hv + 3) // 4, n, 1), o_raw, zba, out, norm_w, n, hv, dim, zba_stride, z_off, eps)
    return run


def k_gdn_chunk_prep(g, qkv, zba, cu, A_log, dt_bias, Wg, Qg, Kg, Ug, Mg, Gg, seqs, hk, hv, zba_stride, b_off, a_off):
    from .ops import gdn as G

    dim = 128
    conv_dim = 2 * hk * dim + hv * dim
    for s in range(seqs):
        r0, r1 = _rows_of(cu, s)
        n = r1 - r0
        if n <= 0:
            continue
        rows = _f(qkv[r0 * conv_dim: r1 * conv_dim].view(n, conv_dim))
        zr = _f(torch.as_strided(zba, (n, a_off + hv), (zba_stride, 1), zba.storage_offset() + r0 * zba_stride))
        q = rows[:, :hk * dim].view(n, hk, dim)
        k = rows[:, hk * dim:2 * hk * dim].view(n, hk, dim)
        v = rows[:, 2 * hk * dim:].view(n, hv, dim)
        parts = G.chunk_prep_ref(q, k, v, zr[:, b_off:b_off + hv], zr[:, a_off:a_off + hv], A_log[:hv], dt_bias[:hv])
        for dst, src, w in zip((Wg, Qg, Kg, Ug, Mg, Gg), parts, (dim, dim, dim, dim, 64, 1)):
            dst[r0 * hv * w: r1 * hv * w] = src.reshape(-1)


def k_gdn_chunk_rule(g, Wg, Qg, Kg, Ug, Mg, Gg, o_raw, state, lines, cu, seqs, hv, line_bytes, s_off):
    from .ops import gdn as G

    dim = 128
    for s in range(seqs):
        r0, r1 = _rows_of(cu, s)
        n = r1 - r0
        if n <= 0:
            continue
        ln = int(lines[s])
        Sb = state[ln * line_bytes + s_off: ln * line_bytes + s_off + hv * dim * dim * 4].view(torch.float32).view(hv, dim, dim)
        S0 = Sb.clone() if ln > 0 else torch.zeros(hv, dim, dim)
        cut = lambda t, w: t[r0 * hv * w: r1 * hv * w].view(n, hv, w) if w > 1 else t[r0 * hv: r1 * hv].view(n, hv)
        o, S1 = G.chunk_rule_ref(cut(Wg, dim), cut(Qg, dim), cut(Kg, dim), cut(Ug, dim), cut(Mg, 64), cut(Gg, 1), S0)
        o_raw[r0 * hv * dim: r1 * hv * dim] = o.reshape(-1)
        if ln > 0:
            Sb.copy_(S1)


def k_gdn_gate_norm(g, o_raw, zba, out, norm_w, tokens, hv, dv, zba_stride, z_off, eps):
    from .ops import gdn as G

    t = g[1]
    o = o_raw[: t * hv * dv].view(t, hv, dv)
    z = _f(torch.as_strided(zba, (t, hv * dv), (zba_stride, 1), zba.storage_offset() + z_off)).view(t, hv, dv)
    out[: t * hv * dv] = G.gate_norm_ref(o, z, norm_w[:dv], eps).to(torch.bfloat16).reshape(-1)


def k_copy_rows(g, src, dst, idx, rows, row_bytes, ss, ds):
    r = g[0]
    s8, d8 = src.view(torch.uint8), dst.view(torch.uint8)
    for i in range(r):
        j = int(idx[i]) if isinstance(idx, torch.Tensor) else i
        if j >= 0:
            d8[i * ds:i * ds + row_bytes] = s8[j * ss:j * ss + row_bytes]


def k_fill(g, p, n, v):
    p[:n] = v


CPU_KERNELS = {
    "kern_embedding_i64_bf16": k_embedding, "kern_embedding_i32_bf16": k_embedding,
    "kern_rms_norm_bf16": k_rms_norm, "kern_rms_norm_wide_bf16": k_rms_norm,
    "kern_fused_add_rms_norm_bf16": k_fused_add_rms_norm,
    "kern_rope_kv_append_bf16": k_rope_append, "kern_rope_table_f32": k_rope_table,
    "kern_attn_plan": k_noop, "kern_attn_merge_splits": k_noop,
    "kern_last_row": k_last_row, "kern_argmax_partial_bf16": k_argmax_partial, "kern_argmax_partial_f32": k_argmax_partial,
    "kern_argmax_final_i64": k_argmax_final, "kern_sample_bf16": k_sample, "kern_sample_f32": k_sample,
    "kern_silu_mul_bf16": k_silu_mul, "kern_copy_rows": k_copy_rows, "kern_sigmoid_mul_bf16": k_sigmoid_mul,
    "kern_gdn_conv_bf16": k_gdn_conv, "kern_gdn_conv_state": k_gdn_conv_state, "kern_gdn_rule_k128_v128": _gdn_rule(128), "kern_gdn_rule_k64_v64": _gdn_rule(64),
    "kern_gdn_rule_k32_v32": _gdn_rule(32), "kern_gdn_gate_norm_bf16": k_gdn_gate_norm,
    "kern_gdn_step_k128_v128": _gdn_step(128), "kern_gdn_step_k64_v64": _gdn_step(64), "kern_gdn_step_k32_v32": _gdn_step(32),
    "kern_gdn_conv_step_bf16": k_gdn_conv_step,
    "kern_gdn_chunk_prep_k128_v128": k_gdn_chunk_prep, "kern_gdn_chunk_rule_k128_v128": k_gdn_chunk_rule,
    "kern_gdn_rule_dec_k128_v128": _gdn_rule(128), "kern_gdn_rule_dec_k64_v64": _gdn_rule(64), "kern_gdn_rule_dec_k32_v32": _gdn_rule(32),
    "kern_fill_f32": k_fill, "kern_fill_i32": k_fill, "kern_fill_i64": k_fill, "kern_fill_u8": k_fill,
}
for _bn in (256, 128, 64, 32):
    for _epi, _sfx in (("store", ""), ("acc", "_acc"), ("f32", "_f32"), ("swiglu", "_swiglu")):
        CPU_KERNELS[f"kern_gemm_bf16_tn{_sfx}_n{_bn}"] = _gemm(_epi)
        for _mt in (1, 2, 4, 8):
            CPU_KERNELS[f"kern_gemv_bf16_tn{_sfx}_m{_mt}"] = _gemv(_epi)
def _attention_fmha(g, kv, q, out, table, seq_lens, cu_q, work, work_count, hq, hk, q_stride, out_stride, max_pages, page,
                    pool_pages, scale_log2, err):
    """The tcgen05 prefill kernel's statement: the same arithmetic as the row-parallel kernel's."""
    _attention(True)(g, kv, q, out, 0, 0, table, seq_lens, cu_q, work, work_count, 0, hq, hk, q_stride, out_stride, max_pages,
                     page, 1, 1, pool_pages, scale_log2, err)


def _attention_ragged(g, kv, q, out, table, seq_lens, cu_q, work_p, count_p, work_d, count_d, hq, hk, q_stride, out_stride,
                      max_pages, page, pool_pages, scale_log2, err):
    """Both work lists of a ragged call in one launch: the row-parallel and the token-parallel kernel's statements."""
    for prefill, work, count in ((True, work_p, count_p), (False, work_d, count_d)):
        _attention(prefill)(g, kv, q, out, 0, 0, table, seq_lens, cu_q, work, count, 0, hq, hk, q_stride, out_stride,
                            max_pages, page, 1, 1, pool_pages, scale_log2, err)


CPU_KERNELS["kern_attn_fmha_prefill_d128"] = _attention_fmha
CPU_KERNELS["kern_attn_fmha_prefill_d128_t64"] = _attention_fmha
for _d in (64, 128):
    CPU_KERNELS[f"kern_attn_ragged_paged_d{_d}"] = _attention_ragged
CPU_KERNELS["kern_attn_ragged_fmha_d128"] = _attention_ragged
for _d in (16, 32, 64, 128, 256):
    CPU_KERNELS[f"kern_attn_prefill_paged_d{_d}"] = _attention(True)
    CPU_KERNELS[f"kern_attn_decode_paged_d{_d}"] = _attention(False)


def register(entry: str, fn) -> None:
    """Add the CPU statement of another kernel entry (model families register theirs on import)."""
    CPU_KERNELS[entry] = fn


class CpuRuntime:
    def __init__(self, manifest, weights=None, tokens: int = 4096, slots: int = 0, topology=None, **_):
        text = manifest_text(manifest)
        m, errs = _native.verify(text)
        if m is None:
            raise ValueError("manifest does not verify:\n  - " + "\n  - ".join(errs))
        self.doc = json.loads(m.to_json())
        try:
            self.protocol = json.loads(m.protocol())
        except ValueError:
            try:
                self.protocol = json.loads(m.protocol(sampled=False))
            except ValueError:
                self.protocol = None
        self.topology = dict(topology or {})
        vmax = {k: v["max"] for k, v in self.doc["vars"].items()}
        self.buffers, self.states = {}, {}
        for name, b in self.doc["buffers"].items():
            shape = [d if isinstance(d, int) else vmax[d] for d in b["shape"]]
            self.buffers[name] = torch.zeros(int(np.prod(shape)) if shape else 1, dtype=_TORCH[b["dtype"]])
        self.page_unit = 1
        for b in self.doc["buffers"].values():
            dom = b.get("domain") or {}
            st = self.doc["states"].get(dom.get("index_into", ""))
            if st and (st.get("bytes_per_token") or st.get("host")) and "fill" not in b:
                self.page_unit = math.lcm(self.page_unit, dom.get("stride", 1))
        self.pages = max(1, tokens // self.page_unit)
        self.slots = slots
        for name, s in self.doc["states"].items():
            if s.get("bytes_per_token"):
                n = s["bytes_per_token"] * self.page_unit * self.pages
            elif s.get("bytes_per_seq"):
                n = s["bytes_per_seq"] * (slots + 1)
            else:
                n = s.get("bytes", 0)
            self.states[name] = torch.zeros(n, dtype=torch.uint8)
        self.scratch = {}
        for oname, op in self.doc["ops"].items():
            for sname, sc in op["impl"].get("scratch", {}).items():
                shape = [d if isinstance(d, int) else vmax[d] for d in sc["shape"]]
                self.scratch[(oname, sname)] = torch.zeros(int(np.prod(shape)), dtype=_TORCH[sc["dtype"]])
        self.launches_total = 0
        self.graphs = 0
        self._vars = {}
        if weights is not None:
            self.load_weights(weights)

    # ---- load ----
    def load_weights(self, weights) -> None:
        tensors = weights if isinstance(weights, dict) else read_safetensors(weights)
        for name, b in self.doc["buffers"].items():
            if b["kind"] not in ("weight", "source"):
                continue
            parts = []
            for seg in b["bind"]:
                t = tensors[self._pick(seg["tensor"])]
                t2 = t.reshape(t.shape[0], -1) if t.dim() > 1 else t.reshape(-1, 1)
                if "interleave" in seg:
                    u = tensors[self._pick(seg["interleave"]["with"])].reshape(t2.shape)
                    n = seg["interleave"]["rows"]
                    parts.append(torch.stack([t2.view(-1, n, t2.shape[1]), u.view(-1, n, t2.shape[1])], 1).reshape(-1))
                    continue
                r = self._range(seg.get("rows"), t2.shape[0])
                c = self._range(seg.get("cols"), t2.shape[1])
                parts.append(t2[r[0]:r[1], c[0]:c[1]].reshape(-1))
            flat = torch.cat(parts)
            if flat.numel() != self.buffers[name].numel():
                raise ValueError(f"buffer `{name}`: bound tensors hold {flat.numel()} elements, the buffer {self.buffers[name].numel()}")
            self.buffers[name].copy_(flat.to(self.buffers[name].dtype))
        for pname, p in self.doc["programs"].items():
            if p.get("derive"):
                self.issue(pname, {k: v["max"] for k, v in self.doc["vars"].items()})

    # ---- hosted ----
    @property
    def awaits_host(self) -> bool:
        return any(s.get("host") and self.states[n].numel() == 0 for n, s in self.doc["states"].items())

    def bind_host_tensors(self, tensors: dict) -> None:
        """Host-owned states: the engine's own (CPU) tensors become the states, shared, not copied."""
        for name, t in tensors.items():
            decl = self.doc["states"].get(name, {}).get("host")
            if decl is None:
                raise ValueError(f"`{name}` is not a host state of this manifest")
            if list(t.shape[1:]) != decl["shape"][1:] or list(t.stride()) != decl["strides"]:
                raise ValueError(f"host state `{name}`: tensor {list(t.shape)}/{list(t.stride())} is not the declared "
                                 f"{decl['shape']}/{decl['strides']}")
            self.states[name] = t.view(-1).view(torch.uint8)
        missing = [n for n, s in self.doc["states"].items() if s.get("host") and n not in tensors]
        if missing:
            raise ValueError(f"host state `{missing[0]}` was not bound")

    def _pick(self, t):
        return t if isinstance(t, str) else t["tensors"][self.rank(t["group"])]

    def _range(self, r, whole):
        if r is None:
            return (0, whole)
        return tuple(r) if isinstance(r, list) else tuple(r["ranges"][self.rank(r["group"])])

    def rank(self, group: str) -> int:
        return self.topology.get(group, (0, 1))[0]

    def once(self) -> None:
        for pname, p in self.doc["programs"].items():
            if p.get("once"):
                self.issue(pname, {k: v["max"] for k, v in self.doc["vars"].items()})

    # ---- memory ----
    def tensor(self, name: str) -> torch.Tensor:
        if name in self.states:
            return self.states[name]
        b = self.doc["buffers"][name]
        shape = [d if isinstance(d, int) else self.doc["vars"][d]["max"] for d in b["shape"]]
        return self.buffers[name].view(shape)

    def write(self, name: str, data, offset: int = 0) -> None:
        buf = self.buffers[name]
        src = data if isinstance(data, torch.Tensor) else torch.as_tensor(np.asarray(data))
        src = src.reshape(-1)
        at = offset // buf.element_size()
        buf[at:at + src.numel()] = src.to(buf.dtype)

    def read(self, name: str, count: int | None = None, offset: int = 0, out=None):
        buf = self.buffers[name]
        at = offset // buf.element_size()
        if out is not None:
            out.copy_(buf[at:at + out.numel()].to(out.dtype))
            return out
        n = buf.numel() - at if count is None else count
        return buf[at:at + n].clone().numpy() if buf.dtype != torch.bfloat16 else buf[at:at + n].view(torch.int16).numpy().view(np.uint16).copy()

    def synchronize(self) -> None:
        pass

    def check_error(self) -> None:
        pass

    def zero_slot(self, slot: int) -> None:
        for name, s in self.doc["states"].items():
            if s.get("bytes_per_seq"):
                n = s["bytes_per_seq"]
                self.states[name][slot * n:(slot + 1) * n] = 0

    def run_copies(self, copies: dict) -> None:
        for name, s in self.doc["states"].items():
            st = self.states[name]
            if s.get("bytes_per_token"):
                n = s["bytes_per_token"] * self.page_unit
                for a, b in copies["pages"]:
                    st[b * n:(b + 1) * n] = st[a * n:(a + 1) * n].clone()
            elif s.get("bytes_per_seq") and copies["slot"] is not None:
                n = s["bytes_per_seq"]
                a, b = copies["slot"]
                st[b * n:(b + 1) * n] = st[a * n:(a + 1) * n].clone()

    # ---- another runtime's pools (prefill tier -> decode tier), in host memory: a "mapped pool" is the other runtime's tensor ----
    def export_states(self) -> dict:
        return dict(self.states)

    def map_pool(self, handles: dict) -> dict:
        return dict(handles)

    def state_bytes(self) -> dict[str, int]:
        return {n: int(t.numel()) for n, t in self.states.items()}

    def _unit_bytes(self, name: str) -> int:
        s = self.doc["states"][name]
        return s["bytes_per_token"] * self.page_unit if s.get("bytes_per_token") else s.get("bytes_per_seq", 0)

    def push_state_unit(self, state: str, dst, src_unit: int, dst_unit: int) -> None:
        n = self._unit_bytes(state)
        dst[dst_unit * n:(dst_unit + 1) * n] = self.states[state][src_unit * n:(src_unit + 1) * n]

    def push(self, mapped: dict, plan: dict) -> None:
        for name, s in self.doc["states"].items():
            if s.get("bytes_per_token"):
                for a, b in plan["pages"]:
                    self.push_state_unit(name, mapped[name], a, b)
            elif s.get("bytes_per_seq") and plan.get("slot") is not None:
                self.push_state_unit(name, mapped[name], plan["slot"][0], plan["slot"][1])

    def _push_copies(self, state: str, src_off: int, dst, dst_off: int, dst_bytes: int, copies) -> int:
        src = self.states[state]
        for (s0, d0, width, sp, dp, rows) in copies:
            if rows and (src_off + s0 + (rows - 1) * sp + width > src.numel() or d0 + (rows - 1) * dp + width > dst_bytes):
                raise ValueError(f"push of `{state}`: a copy runs past the end of one side")
            for r in range(rows):
                a, b = src_off + s0 + r * sp, dst_off + d0 + r * dp
                dst[b:b + width] = src[a:a + width]
        return len(copies)

    def push_rows(self, state: str, dst, dst_bytes: int, runs, row_bytes: int) -> int:
        return self._push_copies(state, 0, dst, 0, dst_bytes, _native.dealt_copies([tuple(r) for r in runs], row_bytes))

    def push_slot_part(self, state: str, dst, dst_bytes: int, from_slot: int, into_slot: int, segments, of: int, part: int) -> int:
        mine = int(self.doc["states"][state]["bytes_per_seq"])
        line = _native.split_line(list(segments), of)
        if mine % line or mine % of:
            raise ValueError(f"state `{state}`: a slot of {mine} bytes is not whole lines of {line} bytes over {of} members")
        theirs = mine // of
        return self._push_copies(state, from_slot * mine, dst, into_slot * theirs, dst_bytes - into_slot * theirs,
                                 _native.split_copies(list(segments), of, mine // line, part))

    # ---- execution ----
    def _resolve_call_arg(self, a, ptype):
        if "buf" in a:
            buf = self.buffers[a["buf"]]
            return buf[a.get("offset", 0) // buf.element_size():]
        if "state" in a:
            return self.states[a["state"]][a.get("offset", 0):]
        if "var" in a:
            return self._vars[a["var"]]
        if "expr" in a:
            return _eval(a["expr"], self._vars)
        if "rank" in a:
            return self.rank(a["rank"])
        return next(iter(a.values()))

    def issue_range(self, program: str, vars: dict[str, int], lo: int, hi: int) -> int:
        return self.issue(program, vars, calls=(lo, hi))

    def issue(self, program: str, vars: dict[str, int], eager: bool = False, calls: tuple[int, int] | None = None) -> int:
        self._vars = dict(vars)
        p = self.doc["programs"][program]
        n = 0
        for call in (p["calls"] if calls is None else p["calls"][calls[0]:calls[1]]):
            op = self.doc["ops"][call["op"]]
            cargs = [self._resolve_call_arg(a, pt) for a, pt in zip(call["args"], op["params"])]
            for l in op["impl"]["launches"]:
                w = l.get("when")
                if w and not (w.get("min", 0) <= vars[w["var"]] <= w.get("max", 1 << 62)):
                    continue
                largs = l.get("args") or [{"param": i} for i in range(len(op["params"]))]
                vals = []
                for la in largs:
                    if "param" in la:
                        vals.append(cargs[la["param"]])
                    elif "scratch" in la:
                        vals.append(self.scratch[(call["op"], la["scratch"])])
                    elif "rank" in la:
                        vals.append(self.rank(la["rank"]))
                    elif "pack" in la:
                        vals.append(self._pack(la["pack"], cargs, call["op"]))
                    else:
                        vals.append(next(iter(la.values())))
                entry = l["entry"]
                if entry.startswith("extern:nccl_"):
                    grp = largs[3].get("rank") or call["args"][largs[3]["param"]]["rank"]
                    self._collective(entry, vals[0], vals[1], int(vals[2]), grp)
                    n += 1
                    continue
                fn = CPU_KERNELS.get(entry)
                if fn is None:          # model families register their kernels' statements when imported
                    import importlib

                    for mod in ("toy_int", "spec", "moe"):
                        importlib.import_module(f"kern_b200.models.{mod}")
                    fn = CPU_KERNELS.get(entry)
                if fn is None:
                    raise NotImplementedError(f"no CPU statement of `{entry}` is registered")
                grid = [_eval(g, vars) for g in l.get("grid", [1, 1, 1])]
                if 0 in grid:
                    continue
                fn(grid, *vals)
                n += 1
        self.launches_total += n
        return n

    run = issue

    def _collective(self, entry: str, send, recv, count: int, group: str) -> None:
        """`extern:nccl_<coll>_<elem>` with [send, recv, count, rank]: count elements per rank (per peer for an
        all-to-all). A group of one is a copy; larger groups go through the process's `torch.distributed` default
        group (gloo on CPU), whose world must be the group.  Reference: crates/kern-runtime/src/nccl.rs:190."""
        coll, elem = entry[len("extern:nccl_"):].split("_")
        dt = {"f32": torch.float32, "bf16": torch.bfloat16, "i32": torch.int32, "u8": torch.uint8}[elem]
        world = self.topology.get(group, (0, 1))[1]
        ins = count * (world if coll in ("reducescatter", "alltoall") else 1)
        outs = count * (world if coll in ("allgather", "alltoall") else 1)
        src, dst = send.view(dt)[:ins], recv.view(dt)[:outs]
        if src.numel() < ins or dst.numel() < outs:
            raise ValueError(f"{entry}: {count} elements per rank need {ins} to send and {outs} to receive")
        if count == 0:
            return
        if world == 1:
            dst.copy_(src)
            return
        import torch.distributed as dist

        if not dist.is_initialized() or dist.get_world_size() != world:
            raise RuntimeError(f"{entry}: group `{group}` of {world} needs torch.distributed initialised with that world")
        wide = src.float() if dt in (torch.bfloat16,) and coll in ("allreduce", "reducescatter") else src.clone()
        if coll == "allreduce":
            dist.all_reduce(wide)
            dst.copy_(wide.to(dt))
        elif coll == "allgather":
            parts = [torch.empty_like(wide) for _ in range(world)]
            dist.all_gather(parts, wide)
            dst.copy_(torch.cat(parts))
        elif coll == "reducescatter":
            dist.all_reduce(wide)
            r = self.rank(group)
            dst.copy_(wide[r * count:(r + 1) * count].to(dt))
        else:
            outp = [torch.empty(count, dtype=dt) for _ in range(world)]
            dist.all_to_all(outp, list(wide.split(count))) if dist.get_backend() != "gloo" else self._a2a_gloo(outp, wide, count, world, group)
            dst.copy_(torch.cat(outp))

    def _a2a_gloo(self, outp, wide, count, world, group):
        """gloo has no all-to-all: every rank gathers all blocks and keeps the ones addressed to it."""
        import torch.distributed as dist

        parts = [torch.empty_like(wide) for _ in range(world)]
        dist.all_gather(parts, wide)
        r = self.rank(group)
        for p in range(world):
            outp[p].copy_(parts[p][r * count:(r + 1) * count])

    def _pack(self, pack, cargs, opname):
        """A pack holding one tensor map stands for the tensor it describes (row stride and head dim kept)."""
        for f in pack["fields"]:
            if "tensormap" in f:
                tm = f["tensormap"]
                t = cargs[tm["param"]]
                es = {"bf16": 2, "f16": 2, "f32": 4, "u8": 1}.get(tm["dtype"], 2)
                view = t.view(t.dtype)
                holder = view[:]           # a fresh tensor object to carry attributes
                holder._row_stride = tm["strides"][0] // es if tm.get("strides") else tm["dims"][0]
                holder._head_dim = tm["dims"][0]
                holder._vars_seqs = self._vars.get(self.protocol["groups"]["var"], 1) if self.protocol else 1
                return holder
        return pack


# ---- block-draft helpers and the state advance (statements: ops/draft.py) ------------------------------------------
def _k_topk(g, logits, ids, vals, n, row_stride, k):
    from .ops import draft as D

    rows = g[0]
    x = torch.as_strided(logits, (rows, n), (row_stride, 1), logits.storage_offset())
    i, v = D.topk_ref(x, k)
    ids[: rows * k] = i.reshape(-1)
    vals[: rows * k] = v.reshape(-1)


def _k_mask_row0(g, dst, src, rows, rows_per_seq, cols):
    from .ops import draft as D

    r = g[0]
    dst[: r * cols] = D.mask_row0_ref(src[: r * cols].view(r, cols), rows_per_seq).reshape(-1)


def _k_conv_shift(g, lines, line_stride, state, accepted, seqs, line_bytes, tok_bytes):
    from .ops import draft as D

    n = g[0]
    D.conv_shift_ref(torch.as_strided(lines, (n, line_stride), (line_stride, 1), lines.storage_offset()), state, accepted,
                     line_bytes, tok_bytes)


def _k_dflash_conv(g, x, delta, base, tokens, dim, groups, delta_stride, side):
    from .ops import draft as D

    T = min(tokens, g[0] * 8)
    d = torch.as_strided(delta, (T, 4 * groups), (delta_stride, 1), delta.storage_offset())
    x[: T * dim] = D.dflash_conv_ref(x[: T * dim].view(T, dim), d, base, groups, side).reshape(-1)


def _k_dflash_select(g, cand, unary, hidden_r, succ, pred, pred_anchor, out, steps, rank, hr_stride, rows_per_seq):
    from .ops import draft as D

    seqs = g[0]
    rows = seqs * rows_per_seq
    res = D.dflash_select_ref(cand[: rows * 16].view(rows, 16), unary[: rows * 16].view(rows, 16),
                              torch.as_strided(hidden_r, (rows, rank), (hr_stride, 1), hidden_r.storage_offset()),
                              succ[: rows * 16 * rank].view(rows, 16, rank), pred[: rows * 16 * rank].view(rows, 16, rank),
                              pred_anchor[: seqs * rank].view(seqs, rank), steps, rows_per_seq)
    out[: seqs * steps] = res.reshape(-1)


CPU_KERNELS.update({"kern_topk_bf16": _k_topk, "kern_mask_row0_bf16": _k_mask_row0, "kern_conv_shift": _k_conv_shift,
                    "kern_dflash_conv_bf16": _k_dflash_conv, "kern_dflash_select": _k_dflash_select})


# ---- the runtime's GEMM built-ins: C[m, n] = A[m, k] . W[n, k]^T ------------------------------------------------------
def _extern_gemm(acc: bool, f32_out: bool, fp8: bool):
    def run(g, a, w, c, *rest):
        if fp8:
            sa, sw, m, n, k = rest[:5]
            A = a[: m * k].view(torch.float8_e4m3fn).float().view(m, k) * float(sa[0])
            W = w[: n * k].view(torch.float8_e4m3fn).float().view(n, k) * float(sw[0])
            ldc = rest[5] if len(rest) > 5 else n
        else:
            m, n, k = rest[:3]
            ldc = rest[3] if len(rest) > 3 else n
            lda = rest[4] if len(rest) > 4 else k
            A = _f(torch.as_strided(a, (m, k), (lda, 1), a.storage_offset()))
            W = _f(w[: n * k].view(n, k))
        out = A @ W.t()
        C = torch.as_strided(c, (m, n), (ldc, 1), c.storage_offset())
        if acc:
            out = out + C.float()
        C.copy_(out if f32_out else out.to(torch.bfloat16))
    return run


def _extern_gemm_mx(g, a, w, c, sa, sw, m, n, k, ldc=None):
    """`extern:cublaslt_mxfp8_tn`: e4m3 operands, UE8M0 scales per 32 elements of K in 128 x 4 atoms."""
    from .ops import gemm_mx as G

    A = G.dequant_mxfp8(a[: m * k].view(m, k), G.atoms_to_sf(sa[: G.atom_bytes(m, k)], m, k))
    W = G.dequant_mxfp8(w[: n * k].view(n, k), G.atoms_to_sf(sw[: G.atom_bytes(n, k)], n, k))
    C = torch.as_strided(c, (m, n), (ldc or n, 1), c.storage_offset())
    C.copy_((A @ W.t()).to(torch.bfloat16))


CPU_KERNELS.update({
    "extern:cublaslt_mxfp8_tn": _extern_gemm_mx,
    "extern:cublaslt_bf16_tn": _extern_gemm(False, False, False), "extern:cublaslt_bf16_tn_acc": _extern_gemm(True, False, False),
    "extern:cublas_bf16_tn_f32": _extern_gemm(False, True, False), "extern:cublaslt_fp8_tn": _extern_gemm(False, False, True),
    "extern:cublaslt_fp8_tn_f32": _extern_gemm(False, True, True)})


# ---- decode context parallelism (statements of attn_paged.cu's dealing and merging kernels) -------------------------
def _k_dcp_local_lens(g, seq_lens, local_lens, seqs, rank, world):
    L = seq_lens[:seqs].long()
    local_lens[:seqs] = torch.where(L > rank, (L - rank + world - 1) // world, torch.zeros_like(L)).to(local_lens.dtype)


def _k_dcp_prepare(g, seq_lens, local_lens, ws_ml, seqs, rank, world, slots):
    n = g[0]
    _k_dcp_local_lens(g, seq_lens, local_lens, n, rank, world)
    w = ws_ml[: n * slots * 2].view(-1, 2)
    w[:, 0], w[:, 1] = float("-inf"), 0.0


def _k_attn_merge_ranks(g, ws_o, ws_ml, out, rows, hq, d, splits, ranks, out_stride):
    n = g[0]                                     # rows * hq as launched
    o = ws_o[: ranks * n * splits * d].view(ranks, n, splits, d).permute(1, 0, 2, 3).reshape(n, ranks * splits, d)
    ml = ws_ml[: ranks * n * splits * 2].view(ranks, n, splits, 2).permute(1, 0, 2, 3).reshape(n, ranks * splits, 2)
    m = ml[..., 0].max(-1, keepdim=True).values
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    f = torch.exp2(ml[..., 0] - m)
    l = (ml[..., 1] * f).sum(-1)
    acc = (o * f[..., None]).sum(1)
    res = torch.where(l[:, None] > 0, acc / l[:, None].clamp_min(1e-38), torch.zeros_like(acc))
    tokens = n // hq
    torch.as_strided(out, (tokens, hq * d), (out_stride, 1), out.storage_offset()).copy_(res.view(tokens, hq * d).to(out.dtype))


def _k_deal_rows(g, src, dst, src_table, dst_table, src_lens, seqs, src_width, dst_width, hk, d, page, rank, world, first_pos, err):
    sp = src.view(torch.bfloat16).view(-1, 2, hk, page, d)
    dp = dst.view(torch.bfloat16).view(-1, 2, hk, page, d)
    st, dt = src_table.view(-1, src_width), dst_table.view(-1, dst_width)
    for s in range(g[1]):
        for pos in range(rank, int(src_lens[s]), world):
            if pos < first_pos:
                continue
            li = pos // world
            dp[int(dt[s, li // page]), :, :, li % page] = sp[int(st[s, pos // page]), :, :, pos % page]


CPU_KERNELS.update({"kern_dcp_local_lens": _k_dcp_local_lens, "kern_dcp_prepare": _k_dcp_prepare,
                    "kern_attn_merge_ranks": _k_attn_merge_ranks, "kern_deal_rows_bf16": _k_deal_rows})


# ---- per-key-decay delta rule and latent attention (statements: ops/gdn.py kda_rule_ref, ops/mla.py) ---------------
def _kda_rule(dim):
    def run(g, qkv, zba, o_raw, state, lines, cu, A_log, dt_bias, gk, seqs, hk, hv, zba_stride, b_off, gk_stride, line_bytes,
            s_off, tb):
        from .ops import gdn as G

        conv_dim = 2 * hk * dim + hv * dim
        for s in range(g[1]):
            r0, r1 = _rows_of(cu, s)
            n = r1 - r0
            if n <= 0:
                continue
            ln = int(lines[s])
            Sb = state[ln * line_bytes + s_off: ln * line_bytes + s_off + hv * dim * dim * 4].view(torch.float32).view(hv, dim, dim)
            S0 = Sb.clone() if ln > 0 else torch.zeros(hv, dim, dim)
            rows = _f(qkv[r0 * conv_dim: r1 * conv_dim].view(n, conv_dim))
            b = _f(torch.as_strided(zba, (n, hv), (zba_stride, 1), zba.storage_offset() + r0 * zba_stride + b_off))
            gate = _f(torch.as_strided(gk, (n, hv * dim), (gk_stride, 1), gk.storage_offset() + r0 * gk_stride)).view(n, hv, dim)
            q = rows[:, :hk * dim].view(n, hk, dim)
            k = rows[:, hk * dim:2 * hk * dim].view(n, hk, dim)
            v = rows[:, 2 * hk * dim:].view(n, hv, dim)
            hvd = hv * dim
            T, rep = n, hv // hk
            qn = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) / dim ** 0.5
            kn = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
            qn, kn = qn.repeat_interleave(rep, 1), kn.repeat_interleave(rep, 1)
            dec = torch.exp(-torch.exp(A_log[:hv].float())[None, :, None] *
                            torch.nn.functional.softplus(gate + dt_bias[:hvd].float().view(1, hv, dim)))
            beta = _f(torch.sigmoid(b).to(torch.bfloat16))
            S = S0.float().clone()
            o = torch.empty(T, hv, dim)
            for t in range(T):
                S = S * dec[t][:, None, :]
                u = (v[t] - torch.einsum("hvk,hk->hv", S, kn[t])) * beta[t][:, None]
                S = S + u[:, :, None] * kn[t][:, None, :]
                o[t] = torch.einsum("hvk,hk->hv", S, qn[t])
            o_raw[r0 * hvd: r1 * hvd] = o.reshape(-1)
            if ln > 0:
                Sb.copy_(S)
    return run


def _kda_step(dim):
    rule = _kda_rule(dim)

    def run(g, qkv, zba, out, state, lines, A_log, dt_bias, norm_w, gk, seqs, hk, hv, zba_stride, z_off, b_off, gk_stride,
            line_bytes, s_off, eps):
        n = g[1]
        o_raw = torch.zeros(n * hv * dim, dtype=torch.float32)
        rule((hv, n, 1), qkv, zba, o_raw, state, lines, 0, A_log, dt_bias, gk, seqs, hk, hv, zba_stride, b_off, gk_stride,
             line_bytes, s_off, 1)
        k_gdn_gate_norm(((hv + 3) // 4, n, 1), o_raw, zba, out, norm_w, n, hv, dim, zba_stride, z_off, eps)
    return run


def _k_mla_rope_append(g, lat, q, cache, positions, slots, cos, sin, w, tokens, heads, lat_stride, q_stride, eps, kv_slots,
                       max_pos, err):
    t = g[0]
    pos = positions[:t].long().clamp(0, max_pos - 1)
    c, s = cos.view(-1, 32)[pos], sin.view(-1, 32)[pos]
    rows = _f(torch.as_strided(lat, (t, 576), (lat_stride, 1), lat.storage_offset()))
    comp = rows[:, :512]
    comp = comp * torch.rsqrt(comp.pow(2).mean(-1, keepdim=True) + eps) * _f(w[:512])
    a, b = rows[:, 512:544], rows[:, 544:]
    new = torch.cat([comp, a * c - b * s, b * c + a * s], -1).to(torch.bfloat16)
    sl = slots[:t].long()
    ok = sl >= 0
    cache.view(torch.bfloat16).view(-1, 576)[sl[ok]] = new[ok]
    qv = torch.as_strided(q, (t, heads, 576), (q_stride, 576, 1), q.storage_offset())
    qa, qb = _f(qv[..., 512:544]), _f(qv[..., 544:])
    qv[..., 512:544] = (qa * c[:, None] - qb * s[:, None]).to(torch.bfloat16)
    qv[..., 544:] = (qb * c[:, None] + qa * s[:, None]).to(torch.bfloat16)


def _k_mla_rows(g, positions, cu, seqs, tokens, row_seq, row_len):
    row_seq[:tokens] = 0
    row_len[:tokens] = 0
    for s in range(seqs):
        r0, r1 = int(cu[s]), int(cu[s + 1])
        row_seq[r0:r1] = s
        row_len[r0:r1] = (positions[r0:r1] + 1).to(torch.int32)


def _k_mla_decode(g, kv, q, out, ws_o, ws_ml, table, lens, seqs, heads, q_stride, out_stride, max_pages, page, splits,
                  pool_pages, scale_log2, err, row_seq):
    pool = kv.view(torch.bfloat16).view(-1, page, 576)
    tb = table.view(-1, max_pages)
    scale = scale_log2 / 1.4426950408889634
    for r in range(g[1]):
        L = int(lens[r])
        if L <= 0:
            continue
        trow = int(row_seq[r]) if isinstance(row_seq, torch.Tensor) else r
        lat = _f(pool[tb[trow, : -(-L // page)].long()]).reshape(-1, 576)[:L]
        qq = _f(torch.as_strided(q, (heads, 576), (576, 1), q.storage_offset() + r * q_stride))
        # a split launch is followed by the merge; here the first writes the finished rows and the merge is a no-op
        p = torch.softmax((qq @ lat.t()) * scale, -1)
        torch.as_strided(out, (heads * 512,), (1,), out.storage_offset() + r * out_stride).copy_((p @ lat[:, :512]).reshape(-1).to(out.dtype))


CPU_KERNELS.update({"kern_kda_rule_k128_v128": _kda_rule(128), "kern_kda_rule_k64_v64": _kda_rule(64),
                    "kern_kda_step_k128_v128": _kda_step(128), "kern_kda_step_k64_v64": _kda_step(64),
                    "kern_mla_rope_append_bf16": _k_mla_rope_append, "kern_mla_rows": _k_mla_rows,
                    "kern_mla_decode_bf16": _k_mla_decode})


def _k_kda_chunk_prep(g, qkv, zba, gk, cu, A_log, dt_bias, Wg, Qg, Kg, Ug, Mg, Dg, seqs, hk, hv, zba_stride, b_off, gk_stride):
    from .ops import gdn as G

    dim = 128
    conv_dim = 2 * hk * dim + hv * dim
    for s in range(seqs):
        r0, r1 = _rows_of(cu, s)
        n = r1 - r0
        if n <= 0:
            continue
        rows = _f(qkv[r0 * conv_dim: r1 * conv_dim].view(n, conv_dim))
        b = _f(torch.as_strided(zba, (n, hv), (zba_stride, 1), zba.storage_offset() + r0 * zba_stride + b_off))
        gate = _f(torch.as_strided(gk, (n, hv * dim), (gk_stride, 1), gk.storage_offset() + r0 * gk_stride)).view(n, hv, dim)
        q = rows[:, :hk * dim].view(n, hk, dim)
        k = rows[:, hk * dim:2 * hk * dim].view(n, hk, dim)
        v = rows[:, 2 * hk * dim:].view(n, hv, dim)
        parts = G.kda_chunk_prep_ref(q, k, v, b, gate, A_log[:hv], dt_bias[:hv * dim].view(hv, dim))
        for dst, src, w in zip((Wg, Qg, Kg, Ug, Mg, Dg), parts, (dim, dim, dim, dim, 64, dim)):
            dst[r0 * hv * w: r1 * hv * w] = src.reshape(-1)


def _k_kda_chunk_rule(g, Wg, Qg, Kg, Ug, Mg, Dg, o_raw, state, lines, cu, seqs, hv, line_bytes, s_off):
    from .ops import gdn as G

    dim = 128
    for s in range(seqs):
        r0, r1 = _rows_of(cu, s)
        n = r1 - r0
        if n <= 0:
            continue
        ln = int(lines[s])
        Sb = state[ln * line_bytes + s_off: ln * line_bytes + s_off + hv * dim * dim * 4].view(torch.float32).view(hv, dim, dim)
        S0 = Sb.clone() if ln > 0 else torch.zeros(hv, dim, dim)
        cut = lambda t, w: t[r0 * hv * w: r1 * hv * w].view(n, hv, w)
        o, S1 = G.chunk_rule_ref(cut(Wg, dim), cut(Qg, dim), cut(Kg, dim), cut(Ug, dim), cut(Mg, 64), cut(Dg, dim), S0)
        o_raw[r0 * hv * dim: r1 * hv * dim] = o.reshape(-1)
        if ln > 0:
            Sb.copy_(S1)


CPU_KERNELS.update({"kern_kda_chunk_prep_k128_v128": _k_kda_chunk_prep, "kern_kda_chunk_rule_k128_v128": _k_kda_chunk_rule})
