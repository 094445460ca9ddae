"""Micro-benchmarks of the hand-written ops with roofline fractions.

    python -m kern_b200.ops.bench_ops gemm --m 4096 --n 4096 --k 4096 [--epilogue store] [--bn 256]
    python -m kern_b200.ops.bench_ops attn_decode --seqs 256 --ctx 2432 [--hq 32 --hk 8 --d 128 --page 64]
    python -m kern_b200.ops.bench_ops attn_prefill --seqs 4 --rows 2048 --prefix 0
    python -m kern_b200.ops.bench_ops norm --rows 4096 --n 4096

Timing: CUDA events on the launching stream, warm-up first, a buffer larger than L2 written between
timed iterations, synchronize on both sides. The roofline denominators are the measured copy bandwidth
and bf16 GEMM throughput of this machine's GPUs when ``MEASURED_PEAKS.json`` is present at the repository
root ("of measured"), otherwise 6.65 TB/s and 1.59 PFLOP/s ("of fallback").
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch


def peaks():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "of measured"
    return 6.65e12, 1.59e15, "of fallback"


_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush.fill_(1)


def timeit(fn, iters=10, warmup=3, flush=True):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            flush_l2()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2], ts[0]


def report(name, ms, flops=0.0, nbytes=0.0, **extra):
    bw, fl, tag = peaks()
    out = {"op": name, "ms_p50": round(ms[0], 4), "ms_min": round(ms[1], 4), **extra}
    if flops:
        out["tflops"] = round(flops / ms[0] / 1e9, 1)
        out["frac_of_gemm_peak"] = f"{flops / (ms[0] * 1e-3) / fl:.3f} {tag}"
    if nbytes:
        out["gbs"] = round(nbytes / ms[0] / 1e6, 1)
        out["frac_of_copy_bw"] = f"{nbytes / (ms[0] * 1e-3) / bw:.3f} {tag}"
    print(json.dumps(out))
    return out


def bench_gemm(a):
    from .gemm import gemm
    from .launcher import Kernels

    x = (torch.randn(a.m, a.k, device="cuda")).to(torch.bfloat16)
    w = (torch.randn(a.n, a.k, device="cuda") * 0.1).to(torch.bfloat16)
    cols = a.n // 2 if a.epilogue == "swiglu" else a.n
    out = torch.zeros(a.m, cols, device="cuda", dtype=torch.float32 if a.epilogue == "f32" else torch.bfloat16)
    ms = timeit(lambda: gemm(x, w, out=out, epilogue=a.epilogue, bn=a.bn, bm=a.bm), a.iters)
    Kernels.get().check_error()
    nbytes = 2 * (a.m * a.k + a.n * a.k) + out.numel() * out.element_size()
    report("gemm_bf16_tn", ms, flops=2.0 * a.m * a.n * a.k, nbytes=nbytes, m=a.m, n=a.n, k=a.k, epilogue=a.epilogue, bn=a.bn, bm=a.bm)
    if a.compare:
        y = torch.empty(a.m, a.n, device="cuda", dtype=torch.bfloat16)
        ms2 = timeit(lambda: torch.matmul(x, w.t(), out=y), a.iters)
        report("torch.matmul (cuBLAS, comparison only)", ms2, flops=2.0 * a.m * a.n * a.k)


def bench_gemm_fp8(a):
    from . import gemm_fp8 as F8
    from .launcher import Kernels

    x = (torch.randn(a.m, a.k, device="cuda")).to(torch.bfloat16)
    w = (torch.randn(a.n, a.k, device="cuda") * 0.1).to(torch.bfloat16)
    xq, sx = F8.quantize(x)
    wq, sw = F8.quantize(w)
    out = torch.zeros(a.m, a.n, device="cuda", dtype=torch.bfloat16)
    ms = timeit(lambda: F8.gemm_fp8(xq, wq, sx, sw, out=out, bn=a.bn), a.iters)
    Kernels.get().check_error()
    report("gemm_e4m3_tn", ms, flops=2.0 * a.m * a.n * a.k, nbytes=a.m * a.k + a.n * a.k + out.numel() * 2, m=a.m, n=a.n, k=a.k, bn=a.bn)


def bench_moe(a):
    """One MoE layer's routed part (plan, gather, two routed GEMMs, combine) at a decode- or prefill-sized batch."""
    from . import moe as M
    from .launcher import Kernels

    x = torch.randn(a.tokens, a.hidden, device="cuda").to(torch.bfloat16)
    wr = (torch.randn(a.experts, a.hidden, device="cuda") * 0.1).to(torch.bfloat16)
    w1 = (torch.randn(a.experts, 2 * a.inter, a.hidden, device="cuda") * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(a.experts, a.hidden, a.inter, device="cuda") * 0.02).to(torch.bfloat16)
    ms = timeit(lambda: M.moe_layer(x, wr, w1, w2, a.top_k), a.iters)
    Kernels.get().check_error()
    flops = 2.0 * a.tokens * a.top_k * 3 * a.hidden * a.inter
    touched = min(a.experts, a.tokens * a.top_k)
    report("moe_layer_bf16", ms, flops=flops, nbytes=touched * 3 * a.hidden * a.inter * 2.0, tokens=a.tokens, experts=a.experts,
           top_k=a.top_k, hidden=a.hidden, inter=a.inter)


def bench_gemm_mx(a):
    """Block-scaled GEMM (MXFP8 x MXFP8 or MXFP8 x MXFP4) on random codes and scales near 1."""
    from . import gemm_mx as G
    from .launcher import Kernels

    aq = torch.randint(0, 256, (a.m, a.k), device="cuda", dtype=torch.uint8) & 0x77        # finite e4m3 codes of small magnitude
    wq = torch.randint(0, 256, (a.n, a.k // 2 if a.fp4 else a.k), device="cuda", dtype=torch.uint8)
    if not a.fp4:
        wq &= 0x77
    sfa = torch.randint(125, 130, (G.atom_bytes(a.m, a.k),), device="cuda", dtype=torch.uint8)
    sfw = torch.randint(125, 130, (G.atom_bytes(a.n, a.k),), device="cuda", dtype=torch.uint8)
    out = torch.zeros(a.m, a.n, device="cuda", dtype=torch.bfloat16)
    ms = timeit(lambda: G.gemm_mx(aq, sfa, wq, sfw, a.fp4, out=out, bn=a.bn or 256), a.iters)
    Kernels.get().check_error()
    report("gemm_mxfp8_mxfp4_tn" if a.fp4 else "gemm_mxfp8_tn", ms, flops=2.0 * a.m * a.n * a.k,
           nbytes=aq.numel() + wq.numel() + out.numel() * 2, m=a.m, n=a.n, k=a.k, bn=a.bn or 256)


def bench_moe_mx(a):
    """The two routed expert GEMMs with MXFP4 weights and MXFP8 activations over a planned batch: `tokens` tokens choose
    `top_k` of `experts_total` experts uniformly, this rank holds the first `experts` of them (expert parallel); FC1 with the
    SwiGLU + MXFP8 epilogue, FC2 to bf16. Random codes: the time does not depend on the values."""
    from . import gemm_mx as G
    from . import moe as M
    from .launcher import Kernels

    dev = "cuda"
    ids = torch.stack([torch.randperm(a.experts_total, device=dev)[:a.top_k] for _ in range(a.tokens)]).int()
    pl = M.plan(ids, a.experts, 0, aligned=True)
    rows = pl["rows_bound"]
    torch.cuda.synchronize()
    live = int(pl["rows"].item())
    xq = torch.randint(0, 256, (rows, a.hidden), device=dev, dtype=torch.uint8) & 0x77
    sfx = torch.randint(125, 130, (G.atom_bytes(rows, a.hidden),), device=dev, dtype=torch.uint8)
    w1 = torch.randint(0, 256, (a.experts, 2 * a.inter, a.hidden // 2), device=dev, dtype=torch.uint8)
    sf1 = torch.randint(125, 130, (a.experts, G.atom_bytes(2 * a.inter, a.hidden)), device=dev, dtype=torch.uint8)
    w2 = torch.randint(0, 256, (a.experts, a.hidden, a.inter // 2), device=dev, dtype=torch.uint8)
    sf2 = torch.randint(125, 130, (a.experts, G.atom_bytes(a.hidden, a.inter)), device=dev, dtype=torch.uint8)
    state = {}

    def fc1():
        state["act"] = M.grouped_gemm_mx(xq, sfx, w1, sf1, pl, swiglu_mxfp8=True, bn=a.bn or 256)

    fc1()
    act_q, sf_act = state["act"]
    ms1 = timeit(fc1, a.iters)
    ms2 = timeit(lambda: M.grouped_gemm_mx(act_q, sf_act, w2, sf2, pl, bn=a.bn or 256), a.iters)
    Kernels.get().check_error()
    real = sum(min(live, live) for _ in range(1))
    report("moe_fc1_mxfp8_mxfp4_swiglu_mxfp8", ms1, flops=2.0 * real * 2 * a.inter * a.hidden,
           nbytes=w1.numel() + real * a.hidden + real * a.inter, rows=real, experts=a.experts, hidden=a.hidden, inter=a.inter)
    report("moe_fc2_mxfp8_mxfp4_bf16", ms2, flops=2.0 * real * a.inter * a.hidden,
           nbytes=w2.numel() + real * a.inter + real * a.hidden * 2, rows=real, experts=a.experts, hidden=a.hidden, inter=a.inter)


def bench_gdn(a):
    """Gated DeltaNet decode step (conv + rule + gated norm) for `seqs` sequences, or a prefill chunk of `rows` rows of one."""
    from . import gdn as G
    from .launcher import Kernels

    hk, hv, d, width = a.hk, a.hv, a.d, 4
    conv_dim = 2 * hk * d + hv * d
    x_stride = conv_dim + hv * d + 2 * hv
    lb, s_off = G.line_bytes(hk, hv, d, d, width)
    seqs, rows = (a.seqs, a.seqs) if a.rows == 1 else (1, a.rows)
    state = torch.zeros(seqs + 1, lb, dtype=torch.uint8, device="cuda")
    lines = torch.arange(1, seqs + 1, dtype=torch.int32, device="cuda")
    cu = None if a.rows == 1 else torch.tensor([0, rows], dtype=torch.int32, device="cuda")
    x = torch.randn(rows, x_stride, device="cuda").to(torch.bfloat16)
    y = torch.empty(rows, conv_dim, dtype=torch.bfloat16, device="cuda")
    out = torch.empty(rows, hv * d, dtype=torch.bfloat16, device="cuda")
    w = (torch.randn(conv_dim, width, device="cuda") * 0.3).to(torch.bfloat16)
    A_log, dtb = torch.zeros(hv, device="cuda"), torch.zeros(hv, device="cuda")
    nw = torch.ones(d, device="cuda").to(torch.bfloat16)
    o_raw = torch.empty(rows, hv * d, dtype=torch.float32, device="cuda")

    scratch = G.chunk_scratch(rows, hv, "cuda", kda=a.kda) if a.rows > 1 and a.chunked else None
    if a.kda:      # the per-key-decay rule: gate rows beside z | b in the projection's row
        A_log, dtb = torch.zeros(hv, device="cuda"), torch.zeros(hv * d, device="cuda")
        gk = torch.randn(rows, hv * d, device="cuda").to(torch.bfloat16)

    def step():
        G.conv(x, y, state, lines, cu, w, None, seqs, conv_dim, width, lb)
        if a.kda and a.rows > 1 and a.chunked:
            G.kda_rule_chunked(y, x[:, conv_dim:], gk, out, state, lines, cu, A_log, dtb, nw, seqs, hk, hv, d, d, 0, hv * d, lb,
                               s_off, o_raw=o_raw, scratch=scratch)
        elif a.kda and a.rows > 1:
            G.kda_rule(y, x[:, conv_dim:], gk, out, state, lines, cu, A_log, dtb, nw, seqs, hk, hv, d, d, 0, hv * d, lb, s_off)
        elif a.kda:
            G.kda_step(y, x[:, conv_dim:], gk, out, state, lines, A_log, dtb, nw, seqs, hk, hv, d, d, 0, hv * d, lb, s_off)
        elif a.rows > 1 and a.chunked:
            G.rule_chunked(y, x[:, conv_dim:], out, state, lines, cu, A_log, dtb, nw, seqs, hk, hv, d, d, 0, hv * d,
                           hv * d + hv, lb, s_off, o_raw=o_raw, scratch=scratch)
        elif a.rows == 1 and not a.unfused:
            G.step(y, x[:, conv_dim:], out, state, lines, A_log, dtb, nw, seqs, hk, hv, d, d, 0, hv * d, hv * d + hv, lb, s_off)
        else:
            G.rule(y, x[:, conv_dim:], out, state, lines, cu, A_log, dtb, nw, seqs, hk, hv, d, d, 0, hv * d, hv * d + hv, lb,
                   s_off, o_raw=o_raw)

    ms = timeit(step, a.iters)
    Kernels.get().check_error()
    nbytes = 2.0 * seqs * hv * d * d * 4 if a.rows == 1 else 0.0      # the recurrent state is read and written once per step
    report(("kda_" if a.kda else "") + ("gdn_step" if a.rows == 1 else ("gdn_prefill_chunked" if a.chunked else "gdn_prefill_chunk")), ms, nbytes=nbytes, seqs=seqs, rows=rows, hk=hk, hv=hv, d=d)


def _cache(seqs, ctx, hk, d, page):
    per = (ctx + page - 1) // page
    pool = torch.randn(seqs * per + 1, 2, hk, page, d, device="cuda").to(torch.bfloat16)
    table = (torch.randperm(seqs * per, device="cuda").to(torch.int32) + 1).view(seqs, per).contiguous()
    return pool, table


def bench_attn_decode(a):
    from .attention import paged_attention
    from .launcher import Kernels

    pool, table = _cache(a.seqs, a.ctx, a.hk, a.d, a.page)
    q = torch.randn(a.seqs * a.rows, a.hq * a.d, device="cuda").to(torch.bfloat16)
    lens = torch.full((a.seqs,), a.ctx, dtype=torch.int32, device="cuda")
    out = torch.empty_like(q)
    ms = timeit(lambda: paged_attention(q, pool, table, lens, a.hq, out=out, rows_per_seq=a.rows, splits=a.splits), a.iters)
    Kernels.get().check_error()
    kv_bytes = a.seqs * a.ctx * 2 * a.hk * a.d * 2
    report("attn_decode_paged", ms, nbytes=kv_bytes + 2 * q.numel() * 2, seqs=a.seqs, ctx=a.ctx, rows=a.rows, splits=a.splits,
           kv_gb=round(kv_bytes / 1e9, 3))


def bench_mla_decode(a):
    """Absorbed latent-attention decode: `seqs` sequences of `ctx` latent rows, `heads` heads on this GPU."""
    from . import mla
    from .launcher import Kernels

    page = a.page
    pages_per = -(-a.ctx // page)
    cache = (torch.randn(a.seqs * pages_per + 1, page, mla.DQK, device="cuda") * 0.3).to(torch.bfloat16)
    table = (torch.arange(a.seqs * pages_per, device="cuda", dtype=torch.int32) + 1).view(a.seqs, pages_per)
    q = (torch.randn(a.seqs, a.heads * mla.DQK, device="cuda") * 0.3).to(torch.bfloat16)
    lens = torch.full((a.seqs,), a.ctx, dtype=torch.int32, device="cuda")
    out = torch.empty(a.seqs, a.heads * mla.DV, dtype=torch.bfloat16, device="cuda")
    ms = timeit(lambda: mla.mla_decode(q, cache, table, lens, a.heads, splits=a.splits, out=out), a.iters)
    Kernels.get().check_error()
    lat_bytes = a.seqs * a.ctx * mla.DQK * 2
    report("mla_decode", ms, nbytes=lat_bytes, flops=2.0 * a.seqs * a.heads * a.ctx * (mla.DQK + mla.DV), seqs=a.seqs, ctx=a.ctx,
           heads=a.heads, splits=a.splits, latent_gb=round(lat_bytes / 1e9, 3))


def bench_attn_prefill(a):
    from .attention import paged_attention
    from .launcher import Kernels

    ctx = a.prefix + a.rows
    pool, table = _cache(a.seqs, ctx, a.hk, a.d, a.page)
    q = torch.randn(a.seqs * a.rows, a.hq * a.d, device="cuda").to(torch.bfloat16)
    lens = torch.full((a.seqs,), ctx, dtype=torch.int32, device="cuda")
    cu = (torch.arange(a.seqs + 1, device="cuda") * a.rows).to(torch.int32)
    out = torch.empty_like(q)
    if a.fmha:
        from .attention import fmha_prefill

        ms = timeit(lambda: fmha_prefill(q, pool, table, lens, a.hq, cu, out=out, tile=a.fmha_tile), a.iters)
    else:
        ms = timeit(lambda: paged_attention(q, pool, table, lens, a.hq, out=out, prefill=True, cu_q=cu, max_rows=a.rows), a.iters)
    Kernels.get().check_error()
    # causal: row r of a chunk sees prefix + r + 1 keys
    keys = a.rows * a.prefix + a.rows * (a.rows + 1) / 2
    report(f"attn_fmha_prefill_tcgen05_t{a.fmha_tile}" if a.fmha else "attn_prefill_paged", ms, flops=4.0 * a.seqs * a.hq * a.d * keys, seqs=a.seqs,
           rows=a.rows, prefix=a.prefix)


def bench_attn_ragged(a):
    """One serving step's attention: a prompt chunk of `rows` rows plus `seqs` decode rows over `ctx` tokens each, as
    one launch (both kernels' CTAs side by side) or as the two launches one after the other (`--two-launches`)."""
    from .attention import ragged_attention
    from .launcher import Kernels

    per = (max(a.ctx, a.rows) + a.page - 1) // a.page
    n = a.seqs + 1
    pool = torch.randn(n * per + 1, 2, a.hk, a.page, a.d, device="cuda").to(torch.bfloat16)
    table = (torch.randperm(n * per, device="cuda").to(torch.int32) + 1).view(n, per).contiguous()
    q = torch.randn(a.rows + a.seqs, a.hq * a.d, device="cuda").to(torch.bfloat16)
    lens = torch.tensor([a.rows] + [a.ctx] * a.seqs, dtype=torch.int32, device="cuda")
    cu = torch.tensor([0] + [a.rows + i for i in range(a.seqs + 1)], dtype=torch.int32, device="cuda")
    out = torch.empty_like(q)
    ms = timeit(lambda: ragged_attention(q, pool, table, lens, a.hq, cu, out=out, one_launch=not a.two_launches, fmha=a.fmha), a.iters)
    Kernels.get().check_error()
    kv_bytes = a.seqs * a.ctx * 2 * a.hk * a.d * 2
    report("attn_ragged_two_launches" if a.two_launches else ("attn_ragged_one_launch_tcgen05" if a.fmha else "attn_ragged_one_launch"), ms, nbytes=kv_bytes,
           flops=4.0 * a.hq * a.d * a.rows * (a.rows + 1) / 2, prompt_rows=a.rows, decode_seqs=a.seqs, ctx=a.ctx)


def bench_attn_context(a):
    """Context attention qk 192 / v 128 over contiguous K / V (un-absorbed latent-attention prefill): `seqs` sequences of
    `rows` new rows each over `prefix` earlier keys, `heads` heads."""
    from .attention import fmha_context
    from .launcher import Kernels

    L = a.prefix + a.rows
    q = torch.randn(a.seqs * a.rows, a.heads * 192, device="cuda").to(torch.bfloat16)
    k = (torch.randn(a.seqs * L, a.heads * 192, device="cuda") * 0.5).to(torch.bfloat16)
    v = (torch.randn(a.seqs * L, a.heads * 128, device="cuda") * 0.5).to(torch.bfloat16)
    cu_q = (torch.arange(a.seqs + 1, device="cuda") * a.rows).to(torch.int32)
    cu_k = (torch.arange(a.seqs + 1, device="cuda") * L).to(torch.int32)
    out = torch.empty(q.shape[0], a.heads * 128, device="cuda", dtype=torch.bfloat16)
    ms = timeit(lambda: fmha_context(q, k, v, cu_q, cu_k, a.heads, out=out, two_per_sm=not a.one_per_sm), a.iters)
    Kernels.get().check_error()
    keys = a.rows * a.prefix + a.rows * (a.rows + 1) / 2
    report("attn_fmha_ctx_qk192_v128" + ("" if a.one_per_sm else "_x2"), ms, flops=2.0 * a.seqs * a.heads * (192 + 128) * keys,
           seqs=a.seqs, rows=a.rows, prefix=a.prefix, heads=a.heads)


def bench_norm(a):
    from .basic import rms_norm

    x = torch.randn(a.rows, a.n, device="cuda").to(torch.bfloat16)
    w = torch.randn(a.n, device="cuda").to(torch.bfloat16)
    y = torch.empty_like(x)
    ms = timeit(lambda: rms_norm(x, w, out=y), a.iters)
    report("rms_norm", ms, nbytes=2 * x.numel() * 2, rows=a.rows, n=a.n)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="op", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=4096); g.add_argument("--n", type=int, default=4096); g.add_argument("--k", type=int, default=4096)
    g.add_argument("--epilogue", default="store"); g.add_argument("--bn", type=int, default=None); g.add_argument("--compare", action="store_true")
    g.add_argument("--bm", type=int, default=None, help="128 or 256 rows per tile (default: chosen by shape)")
    g8 = sub.add_parser("gemm_fp8")
    g8.add_argument("--m", type=int, default=4096); g8.add_argument("--n", type=int, default=4096); g8.add_argument("--k", type=int, default=4096)
    g8.add_argument("--bn", type=int, default=None)
    gx = sub.add_parser("gemm_mx")
    gx.add_argument("--m", type=int, default=4096); gx.add_argument("--n", type=int, default=4096); gx.add_argument("--k", type=int, default=4096)
    gx.add_argument("--bn", type=int, default=None); gx.add_argument("--fp4", action="store_true", help="MXFP4 weights (packed e2m1)")
    mx = sub.add_parser("moe_mx")
    mx.add_argument("--tokens", type=int, default=16384); mx.add_argument("--experts-total", type=int, default=384)
    mx.add_argument("--experts", type=int, default=96, help="experts held by this rank"); mx.add_argument("--top-k", type=int, default=8)
    mx.add_argument("--hidden", type=int, default=7168); mx.add_argument("--inter", type=int, default=2048); mx.add_argument("--bn", type=int, default=None)
    mo = sub.add_parser("moe")
    mo.add_argument("--tokens", type=int, default=2048); mo.add_argument("--experts", type=int, default=128); mo.add_argument("--top-k", type=int, default=8)
    mo.add_argument("--hidden", type=int, default=2048); mo.add_argument("--inter", type=int, default=768)
    gd = sub.add_parser("gdn")
    gd.add_argument("--seqs", type=int, default=64); gd.add_argument("--rows", type=int, default=1)
    gd.add_argument("--hk", type=int, default=16); gd.add_argument("--hv", type=int, default=48); gd.add_argument("--d", type=int, default=128)
    gd.add_argument("--kda", action="store_true", help="a decay per key channel (Kimi Delta Attention)")
    gd.add_argument("--chunked", action="store_true", help="prefill rows through the chunked (WY) kernels")
    gd.add_argument("--unfused", action="store_true", help="decode rows through the two-launch rule + norm instead of the fused step")
    d = sub.add_parser("attn_decode")
    p = sub.add_parser("attn_prefill")
    for s in (d, p):
        s.add_argument("--seqs", type=int, default=64); s.add_argument("--hq", type=int, default=32); s.add_argument("--hk", type=int, default=8)
        s.add_argument("--d", type=int, default=128); s.add_argument("--page", type=int, default=64); s.add_argument("--rows", type=int, default=1)
    d.add_argument("--ctx", type=int, default=2432); d.add_argument("--splits", type=int, default=None)
    p.add_argument("--prefix", type=int, default=0)
    p.add_argument("--fmha", action="store_true", help="the tcgen05 kernel (head_dim 128) instead of the mma.sync one")
    p.add_argument("--fmha-tile", type=int, default=64, choices=[64, 128], help="tokens per KV tile of the tcgen05 kernel")
    rg = sub.add_parser("attn_ragged")
    rg.add_argument("--seqs", type=int, default=256); rg.add_argument("--hq", type=int, default=32); rg.add_argument("--hk", type=int, default=8)
    rg.add_argument("--d", type=int, default=128); rg.add_argument("--page", type=int, default=64); rg.add_argument("--rows", type=int, default=2304)
    rg.add_argument("--ctx", type=int, default=2432); rg.add_argument("--two-launches", action="store_true")
    rg.add_argument("--fmha", action="store_true", help="the prompt rows' CTAs on the tcgen05 kernel (head_dim 128)")
    cx = sub.add_parser("attn_context")
    cx.add_argument("--seqs", type=int, default=2); cx.add_argument("--rows", type=int, default=4096); cx.add_argument("--prefix", type=int, default=0)
    cx.add_argument("--heads", type=int, default=16); cx.add_argument("--one-per-sm", action="store_true", help="the two-stage form, one CTA per SM")
    ml = sub.add_parser("mla_decode")
    ml.add_argument("--seqs", type=int, default=64); ml.add_argument("--ctx", type=int, default=8192)
    ml.add_argument("--heads", type=int, default=16); ml.add_argument("--page", type=int, default=64)
    ml.add_argument("--splits", type=int, default=None)
    n = sub.add_parser("norm")
    n.add_argument("--rows", type=int, default=4096); n.add_argument("--n", type=int, default=4096)
    for s in (g, d, p, n, g8, mo, gd, ml, gx, mx, rg, cx):
        s.add_argument("--iters", type=int, default=10)
    a = ap.parse_args(argv)
    {"gemm": bench_gemm, "gemm_mx": bench_gemm_mx, "moe_mx": bench_moe_mx, "gdn": bench_gdn, "gemm_fp8": bench_gemm_fp8, "moe": bench_moe, "attn_decode": bench_attn_decode, "mla_decode": bench_mla_decode, "attn_prefill": bench_attn_prefill, "attn_ragged": bench_attn_ragged, "attn_context": bench_attn_context, "norm": bench_norm}[a.op](a)


if __name__ == "__main__":
    main()
