"""Gated DeltaNet: wrappers for the causal conv and the gated delta rule kernels, and their PyTorch
fp32 statement (the oracle the GPU tests and the CPU executor use).

State line of one sequence for one layer: ``[(width-1) x conv_dim bf16 | HV x DV x DK f32]``; line 0 is null.
Reference counterpart of the decode step: tools/kernels-src/gdn_decode.cu:90, :171.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .launcher import Kernels, f32, i32, i64, ptr

NULL = 0


def line_bytes(hk: int, hv: int, dk: int, dv: int, width: int = 4) -> tuple[int, int]:
    """(bytes of one state line, byte offset of S inside it); S starts 256-byte aligned."""
    conv = (width - 1) * (2 * hk * dk + hv * dv) * 2
    s_off = (conv + 255) // 256 * 256
    return s_off + hv * dv * dk * 4, s_off


def rule_rows(dv: int, decode: bool) -> int:
    """Value rows per CTA (64 per CTA measured slower for prefill chunks: too few CTAs for 148 SMs)."""
    return 16


def rule_smem(dk: int, tb: int, rows: int = 16) -> int:
    return tb * (2 * dk + rows + 4) * 4


def conv(x, y, state, lines, cu_q, w, bias, seqs, conv_dim, width, line_b, rows=None):
    """Causal conv + SiLU over the rows of the call (row-parallel), then the state windows advance."""
    k = Kernels.get(x.device)
    rows = x.shape[0] if rows is None else rows
    assert conv_dim % 4 == 0 and x.stride(0) % 4 == 0, "the conv kernel moves four channels (8 bytes) per thread"
    if cu_q is None:      # one row per sequence: conv and window shift in one launch
        k.launch("gdn", "kern_gdn_conv_step_bf16", (seqs, (conv_dim + 1023) // 1024), (256,),
                 [ptr(x), ptr(y), ptr(state), ptr(lines), ptr(w), ptr(bias), i32(seqs), i32(conv_dim), i32(width),
                  i32(x.stride(0)), i64(line_b)])
        return y
    rpc = 16
    k.launch("gdn", "kern_gdn_conv_bf16", ((rows + rpc - 1) // rpc, (conv_dim + 1023) // 1024), (256,),
             [ptr(x), ptr(y), ptr(state), ptr(lines), ptr(cu_q), ptr(w), ptr(bias), i32(seqs), i32(rows), i32(conv_dim),
              i32(width), i32(x.stride(0)), i64(line_b), i32(rpc)])
    k.launch("gdn", "kern_gdn_conv_state", (seqs, (conv_dim + 255) // 256), (256,),
             [ptr(x), ptr(state), ptr(lines), ptr(cu_q), i32(seqs), i32(conv_dim), i32(width), i32(x.stride(0)), i64(line_b)])
    return y


def rule(qkv, zba, out, state, lines, cu_q, A_log, dt_bias, norm_w, seqs, hk, hv, dk, dv, z_off, b_off, a_off,
         line_b, s_off, eps=1e-6, o_raw=None):
    """Gated delta rule (value rows split over CTAs, state in registers) then the gated RMSNorm."""
    k = Kernels.get(qkv.device)
    assert dk == dv and dk in (32, 64, 128)
    tokens = out.shape[0]
    if o_raw is None:
        o_raw = torch.empty(tokens, hv * dv, dtype=torch.float32, device=qkv.device)
    tb = 1 if cu_q is None else 32          # tokens staged per pass: a decode row needs one
    rows_cta = rule_rows(dv, cu_q is None)
    k.launch("gdn", f"kern_gdn_rule_{'dec_' if cu_q is None else ''}k{dk}_v{dv}", (hv * (dv // rows_cta), seqs), (256,),
             [ptr(qkv), ptr(zba), ptr(o_raw), ptr(state), ptr(lines), ptr(cu_q), ptr(A_log), ptr(dt_bias),
              i32(seqs), i32(hk), i32(hv), i32(zba.stride(0)), i32(b_off), i32(a_off), i64(line_b), i64(s_off), i32(tb)],
             shared_mem=rule_smem(dk, tb, rows_cta))
    k.launch("gdn", "kern_gdn_gate_norm_bf16", ((hv + 3) // 4, tokens), (128,),
             [ptr(o_raw), ptr(zba), ptr(out), ptr(norm_w), i32(tokens), i32(hv), i32(dv), i32(zba.stride(0)),
              i32(z_off), f32(eps)])
    return out


def step_smem(dk: int, dv: int) -> int:
    return dv * dk * 4 + (2 * dk + 2 * dv + 16) * 4 + 16


def step(qkv, zba, out, state, lines, A_log, dt_bias, norm_w, seqs, hk, hv, dk, dv, z_off, b_off, a_off, line_b, s_off,
         eps=1e-6):
    """Fused decode step (one row per sequence): the head's state by bulk copy into shared memory, the rule, the new
    state straight to global memory, and the gated RMSNorm, in one launch of [HV, seqs] CTAs."""
    k = Kernels.get(qkv.device)
    assert dk == dv and dk in (32, 64, 128)
    k.launch("gdn", f"kern_gdn_step_k{dk}_v{dv}", (hv, seqs), (256,),
             [ptr(qkv), ptr(zba), ptr(out), ptr(state), ptr(lines), ptr(A_log), ptr(dt_bias), ptr(norm_w), i32(seqs),
              i32(hk), i32(hv), i32(zba.stride(0)), i32(z_off), i32(b_off), i32(a_off), i64(line_b), i64(s_off), f32(eps)],
             shared_mem=step_smem(dk, dv))
    return out


def kda_step(qkv, zba, gk, out, state, lines, A_log, dt_bias, norm_w, seqs, hk, hv, dk, dv, z_off, b_off, line_b, s_off,
             eps=1e-6):
    """Fused decode step with a decay per key channel (Kimi Delta Attention): `gk` [tokens, HV * DK] bf16 gate rows,
    `dt_bias` [HV * DK]; everything else as `step`."""
    k = Kernels.get(qkv.device)
    assert dk == dv and dk in (64, 128)
    k.launch("gdn", f"kern_kda_step_k{dk}_v{dv}", (hv, seqs), (256,),
             [ptr(qkv), ptr(zba), ptr(out), ptr(state), ptr(lines), ptr(A_log), ptr(dt_bias), ptr(norm_w), ptr(gk), i32(seqs),
              i32(hk), i32(hv), i32(zba.stride(0)), i32(z_off), i32(b_off), i32(gk.stride(0)), i64(line_b), i64(s_off), f32(eps)],
             shared_mem=step_smem(dk, dv) + dk * 4)
    return out


def kda_rule(qkv, zba, gk, out, state, lines, cu_q, A_log, dt_bias, norm_w, seqs, hk, hv, dk, dv, z_off, b_off, line_b, s_off,
             eps=1e-6):
    """Ragged rows (prefill chunks, speculative rows) of the per-key-decay rule, token by token with the state in
    registers, then the gated RMSNorm."""
    k = Kernels.get(qkv.device)
    assert dk == dv and dk in (64, 128) and cu_q is not None
    tokens = out.shape[0]
    o_raw = torch.empty(tokens, hv * dv, dtype=torch.float32, device=qkv.device)
    tb = 32
    k.launch("gdn", f"kern_kda_rule_k{dk}_v{dv}", (hv * (dv // 16), seqs), (256,),
             [ptr(qkv), ptr(zba), ptr(o_raw), ptr(state), ptr(lines), ptr(cu_q), ptr(A_log), ptr(dt_bias), ptr(gk), i32(seqs),
              i32(hk), i32(hv), i32(zba.stride(0)), i32(b_off), i32(gk.stride(0)), i64(line_b), i64(s_off), i32(tb)],
             shared_mem=tb * (3 * dk + 16 + 4) * 4)
    k.launch("gdn", "kern_gdn_gate_norm_bf16", ((hv + 3) // 4, tokens), (128,),
             [ptr(o_raw), ptr(zba), ptr(out), ptr(norm_w), i32(tokens), i32(hv), i32(dv), i32(zba.stride(0)),
              i32(z_off), f32(eps)])
    return out


CHUNK_PREP_SMEM = (2 * 64 * 132 + 64 * 68 + 2 * 64) * 4
CHUNK_RULE_SMEM = (64 * 132 * 3 + 64 * 136 + 64 * 68 + 2 * 64 * 72) * 4


def chunk_scratch(tokens: int, hv: int, device, kda: bool = False) -> dict:
    """Scratch of the chunked rule: W, Qg, Kd, Ut [tokens, HV, 128], M [tokens, HV, 64], gC [tokens, HV], all f32
    (`kda`: gC is [tokens, HV, 128], the decay of every key over a chunk at the chunk's first token)."""
    big = lambda: torch.empty(tokens, hv, 128, dtype=torch.float32, device=device)
    return {"W": big(), "Qg": big(), "Kd": big(), "Ut": big(),
            "M": torch.empty(tokens, hv, 64, dtype=torch.float32, device=device),
            "gC": big() if kda else torch.empty(tokens, hv, dtype=torch.float32, device=device)}


def rule_chunked(qkv, zba, out, state, lines, cu_q, A_log, dt_bias, norm_w, seqs, hk, hv, dk, dv, z_off, b_off, a_off,
                 line_b, s_off, eps=1e-6, o_raw=None, scratch=None):
    """Prefill rows through the chunked (WY) form: a parallel launch over (64-token chunk, head) prepares the
    state-independent factors on the tensor cores, a second launch walks the chunks with the state on chip, then the
    gated RMSNorm. dk = dv = 128 only."""
    k = Kernels.get(qkv.device)
    assert dk == dv == 128 and cu_q is not None
    tokens = out.shape[0]
    if o_raw is None:
        o_raw = torch.empty(tokens, hv * dv, dtype=torch.float32, device=qkv.device)
    sc = scratch if scratch is not None else chunk_scratch(tokens, hv, qkv.device)
    k.launch("gdn_chunk", "kern_gdn_chunk_prep_k128_v128", ((tokens + 63) // 64 + seqs, hv), (256,),
             [ptr(qkv), ptr(zba), ptr(cu_q), ptr(A_log), ptr(dt_bias), ptr(sc["W"]), ptr(sc["Qg"]), ptr(sc["Kd"]),
              ptr(sc["Ut"]), ptr(sc["M"]), ptr(sc["gC"]), i32(seqs), i32(hk), i32(hv), i32(zba.stride(0)), i32(b_off),
              i32(a_off)], shared_mem=CHUNK_PREP_SMEM)
    k.launch("gdn_chunk", "kern_gdn_chunk_rule_k128_v128", (hv * 2, seqs), (256,),
             [ptr(sc["W"]), ptr(sc["Qg"]), ptr(sc["Kd"]), ptr(sc["Ut"]), ptr(sc["M"]), ptr(sc["gC"]), ptr(o_raw), ptr(state),
              ptr(lines), ptr(cu_q), i32(seqs), i32(hv), i64(line_b), i64(s_off)], shared_mem=CHUNK_RULE_SMEM)
    k.launch("gdn", "kern_gdn_gate_norm_bf16", ((hv + 3) // 4, tokens), (128,),
             [ptr(o_raw), ptr(zba), ptr(out), ptr(norm_w), i32(tokens), i32(hv), i32(dv), i32(zba.stride(0)),
              i32(z_off), f32(eps)])
    return out


KDA_CHUNK_PREP_SMEM = (3 * 64 * 132 + 64 + 3 * 128) * 4


def kda_rule_chunked(qkv, zba, gk, out, state, lines, cu_q, A_log, dt_bias, norm_w, seqs, hk, hv, dk, dv, z_off, b_off, line_b,
                     s_off, eps=1e-6, o_raw=None, scratch=None):
    """Prefill rows of the per-key-decay rule through the chunked (WY) form: the pairwise sums of a chunk carry a
    weight per (i, j, key) and run on the CUDA cores with every exponent <= 0, the triangular solve and the products
    with the state on the tensor cores; `scratch["gC"]` is [tokens, HV, 128] here (a decay per key). dk = dv = 128."""
    k = Kernels.get(qkv.device)
    assert dk == dv == 128 and cu_q is not None and gk.stride(0) % 8 == 0 and gk.data_ptr() % 16 == 0
    tokens = out.shape[0]
    if o_raw is None:
        o_raw = torch.empty(tokens, hv * dv, dtype=torch.float32, device=qkv.device)
    sc = scratch if scratch is not None else chunk_scratch(tokens, hv, qkv.device, kda=True)
    k.launch("gdn_chunk", "kern_kda_chunk_prep_k128_v128", ((tokens + 63) // 64 + seqs, hv), (256,),
             [ptr(qkv), ptr(zba), ptr(gk), ptr(cu_q), ptr(A_log), ptr(dt_bias), ptr(sc["W"]), ptr(sc["Qg"]), ptr(sc["Kd"]),
              ptr(sc["Ut"]), ptr(sc["M"]), ptr(sc["gC"]), i32(seqs), i32(hk), i32(hv), i32(zba.stride(0)), i32(b_off),
              i32(gk.stride(0))], shared_mem=KDA_CHUNK_PREP_SMEM)
    k.launch("gdn_chunk", "kern_kda_chunk_rule_k128_v128", (hv * 2, seqs), (256,),
             [ptr(sc["W"]), ptr(sc["Qg"]), ptr(sc["Kd"]), ptr(sc["Ut"]), ptr(sc["M"]), ptr(sc["gC"]), ptr(o_raw), ptr(state),
              ptr(lines), ptr(cu_q), i32(seqs), i32(hv), i64(line_b), i64(s_off)], shared_mem=CHUNK_RULE_SMEM)
    k.launch("gdn", "kern_gdn_gate_norm_bf16", ((hv + 3) // 4, tokens), (128,),
             [ptr(o_raw), ptr(zba), ptr(out), ptr(norm_w), i32(tokens), i32(hv), i32(dv), i32(zba.stride(0)),
              i32(z_off), f32(eps)])
    return out


# ---- fp32 statement ------------------------------------------------------------------------------------
def conv_ref(x, window, w, bias=None):
    """x: [T, C] f32 rows of one sequence, window: [width-1, C] (history, oldest first), w: [C, width].
    Returns (silu(conv) [T, C], new window)."""
    width = w.shape[1]
    full = torch.cat([window.float(), x.float()], 0)                      # [T + width - 1, C]
    y = sum(full[j:j + x.shape[0]] * w[:, j].float() for j in range(width))
    if bias is not None:
        y = y + bias.float()
    return F.silu(y), full[full.shape[0] - (width - 1):].clone()


def rule_ref(q, k, v, z, b, a, S, A_log, dt_bias, norm_w, eps=1e-6, normalize=True):
    """One sequence: q,k [T, HK, DK]; v,z [T, HV, DV]; b,a [T, HV]; S [HV, DV, DK] f32 (updated copy returned)."""
    T, hk, dk = q.shape
    hv, dv = v.shape[1], v.shape[2]
    rep = hv // hk
    q = q.float() * torch.rsqrt(q.float().pow(2).sum(-1, keepdim=True) + 1e-6)
    k = k.float() * torch.rsqrt(k.float().pow(2).sum(-1, keepdim=True) + 1e-6)
    q = (q / dk ** 0.5).repeat_interleave(rep, 1)
    k = k.repeat_interleave(rep, 1)
    g = -torch.exp(A_log.float()) * F.softplus(a.float() + dt_bias.float())          # [T, HV]
    beta = torch.sigmoid(b.float()).to(torch.bfloat16).float()
    S = S.float().clone()
    out = torch.empty(T, hv, dv, dtype=torch.float32, device=q.device)
    for t in range(T):
        S = S * torch.exp(g[t])[:, None, None]
        sk = torch.einsum("hvk,hk->hv", S, k[t])
        u = (v[t].float() - sk) * beta[t][:, None]
        S = S + u[:, :, None] * k[t][:, None, :]
        out[t] = torch.einsum("hvk,hk->hv", S, q[t])
    if not normalize:
        return out, S
    return gate_norm_ref(out, z, norm_w, eps), S


def gate_norm_ref(o, z, norm_w, eps=1e-6):
    o = o.float()
    return o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps) * norm_w.float() * F.silu(z.float())


# ---- chunked (WY) form of the rule: the statement of the two prefill kernels --------------------------------
CHUNK = 64


def chunk_prep_ref(q, k, v, b, a, A_log, dt_bias):
    """Per chunk of 64 tokens of one sequence, everything that does not depend on the carried state.
    q,k [T, HK, D]; v [T, HV, D]; b,a [T, HV]. Returns W, Qg, Kd, Ut [T, HV, D], M [T, HV, 64], gC [T, HV]:
      g   = inclusive cumulative log decay inside the chunk
      L   = beta_i exp(g_i - g_j) (k_i.k_j) for j < i;   T = (I + L)^-1
      W   = T (beta exp(g) K);  Ut = T (beta V);  Qg = exp(g) q;  Kd = exp(g_last - g) k
      M   = exp(g_i - g_j) (q_i.k_j) for j <= i;  gC = exp(g_last)
    so that with the chunk's incoming state S0:  U = Ut - W S0^T,  O = Qg S0^T + M U,  S1 = gC S0 + U^T Kd."""
    T_, hk, d = q.shape
    hv = v.shape[1]
    rep = hv // hk
    qn = q.float() * torch.rsqrt(q.float().pow(2).sum(-1, keepdim=True) + 1e-6) / d ** 0.5
    kn = k.float() * torch.rsqrt(k.float().pow(2).sum(-1, keepdim=True) + 1e-6)
    qn, kn = qn.repeat_interleave(rep, 1), kn.repeat_interleave(rep, 1)          # [T, HV, D]
    ga = -torch.exp(A_log.float()) * F.softplus(a.float() + dt_bias.float())     # [T, HV] log decay
    beta = torch.sigmoid(b.float()).to(torch.bfloat16).float()
    W, Qg, Kd, Ut = (torch.zeros(T_, hv, d, device=q.device) for _ in range(4))
    M = torch.zeros(T_, hv, CHUNK, device=q.device)
    gC = torch.zeros(T_, hv, device=q.device)
    for c0 in range(0, T_, CHUNK):
        n = min(CHUNK, T_ - c0)
        sl = slice(c0, c0 + n)
        g = ga[sl].cumsum(0)                                                      # [n, HV]
        kk = torch.einsum("ihd,jhd->hij", kn[sl], kn[sl])
        qk = torch.einsum("ihd,jhd->hij", qn[sl], kn[sl])
        e = torch.exp((g.t()[:, :, None] - g.t()[:, None, :]).clamp(max=0.0))     # [HV, i, j]; only j <= i is used
        low = torch.tril(torch.ones(n, n, device=q.device), -1)
        L = beta[sl].t()[:, :, None] * e * kk * low
        Tm = torch.linalg.inv(torch.eye(n, device=q.device) + L)                  # unit lower triangular
        W[sl] = torch.einsum("hij,jhd->ihd", Tm, (beta[sl] * torch.exp(g))[:, :, None] * kn[sl])
        Ut[sl] = torch.einsum("hij,jhd->ihd", Tm, beta[sl][:, :, None] * v[sl].float())
        Qg[sl] = torch.exp(g)[:, :, None] * qn[sl]
        Kd[sl] = torch.exp(g[-1][None] - g)[:, :, None] * kn[sl]
        M[sl, :, :n] = (e * qk * torch.tril(torch.ones(n, n, device=q.device))).permute(1, 0, 2)
        gC[sl] = torch.exp(g[-1])[None]
    return W, Qg, Kd, Ut, M, gC


def chunk_rule_ref(W, Qg, Kd, Ut, M, gC, S):
    """The state-dependent half: one pass over the chunks of one sequence. S [HV, DV, DK] f32. Returns (o [T, HV, DV], S)."""
    T_, hv, d = W.shape
    S = S.float().clone()
    out = torch.empty(T_, hv, d, dtype=torch.float32, device=W.device)
    for c0 in range(0, T_, CHUNK):
        n = min(CHUNK, T_ - c0)
        sl = slice(c0, c0 + n)
        U = Ut[sl] - torch.einsum("ihk,hvk->ihv", W[sl], S)
        out[sl] = torch.einsum("ihk,hvk->ihv", Qg[sl], S) + torch.einsum("ihj,jhv->ihv", M[sl, :, :n], U)
        dec = gC[c0][:, None, None] if gC.dim() == 2 else gC[c0][:, None, :]      # a scalar per head, or a vector over keys
        S = dec * S + torch.einsum("ihv,ihk->hvk", U, Kd[sl])
    return out, S


def kda_rule_ref(q, k, v, z, b, gk, S, A_log, dt_bias, norm_w, eps=1e-6):
    """The delta rule with a decay per key channel, one sequence: gk [T, HV, DK] gate rows, dt_bias [HV, DK];
    S[h, v, k] <- dec[h, k] S[h, v, k], then the delta update and the read-out as in `rule_ref`."""
    T, hk, dk = q.shape
    hv = v.shape[1]
    rep = hv // hk
    q = q.float() * torch.rsqrt(q.float().pow(2).sum(-1, keepdim=True) + 1e-6)
    k = k.float() * torch.rsqrt(k.float().pow(2).sum(-1, keepdim=True) + 1e-6)
    q = (q / dk ** 0.5).repeat_interleave(rep, 1)
    k = k.repeat_interleave(rep, 1)
    dec = torch.exp(-torch.exp(A_log.float())[None, :, None] * F.softplus(gk.float() + dt_bias.float()[None]))      # [T, HV, DK]
    beta = torch.sigmoid(b.float()).to(torch.bfloat16).float()
    S = S.float().clone()
    out = torch.empty(T, hv, v.shape[2], dtype=torch.float32, device=q.device)
    for t in range(T):
        S = S * dec[t][:, None, :]
        u = (v[t].float() - torch.einsum("hvk,hk->hv", S, k[t])) * beta[t][:, None]
        S = S + u[:, :, None] * k[t][:, None, :]
        out[t] = torch.einsum("hvk,hk->hv", S, q[t])
    return gate_norm_ref(out, z, norm_w, eps), S


def kda_chunk_prep_ref(q, k, v, b, gk, A_log, dt_bias):
    """`chunk_prep_ref` with a decay per key: gk [T, HV, D] gate rows, dt_bias [HV, D]; G the inclusive running sum of
    the log decay per key inside the chunk, and the pairwise weights exp(G_i - G_j) sit inside the sums over keys.
    Returns W, Qg, Kd, Ut [T, HV, D], M [T, HV, 64], D [T, HV, D] (exp(G_last) on every row of the chunk)."""
    T_, hk, d = q.shape
    hv = v.shape[1]
    rep = hv // hk
    qn = q.float() * torch.rsqrt(q.float().pow(2).sum(-1, keepdim=True) + 1e-6) / d ** 0.5
    kn = k.float() * torch.rsqrt(k.float().pow(2).sum(-1, keepdim=True) + 1e-6)
    qn, kn = qn.repeat_interleave(rep, 1), kn.repeat_interleave(rep, 1)          # [T, HV, D]
    ga = -torch.exp(A_log.float())[None, :, None] * F.softplus(gk.float() + dt_bias.float()[None])      # [T, HV, D]
    beta = torch.sigmoid(b.float()).to(torch.bfloat16).float()
    W, Qg, Kd, Ut, Dv = (torch.zeros(T_, hv, d, device=q.device) for _ in range(5))
    M = torch.zeros(T_, hv, CHUNK, device=q.device)
    for c0 in range(0, T_, CHUNK):
        n = min(CHUNK, T_ - c0)
        sl = slice(c0, c0 + n)
        G = ga[sl].cumsum(0)                                                       # [n, HV, D]
        e = torch.exp((G[:, None] - G[None, :]).clamp(max=0.0))                    # [i, j, HV, D]
        kk = torch.einsum("ihd,jhd,ijhd->hij", kn[sl], kn[sl], e)
        qk = torch.einsum("ihd,jhd,ijhd->hij", qn[sl], kn[sl], e)
        L = beta[sl].t()[:, :, None] * kk * torch.tril(torch.ones(n, n, device=q.device), -1)
        Tm = torch.linalg.inv(torch.eye(n, device=q.device) + L)
        W[sl] = torch.einsum("hij,jhd->ihd", Tm, beta[sl][:, :, None] * torch.exp(G) * kn[sl])
        Ut[sl] = torch.einsum("hij,jhd->ihd", Tm, beta[sl][:, :, None] * v[sl].float())
        Qg[sl] = torch.exp(G) * qn[sl]
        Kd[sl] = torch.exp(G[-1][None] - G) * kn[sl]
        M[sl, :, :n] = (qk * torch.tril(torch.ones(n, n, device=q.device))).permute(1, 0, 2)
        Dv[sl] = torch.exp(G[-1])[None]
    return W, Qg, Kd, Ut, M, Dv
