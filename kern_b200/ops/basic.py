"""Wrappers for the row-wise kernels (embedding, RMSNorm, gating, argmax, sampling) and their
PyTorch fp32 reference statements."""
from __future__ import annotations

import torch

from .launcher import Kernels, f32, i32, i64, ptr


def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    k = Kernels.get(table.device)
    t, (v, h) = ids.numel(), table.shape
    assert h % 8 == 0 and table.dtype == torch.bfloat16
    if out is None:
        out = torch.empty(t, h, dtype=torch.bfloat16, device=table.device)
    entry = "kern_embedding_i64_bf16" if ids.dtype == torch.int64 else "kern_embedding_i32_bf16"
    k.launch("norm_embed", entry, (t,), (min(256, max(32, h // 8)),),
             [ptr(ids), ptr(table), ptr(out), i32(t), i32(h), i32(v), ptr(k.err_word())])
    return out


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6, out: torch.Tensor | None = None,
             plus_one: bool = False, rows: int | None = None) -> torch.Tensor:
    """``y = x * rsqrt(mean(x²) + eps) * w`` per row of a 2-D bf16 tensor (row stride free)."""
    k = Kernels.get(x.device)
    r = x.shape[0] if rows is None else rows
    n = x.shape[1]
    assert n % 8 == 0 and n <= 16384 and x.stride(1) == 1
    if out is None:
        out = torch.empty(x.shape[0], n, dtype=torch.bfloat16, device=x.device)
    entry = "kern_rms_norm_bf16" if n <= 8192 else "kern_rms_norm_wide_bf16"
    k.launch("norm_embed", entry, (r,), (256,),
             [ptr(x), ptr(w), ptr(out), i32(r), i32(n), i32(x.stride(0)), i32(out.stride(0)),
              f32(eps), i32(int(plus_one))])
    return out


def fused_add_rms_norm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float = 1e-6,
                       out: torch.Tensor | None = None, plus_one: bool = False) -> torch.Tensor:
    """``residual += x`` in place; returns ``norm(residual) * w``."""
    k = Kernels.get(x.device)
    r, n = x.shape
    assert n % 8 == 0 and n <= 16384 and x.is_contiguous() and residual.is_contiguous()
    if out is None:
        out = torch.empty_like(x)
    k.launch("norm_embed", "kern_fused_add_rms_norm_bf16", (r,), (256,),
             [ptr(x), ptr(residual), ptr(w), ptr(out), i32(r), i32(n), f32(eps), i32(int(plus_one))])
    return out


def silu_mul(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    k = Kernels.get(x.device)
    t, d2 = x.shape
    d = d2 // 2
    assert d % 8 == 0 and x.is_contiguous()
    if out is None:
        out = torch.empty(t, d, dtype=torch.bfloat16, device=x.device)
    k.launch("norm_embed", "kern_silu_mul_bf16", (t, max(1, (d // 8 + 255) // 256)), (256,),
             [ptr(x), ptr(out), i32(t), i32(d)])
    return out


def sigmoid_mul(x: torch.Tensor, gate: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    k = Kernels.get(x.device)
    t, d = x.shape
    if out is None:
        out = torch.empty(t, d, dtype=torch.bfloat16, device=x.device)
    k.launch("norm_embed", "kern_sigmoid_mul_bf16", (t, max(1, (d + 255) // 256)), (256,),
             [ptr(x), ptr(gate), ptr(out), i32(t), i32(d), i32(x.stride(0)), i32(gate.stride(0))])
    return out


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None, rows: int | None = None,
           parts: int = 32) -> torch.Tensor:
    """Greedy token per row (ties → lowest index), int64."""
    k = Kernels.get(logits.device)
    r = logits.shape[0] if rows is None else rows
    v = logits.shape[1]
    if out is None:
        out = torch.empty(logits.shape[0], dtype=torch.int64, device=logits.device)
    pv = torch.empty(r, parts, dtype=torch.float32, device=logits.device)
    pi = torch.empty(r, parts, dtype=torch.int32, device=logits.device)
    entry = "kern_argmax_partial_bf16" if logits.dtype == torch.bfloat16 else "kern_argmax_partial_f32"
    k.launch("sampling", entry, (r, parts), (256,),
             [ptr(logits), ptr(pv), ptr(pi), i32(r), i32(v), i32(logits.stride(0))])
    k.launch("sampling", "kern_argmax_final_i64", (r,), (32,),
             [ptr(pv), ptr(pi), ptr(out), i32(r), i32(parts)])
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor | None = None,
           top_p: torch.Tensor | None = None, min_p: torch.Tensor | None = None,
           seeds: torch.Tensor | None = None, offsets: torch.Tensor | None = None,
           out: torch.Tensor | None = None) -> torch.Tensor:
    """Temperature / top-k / top-p / min-p sampling; rows with temperature <= 0 are greedy."""
    k = Kernels.get(logits.device)
    r, v = logits.shape
    if out is None:
        out = torch.empty(r, dtype=torch.int64, device=logits.device)
    probs = torch.empty(r, v, dtype=torch.float32, device=logits.device)
    entry = "kern_sample_bf16" if logits.dtype == torch.bfloat16 else "kern_sample_f32"
    k.launch("sampling", entry, (r,), (1024,),
             [ptr(logits), ptr(probs), ptr(out), ptr(temperature), ptr(top_k), ptr(top_p), ptr(min_p),
              ptr(seeds), ptr(offsets), i32(r), i32(v), i32(logits.stride(0))])
    return out


# ---- PyTorch fp32 references ---------------------------------------------------------------------
def rms_norm_reference(x, w, eps=1e-6, plus_one=False):
    xf = x.float()
    ww = w.float() + 1.0 if plus_one else w.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * ww).to(torch.bfloat16)


def silu_mul_reference(x):
    d = x.shape[1] // 2
    return (torch.nn.functional.silu(x[:, :d].float()) * x[:, d:].float()).to(torch.bfloat16)


def kept_set_reference(logits_row: torch.Tensor, temperature: float, top_k: int, top_p: float,
                       min_p: float) -> torch.Tensor:
    """Boolean mask of the tokens a sampler may return for one row (fp32 statement of the filters)."""
    p = torch.softmax(logits_row.float() / temperature, -1)
    keep = torch.ones_like(p, dtype=torch.bool)
    if top_k and top_k < p.numel():
        kth = torch.topk(p, top_k).values[-1]
        keep &= p >= kth
    if top_p < 1.0:
        q = torch.where(keep, p, torch.zeros_like(p))
        sv, si = torch.sort(q, descending=True)
        cum = torch.cumsum(sv, 0)
        total = q.sum()
        n = int((cum < top_p * total).sum().item()) + 1
        m = torch.zeros_like(keep)
        m[si[:n]] = True
        keep &= m
    if min_p > 0:
        keep &= p >= min_p * p.max()
    return keep
