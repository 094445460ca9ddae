"""Mixture-of-experts on one GPU: routing, the expert-sorted layout, the routed tcgen05 GEMMs and the weighted
combine; and the PyTorch fp32 statement of the same layer. Experts outside ``[e_lo, e_hi)`` are another rank's:
an expert-parallel rank computes its experts' share of every token and the shares are summed by the all-reduce."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .launcher import _TM_OF, Kernels, f32, i32, ptr

BM, BK = 128, 64


def route(logits: torch.Tensor, k: int, bias: torch.Tensor | None = None, mode: str = "sigmoid", renorm: bool = True,
          scale: float = 1.0):
    """logits f32 [T, E] -> (ids i32 [T, k], weights f32 [T, k])."""
    kn = Kernels.get(logits.device)
    t, e = logits.shape
    assert logits.dtype == torch.float32 and e <= 1024 and k <= 32
    ids = torch.empty(t, k, dtype=torch.int32, device=logits.device)
    w = torch.empty(t, k, dtype=torch.float32, device=logits.device)
    kn.launch("moe", "kern_moe_route_f32", ((t + 3) // 4,), (128,),
              [ptr(logits), ptr(bias), ptr(ids), ptr(w), i32(t), i32(e), i32(k), i32(1 if mode == "softmax" else 0),
               i32(int(renorm)), f32(scale), i32(logits.stride(0))])
    return ids, w


def route_reference(logits, k, bias=None, mode="sigmoid", renorm=True, scale=1.0):
    s = torch.softmax(logits.float(), -1) if mode == "softmax" else torch.sigmoid(logits.float())
    sel = s + (bias.float() if bias is not None else 0.0)
    ids = torch.topk(sel, k, dim=-1).indices
    w = torch.gather(s, 1, ids)
    if renorm:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return ids.int(), w * scale


def max_tiles(entries: int, experts: int) -> int:
    return entries // BM + experts


def plan(ids: torch.Tensor, experts_local: int, e_lo: int = 0):
    """-> dict(perm [T*k], offsets [E+1], tiles [max,4], tile_count [1], rows [1])."""
    kn = Kernels.get(ids.device)
    entries = ids.numel()
    dev = ids.device
    mt = max_tiles(entries, experts_local)
    out = {"perm": torch.empty(entries, dtype=torch.int32, device=dev),
           "offsets": torch.empty(experts_local + 1, dtype=torch.int32, device=dev),
           "tiles": torch.zeros(mt, 4, dtype=torch.int32, device=dev),
           "tile_count": torch.zeros(1, dtype=torch.int32, device=dev),
           "rows": torch.zeros(1, dtype=torch.int32, device=dev), "max_tiles": mt}
    kn.launch("moe", "kern_moe_plan", (1,), (1024,),
              [ptr(ids), ptr(out["perm"]), ptr(out["offsets"]), ptr(out["tiles"]), ptr(out["tile_count"]), ptr(out["rows"]),
               i32(entries), i32(e_lo), i32(e_lo + experts_local), i32(BM), i32(mt), ptr(kn.err_word()), i32(0), i32(0)],
              shared_mem=2 * experts_local * 4)
    return out


def gather(x: torch.Tensor, perm: torch.Tensor, k: int, rows: int) -> torch.Tensor:
    kn = Kernels.get(x.device)
    t, h = x.shape
    xp = torch.zeros(rows, h, dtype=torch.bfloat16, device=x.device)
    kn.launch("moe", "kern_moe_gather_bf16", (t * k,), (128,), [ptr(x), ptr(perm), ptr(xp), i32(t * k), i32(k), i32(h)])
    return xp


def tensor_map_3d(kn: Kernels, w: torch.Tensor, box_rows: int) -> bytes:
    e, n, k = w.shape
    assert w.is_contiguous()
    es = w.element_size()
    return kn.dev.encode_tensor_map(w.data_ptr(), _TM_OF[w.dtype], [k, n, e], [k * es, n * k * es], [BK, box_rows, 1],
                                    128, 256, False)


def grouped_gemm(a_perm: torch.Tensor, w: torch.Tensor, pl: dict, epilogue: str = "store", bn: int | None = None) -> torch.Tensor:
    """C_perm[r] = A_perm[r] . W[expert of r]^T; w: [E_local, N, K]; swiglu: W rows are [gate ; up], C has N/2 columns."""
    kn = Kernels.get(a_perm.device)
    rows, k = a_perm.shape
    e, n, k2 = w.shape
    assert k == k2 and k % 8 == 0
    out_cols = n // 2 if epilogue == "swiglu" else n
    bn = bn or (256 if pl["max_tiles"] * (n // 256) >= 100 else 128 if n >= 128 else 64)
    c = torch.empty(rows, out_cols, dtype=torch.bfloat16, device=a_perm.device)
    tma_a = kn.tensor_map_2d(a_perm, BM, BK)
    tma_b = tensor_map_3d(kn, w, bn // 2 if epilogue == "swiglu" else bn)
    stages = {256: 4, 128: 6, 64: 8}[bn]
    smem = 1024 + stages * (BM * BK * 2 + bn * BK * 2) + 256
    entry = f"kern_moe_gemm_bf16{'_swiglu' if epilogue == 'swiglu' else ''}_n{bn}"
    kn.launch("moe", entry, (kn.sm_count,), (192,),
              [tma_a, tma_b, ptr(c), ptr(pl["tiles"]), ptr(pl["tile_count"]), i32(rows), i32(n), i32(k), i32(out_cols),
               ptr(kn.err_word())], shared_mem=smem)
    return c


def combine(y_perm, perm, weights, out, shared=None, accumulate=False):
    kn = Kernels.get(out.device)
    t, h = out.shape
    k = weights.shape[1]
    kn.launch("moe", "kern_moe_combine_bf16", (t,), (128,),
              [ptr(y_perm), ptr(perm), ptr(weights), ptr(shared), ptr(out), i32(t), i32(k), i32(h), i32(int(accumulate))])
    return out


def moe_layer(x, w_router, w1, w2, k, bias=None, mode="sigmoid", scale=1.0, e_lo=0, shared=None):
    """x bf16 [T, H]; w_router bf16 [E, H]; w1 [E_local, 2I, H] (gate rows then up rows); w2 [E_local, H, I]."""
    from .gemm import gemm

    logits = gemm(x, w_router, epilogue="f32")
    ids, wts = route(logits, k, bias, mode, True, scale)
    pl = plan(ids, w1.shape[0], e_lo)
    rows = x.shape[0] * k          # upper bound of local rows; the tile table says which exist
    xp = gather(x, pl["perm"], k, rows)
    act = grouped_gemm(xp, w1, pl, "swiglu")
    yp = grouped_gemm(act, w2, pl, "store")
    out = torch.empty_like(x)
    return combine(yp, pl["perm"], wts, out, shared)


def moe_reference(x, w_router, w1, w2, k, bias=None, mode="sigmoid", scale=1.0, e_lo=0, shared=None):
    xf = x.float()
    logits = xf @ w_router.float().t()
    ids, wts = route_reference(logits, k, bias, mode, True, scale)
    out = torch.zeros_like(xf) if shared is None else shared.float().clone()
    inter = w1.shape[1] // 2
    for e in range(w1.shape[0]):
        tok, j = torch.nonzero(ids == e + e_lo, as_tuple=True)
        if tok.numel() == 0:
            continue
        h = xf[tok] @ w1[e].float().t()
        act = (F.silu(h[:, :inter]) * h[:, inter:]).to(torch.bfloat16).float()
        y = (act @ w2[e].float().t()).to(torch.bfloat16).float()
        out.index_add_(0, tok, y * wts[tok, j][:, None])
    return out
