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


def plan(ids: torch.Tensor, experts_local: int, e_lo: int = 0, aligned: bool = False):
    """-> dict(perm [T*k], offsets [E+1], tiles [max,4], tile_count [1], rows [1]). `aligned`: every expert's rows start
    on a 128-row boundary of the sorted buffer (what the block-scaled GEMM needs); `rows_bound` is then the buffer size."""
    kn = Kernels.get(ids.device)
    entries = ids.numel()
    dev = ids.device
    mt = max_tiles(entries, experts_local)
    out = {"perm": torch.empty(entries, dtype=torch.int32, device=dev),
           "offsets": torch.empty(experts_local + 1, dtype=torch.int32, device=dev),
           "tiles": torch.zeros(mt, 4, dtype=torch.int32, device=dev),
           "tile_count": torch.zeros(1, dtype=torch.int32, device=dev),
           "rows": torch.zeros(1, dtype=torch.int32, device=dev), "max_tiles": mt,
           "rows_bound": (-(-entries // BM) + experts_local) * BM if aligned else entries}
    kn.launch("moe", "kern_moe_plan_aligned" if aligned else "kern_moe_plan", (1,), (1024,),
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


# ---- block-scaled experts: MXFP8 activations x MXFP4 weights ------------------------------------------------------
def prepare_expert_weights_mx(w1: torch.Tensor, w2: torch.Tensor):
    """bf16/fp32 expert weights -> what the block-scaled layer reads: w1 [E, 2I, H] (gate rows then up rows) is
    re-ordered into groups of 128 rows = 64 gate rows + the matching 64 up rows, both are quantised to MXFP4 (packed
    nibbles) with their scales as atoms per expert. Returns (w1_q [E, 2I, H/2], sf1 [E, atoms], w2_q [E, H, I/2], sf2)."""
    from . import gemm_mx as G

    e, two_i, h = w1.shape
    inter = two_i // 2
    assert inter % 64 == 0
    gate, up = w1[:, :inter].reshape(e, inter // 64, 64, h), w1[:, inter:].reshape(e, inter // 64, 64, h)
    w1i = torch.cat([gate, up], 2).reshape(e, two_i, h)
    q1, s1, q2, s2 = [], [], [], []
    for x in range(e):
        q, sf = G.quantize_mxfp4_torch(w1i[x])
        q1.append(q); s1.append(G.sf_to_atoms(sf))
        q, sf = G.quantize_mxfp4_torch(w2[x])
        q2.append(q); s2.append(G.sf_to_atoms(sf))
    return torch.stack(q1), torch.stack(s1), torch.stack(q2), torch.stack(s2)


def gather_quant_mx(x: torch.Tensor, perm: torch.Tensor, k: int, rows_bound: int):
    """Expert-sorted MXFP8 activations (+ scale atoms) straight from the bf16 rows."""
    from . import gemm_mx as G

    kn = Kernels.get(x.device)
    t, h = x.shape
    q = torch.zeros(rows_bound, h, dtype=torch.uint8, device=x.device)
    sf = torch.full((G.atom_bytes(rows_bound, h),), 0x7F, dtype=torch.uint8, device=x.device)
    kn.launch("gemm_mx", "kern_moe_gather_quant_mxfp8", (t * k,), (128,), [ptr(x), ptr(perm), ptr(q), ptr(sf), i32(t * k), i32(k), i32(h)])
    return q, sf


def grouped_gemm_mx(a_q, sfa, w_q, sfw, pl: dict, swiglu_mxfp8: bool = False, bn: int = 256):
    """Routed block-scaled GEMM over the planner's (aligned) tile table. a_q [rows, K] e4m3, w_q [E, N, K/2] packed e2m1,
    scales as atoms (sfw per expert). Store form -> bf16 [rows, N]; `swiglu_mxfp8` -> (e4m3 [rows, N/2], its scale atoms)."""
    from . import gemm_mx as G
    from .launcher import i64

    kn = Kernels.get(a_q.device)
    rows, k = a_q.shape
    e, n, half = w_q.shape
    assert half * 2 == k and k % G.BK == 0 and n % bn == 0 and w_q.is_contiguous() and sfw.is_contiguous()
    tma_a = kn.tensor_map_2d(a_q, G.BM, G.BK)
    tma_b = kn.dev.encode_tensor_map(w_q.data_ptr(), G.TM_16U4_ALIGN16B, [k, n, e], [half, n * half], [G.BK, bn, 1], 128, 256, False)
    stages = 4 if bn == 256 else 6
    smem = 1024 + stages * (G.BM * G.BK + bn * G.BK + (2048 if bn == 256 else 1024)) + 256
    if swiglu_mxfp8:
        out = torch.zeros(rows, n // 2, dtype=torch.uint8, device=a_q.device)
        sf_out = torch.full((G.atom_bytes(rows, n // 2),), 0x7F, dtype=torch.uint8, device=a_q.device)
        entry = f"kern_moe_gemm_mxfp8_mxfp4_swiglu_mxfp8_n{bn}"
    else:
        out = torch.empty(rows, n, dtype=torch.bfloat16, device=a_q.device)
        sf_out = None
        entry = f"kern_moe_gemm_mxfp8_mxfp4_n{bn}"
    kn.launch("gemm_mx", entry, (kn.sm_count,), (192,),
              [tma_a, tma_b, ptr(sfa), ptr(sfw), ptr(out), i32(rows), i32(n), i32(k), i32(out.stride(0)), ptr(kn.err_word()),
               ptr(pl["tiles"]), ptr(pl["tile_count"]), i64(sfw.stride(0)), ptr(sf_out)], shared_mem=smem)
    return (out, sf_out) if swiglu_mxfp8 else out


def moe_layer_mx(x, w_router, w1_q, sf1, w2_q, sf2, k, bias=None, mode="sigmoid", scale=1.0, e_lo=0, shared=None, bn=256):
    """The routed layer with MXFP4 expert weights and MXFP8 activations: route (bf16 router) -> aligned plan ->
    gather + quantise -> FC1 (SwiGLU, MXFP8 out) -> FC2 (bf16 out) -> weighted combine."""
    from .gemm import gemm

    logits = gemm(x, w_router, epilogue="f32")
    ids, wts = route(logits, k, bias, mode, True, scale)
    pl = plan(ids, w1_q.shape[0], e_lo, aligned=True)
    xq, sfx = gather_quant_mx(x, pl["perm"], k, pl["rows_bound"])
    act_q, sf_act = grouped_gemm_mx(xq, sfx, w1_q, sf1, pl, swiglu_mxfp8=True, bn=bn)
    yp = grouped_gemm_mx(act_q, sf_act, w2_q, sf2, pl, bn=bn)
    out = torch.empty_like(x)
    return combine(yp, pl["perm"], wts, out, shared)


def moe_reference_mx(x, w_router, w1, w2, k, bias=None, mode="sigmoid", scale=1.0, e_lo=0, shared=None):
    """fp32 statement of the block-scaled layer: the same quantisation points (activations to MXFP8 before each expert
    GEMM, weights to MXFP4), everything else in fp32. w1 / w2 are the unquantised weights in checkpoint order."""
    from . import gemm_mx as G

    xf = x.float()
    logits = xf @ w_router.float().t()
    ids, wts = route_reference(logits, k, bias, mode, True, scale)
    out = torch.zeros_like(xf) if shared is None else shared.float().clone()
    inter = w1.shape[1] // 2
    xq = G.dequant_mxfp8(*G.quantize_mxfp8_torch(xf))
    for e in range(w1.shape[0]):
        tok, j = torch.nonzero(ids == e + e_lo, as_tuple=True)
        if tok.numel() == 0:
            continue
        w1d = G.dequant_mxfp4(*G.quantize_mxfp4_torch(w1[e].float()))
        w2d = G.dequant_mxfp4(*G.quantize_mxfp4_torch(w2[e].float()))
        h = xq[tok] @ w1d.t()
        act = F.silu(h[:, :inter]) * h[:, inter:]
        act = G.dequant_mxfp8(*G.quantize_mxfp8_torch(act))
        y = (act @ w2d.t()).to(torch.bfloat16).float()
        out.index_add_(0, tok, y * wts[tok, j][:, None])
    return out
