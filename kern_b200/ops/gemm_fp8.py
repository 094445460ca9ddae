"""FP8 (e4m3, per-tensor scale) GEMM on tcgen05 kind::f8f6f4, the quantiser that feeds it, and the fp32 statement."""
from __future__ import annotations

import struct

import torch

from .launcher import Kernels, i32, ptr

BM, BKE = 128, 128


def quantize(x: torch.Tensor):
    """bf16 [*, K] -> (e4m3 bytes as uint8, same shape; f32 scale[1]) with scale = amax / 448."""
    k = Kernels.get(x.device)
    assert x.dtype == torch.bfloat16 and x.is_contiguous()
    n = x.numel()
    amax = torch.zeros(1, dtype=torch.int32, device=x.device)
    scale = torch.empty(1, dtype=torch.float32, device=x.device)
    y = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    grid = (max(1, min(1184, (n + 255) // 256)),)
    k.launch("gemm_fp8", "kern_amax_bf16", grid, (256,), [ptr(x), struct.pack("<Q", n), ptr(amax)])
    k.launch("gemm_fp8", "kern_quant_e4m3", grid, (256,), [ptr(x), ptr(y), struct.pack("<Q", n), ptr(amax), ptr(scale)])
    return y, scale


def gemm_fp8(a: torch.Tensor, w: torch.Tensor, scale_a: torch.Tensor, scale_w: torch.Tensor, out: torch.Tensor | None = None,
             residual: torch.Tensor | None = None, bn: int | None = None) -> torch.Tensor:
    """a [M, K] e4m3 bytes, w [N, K] e4m3 bytes -> bf16 [M, N] = sa * sw * a . w^T (+ residual)."""
    k = Kernels.get(a.device)
    assert a.dtype == torch.uint8 and w.dtype == torch.uint8 and a.shape[1] == w.shape[1] and a.shape[1] % 16 == 0
    M, K = a.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    acc = residual is not None
    if bn is None:
        tiles_m = (M + BM - 1) // BM
        bn = 256 if tiles_m * ((N + 255) // 256) >= k.sm_count else (128 if N >= 128 else 64)
        if acc and bn == 64:
            bn = 128
    tma_a = k.tensor_map_2d(a, BM, BKE)
    tma_b = k.tensor_map_2d(w, bn, BKE)
    stages = {256: 4, 128: 6, 64: 8}[bn]
    smem = 1024 + stages * (BM * 128 + bn * 128) + 256
    entry = f"kern_gemm_e4m3_tn{'_acc' if acc else ''}_n{bn}"
    k.launch("gemm_fp8", entry, (k.sm_count,), (192,),
             [tma_a, tma_b, ptr(out), ptr(residual), ptr(scale_a), ptr(scale_w), i32(M), i32(N), i32(K), i32(out.stride(0)),
              ptr(k.err_word())], shared_mem=smem)
    return out


def dequant(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return q.view(torch.float8_e4m3fn).float() * scale.float()
