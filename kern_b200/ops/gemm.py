"""bf16 TN GEMM on tcgen05: ``C[M,N] = A[M,K] @ W[N,K]^T`` with fused epilogues.

The op behind the manifest externs ``extern:cublaslt_bf16_tn`` (store), ``extern:cublaslt_bf16_tn_acc``
(C += A·Wᵀ) and ``extern:cublas_bf16_tn_f32`` (f32 out) — reference call sites:
crates/kern-runtime/src/cublas.rs:78-107, 242-277, 329-378 — plus a SwiGLU epilogue that replaces
the separate ``silu_mul`` launch (tools/kernels-src/silu_mul.cu:10).
"""
from __future__ import annotations

import torch

from .launcher import Kernels, i32, ptr

BM, BK = 128, 64
_STAGES = {256: 4, 128: 6, 64: 8, 32: 8}
_EPI = {"store": "", "f32": "_f32", "acc": "_acc", "swiglu": "_swiglu"}
_TILES = {"store": (256, 128, 64, 32), "f32": (256, 128, 64), "acc": (256, 128, 64, 32),
          "swiglu": (256, 128, 64)}


def smem_bytes(bn: int) -> int:
    return 1024 + _STAGES[bn] * (BM * BK * 2 + bn * BK * 2) + 256


def pick_bn(m: int, n: int, sms: int, epilogue: str = "store") -> int:
    """Largest N tile that still gives every SM a tile; small problems fall to narrower tiles."""
    num_m = (m + BM - 1) // BM
    choices = _TILES[epilogue]
    if num_m <= 2:       # weight-bound: the width with the least waves x width, i.e. the most even cover of the SMs
        return min([c for c in choices if c >= 64], key=lambda bn: (-(-(num_m * ((n + bn - 1) // bn)) // sms) * bn * (1 + 8 / bn), -bn))
    for bn in choices:
        if num_m * ((n + bn - 1) // bn) >= sms:
            return bn
    return choices[-1]


def pick_bm(m: int, n: int, bn: int, sms: int, epilogue: str = "store") -> int:
    """256-row tiles (a third less L2 traffic per FLOP) once they still fill the machine evenly; else 128."""
    if bn != 256 or epilogue not in ("store", "acc", "swiglu") or not M256_ENABLED:
        return 128
    t256 = ((m + 255) // 256) * ((n + 255) // 256)
    t128 = ((m + 127) // 128) * ((n + 255) // 256)
    # time ~ waves x tile work; a 256-row tile is two 128-row tiles of work done M256_GAIN times faster
    cost256 = -(-t256 // sms) * 2.0 / M256_GAIN
    cost128 = -(-t128 // sms) * 1.0
    return 256 if cost256 < cost128 else 128


M256_ENABLED = True
M256_GAIN = 1.10          # measured speed of the 256-row tile over two 128-row tiles at large sizes


def stack_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Weights for the SwiGLU epilogue: all gate rows, then all up rows."""
    assert up.shape == gate.shape
    return torch.cat([gate, up], 0).contiguous()


GEMV_ROWS = 4        # up to this many rows the weight-streaming kernel runs instead of the tensor-core tiles
                     # (measured: at 16 rows the activations' L1 traffic makes it 2-3x slower than the tiles)


def gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None, *,
         epilogue: str = "store", residual: torch.Tensor | None = None, bn: int | None = None,
         m: int | None = None, pdl: bool = False, bm: int | None = None) -> torch.Tensor:
    """``a[M,K]`` bf16 row-major (row stride free), ``w[N,K]`` bf16; returns ``out``.

    epilogue: ``store`` (bf16), ``f32``, ``acc`` (bf16 ``out = a·wᵀ + residual``; residual defaults
    to ``out`` itself), ``swiglu`` (``out[M, N/2] = silu(gate)·up`` over weights stacked [gate; up]).
    ``m`` runs only the first m rows (the tensor maps are made for the whole buffer, so a decode
    step with fewer rows reuses them).
    """
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert a.dim() == 2 and w.dim() == 2 and a.shape[1] == w.shape[1]
    M = a.shape[0] if m is None else m
    N, K = w.shape
    assert K % 8 == 0 and N % (16 if epilogue == "swiglu" else 8) == 0
    k = Kernels.get(a.device)
    out_cols = N // 2 if epilogue == "swiglu" else N
    if out is None:
        dt = torch.float32 if epilogue == "f32" else torch.bfloat16
        out = torch.empty(a.shape[0], out_cols, dtype=dt, device=a.device)
    assert out.stride(1) == 1 and out.shape[1] == out_cols
    if epilogue == "acc" and residual is None:
        residual = out
    if residual is not None:
        assert residual.stride(0) == out.stride(0) and residual.dtype == torch.bfloat16
    if M == 0:
        return out
    if bn is None and M <= GEMV_ROWS and w.is_contiguous():
        # a handful of rows: stream the weights once on every SM instead of filling one 128-row tile
        mt = next(t for t in (1, 2, 4, 8) if M <= t)
        k.launch("gemv_bf16", f"kern_gemv_bf16_tn{_EPI[epilogue]}_m{mt}", (k.sm_count * 8,), (256,),
                 [ptr(a), ptr(w), ptr(out), ptr(residual), i32(M), i32(N), i32(K), i32(a.stride(0)), i32(out.stride(0)), ptr(k.err_word())], pdl=pdl)
        return out
    if bn is None:
        bn = pick_bn(M, N, k.sm_count, epilogue)
    if bm is None:
        bm = pick_bm(M, N, bn, k.sm_count, epilogue)
    assert bm in (128, 256) and (bm == 128 or (bn == 256 and epilogue in ("store", "acc", "swiglu")))
    tma_a = k.tensor_map_2d(a, bm, BK)
    tma_b = k.tensor_map_2d(w, bn // 2 if epilogue == "swiglu" else bn, BK)
    tiles = ((M + bm - 1) // bm) * ((N + bn - 1) // bn)
    grid = min(tiles, k.sm_count)
    entry = f"kern_gemm_bf16_tn{_EPI[epilogue]}{'_m256' if bm == 256 else ''}_n{bn}"
    k.launch("gemm_bf16", entry, (grid,), (192,),
             [tma_a, tma_b, ptr(out), ptr(residual), i32(M), i32(N), i32(K), i32(out.stride(0)),
              ptr(k.err_word())],
             shared_mem=smem_bytes(bn), pdl=pdl)
    return out


def gemm_reference(a: torch.Tensor, w: torch.Tensor, epilogue: str = "store",
                   residual: torch.Tensor | None = None) -> torch.Tensor:
    """Plain PyTorch fp32 statement of the same op (the numerics oracle)."""
    acc = a.float() @ w.float().t()
    if epilogue == "f32":
        return acc
    if epilogue == "acc":
        return (acc + residual.float()).to(torch.bfloat16)
    if epilogue == "swiglu":
        n = acc.shape[1]
        return (torch.nn.functional.silu(acc[:, : n // 2]) * acc[:, n // 2:]).to(torch.bfloat16)
    return acc.to(torch.bfloat16)
