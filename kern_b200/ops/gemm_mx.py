"""Block-scaled (OCP microscaling) GEMMs on tcgen05 `kind::mxf8f6f4.block_scale`: MXFP8 activations against MXFP8 or
MXFP4 weights, one UE8M0 scale per 32 elements; the quantisers, the scale-factor atom layout and the fp32 statements
the GPU tests compare against. Kernel: csrc/kernels/sm100/gemm_mx.cu.
Reference counterpart: crates/kern-runtime/src/cublas.rs:401-505 (cuBLASLt MXFP8, VEC32_UE8M0), and the routed expert
GEMMs it loads as prebuilt blobs (kernel_index/trtllm_bmm_mxe4m3_mxe2m1_mxe4m3.toml)."""
from __future__ import annotations

import torch

from .launcher import Kernels, i32, i64, ptr

BM, BK, ATOM = 128, 128, 512
TM_U8, TM_16U4_ALIGN16B = 0, 14              # CUtensorMapDataType codes
E2M1 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


# ---- scale-factor atoms ------------------------------------------------------------------------------
def atom_bytes(rows: int, k: int) -> int:
    return -(-rows // 128) * -(-k // BK) * ATOM


def sf_to_atoms(sf: torch.Tensor) -> torch.Tensor:
    """[R, K/32] UE8M0 bytes -> the atom layout the kernel reads: atom (r // 128, kb // 4) of 512 bytes, inside it
    (r % 32) * 16 + ((r // 32) % 4) * 4 + kb % 4. Rows and blocks are padded with scale 1 (0x7f)."""
    r, kb = sf.shape
    ra, ka = -(-r // 128), -(-kb // 4)
    full = torch.full((ra * 128, ka * 4), 0x7F, dtype=torch.uint8, device=sf.device)
    full[:r, :kb] = sf
    # [ra, 4 (r // 32 % 4), 32 (r % 32), ka, 4 (kb % 4)] -> [ra, ka, 32, 4, 4]
    return full.view(ra, 4, 32, ka, 4).permute(0, 3, 2, 1, 4).contiguous().view(-1)


def atoms_to_sf(atoms: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    ra, ka = -(-rows // 128), -(-k // BK)
    return atoms.view(ra, ka, 32, 4, 4).permute(0, 3, 2, 1, 4).contiguous().view(ra * 128, ka * 4)[:rows, : k // 32]


# ---- quantisers ----------------------------------------------------------------------------------------
def quantize_mxfp8(x: torch.Tensor):
    """bf16 [M, K] -> (e4m3 bytes [M, K], scale atoms) on the device (kern_quant_mxfp8)."""
    k = Kernels.get(x.device)
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1 and x.shape[1] % 32 == 0
    m, kk = x.shape
    q = torch.empty(m, kk, dtype=torch.uint8, device=x.device)
    sf = torch.full((atom_bytes(m, kk),), 0x7F, dtype=torch.uint8, device=x.device)
    grid = (max(1, min(8 * k.sm_count, (m * (kk // 32) + 7) // 8)),)
    k.launch("gemm_mx", "kern_quant_mxfp8", grid, (256,), [ptr(x), ptr(q), ptr(sf), i32(m), i32(kk), i32(x.stride(0))])
    return q, sf


def quantize_mxfp8_torch(x: torch.Tensor):
    """The same arithmetic in PyTorch (fp32): (e4m3 bytes, [M, K/32] scale bytes)."""
    m, kk = x.shape
    xb = x.float().view(m, kk // 32, 32)
    amax = xb.abs().amax(-1)
    mant, ex = torch.frexp(amax)                      # amax = mant * 2^ex, mant in [0.5, 1); 448 = 0.875 * 2^9
    e = torch.where(amax > 0, torch.where(mant <= 0.875, ex - 9, ex - 8).float(), torch.zeros_like(amax)).clamp(-127, 127)
    q = (xb * torch.exp2(-e)[..., None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).view(m, kk)
    return q, (e + 127).to(torch.uint8)


def quantize_mxfp4_torch(w: torch.Tensor):
    """fp32/bf16 [N, K] -> (packed e2m1 nibbles [N, K/2], [N, K/32] UE8M0 scale bytes): the scale is the smallest power
    of two that brings the block's amax under 6, values round to the nearest e2m1 point."""
    n, kk = w.shape
    wb = w.float().view(n, kk // 32, 32)
    amax = wb.abs().amax(-1)
    mant, ex = torch.frexp(amax)                      # 6 = 0.75 * 2^3
    e = torch.where(amax > 0, torch.where(mant <= 0.75, ex - 3, ex - 2).float(), torch.zeros_like(amax)).clamp(-127, 127)
    v = wb * torch.exp2(-e)[..., None]
    grid = torch.tensor(E2M1, device=w.device)
    idx = (v.abs()[..., None] - grid).abs().argmin(-1)
    code = (idx | ((v < 0).long() << 3)).to(torch.uint8).view(n, kk)
    packed = code[:, 0::2] | (code[:, 1::2] << 4)
    return packed.contiguous(), (e + 127).to(torch.uint8)


def dequant_mxfp8(q: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
    m, kk = q.shape
    return (q.view(torch.float8_e4m3fn).float().view(m, kk // 32, 32) * torch.exp2(sf.float() - 127)[..., None]).view(m, kk)


def dequant_mxfp4(packed: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
    n, half = packed.shape
    code = torch.stack([packed & 0xF, packed >> 4], -1).view(n, half * 2).long()
    val = torch.tensor(E2M1, device=packed.device)[code & 7] * torch.where((code & 8) != 0, -1.0, 1.0)
    return (val.view(n, half * 2 // 32, 32) * torch.exp2(sf.float() - 127)[..., None]).view(n, half * 2)


# ---- the GEMM ----------------------------------------------------------------------------------------------
def gemm_mx(a_q: torch.Tensor, sfa_atoms: torch.Tensor, w_q: torch.Tensor, sfw_atoms: torch.Tensor, fp4: bool,
            out: torch.Tensor | None = None, bn: int = 128) -> torch.Tensor:
    """a_q [M, K] e4m3 bytes; w_q [N, K] e4m3 bytes or [N, K/2] packed e2m1; scales as atoms -> bf16 [M, N]."""
    k = Kernels.get(a_q.device)
    m, kk = a_q.shape
    n = w_q.shape[0]
    assert a_q.dtype == torch.uint8 and w_q.dtype == torch.uint8 and kk % BK == 0
    assert w_q.shape[1] == (kk // 2 if fp4 else kk)
    assert sfa_atoms.numel() >= atom_bytes(m, kk) and sfw_atoms.numel() >= atom_bytes(n, kk)
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=a_q.device)
    tma_a = k.tensor_map_2d(a_q, BM, BK)
    if fp4:
        assert w_q.data_ptr() % 32 == 0 and (kk // 2) % 32 == 0, "packed 4-bit rows must be 32-byte aligned"
        tma_b = k.dev.encode_tensor_map(w_q.data_ptr(), TM_16U4_ALIGN16B, [kk, n], [kk // 2], [BK, bn], 128, 256, False)
    else:
        tma_b = k.tensor_map_2d(w_q, bn, BK)
    stages = 4 if bn == 256 else 6
    smem = 1024 + stages * (BM * BK + bn * BK + (2048 if bn == 256 else 1024)) + 256
    entry = f"kern_gemm_mxfp8_{'mxfp4_' if fp4 else ''}tn_n{bn}"
    k.launch("gemm_mx", entry, (k.sm_count,), (192,),
             [tma_a, tma_b, ptr(sfa_atoms), ptr(sfw_atoms), ptr(out), i32(m), i32(n), i32(kk), i32(out.stride(0)),
              ptr(k.err_word())], shared_mem=smem)
    return out
