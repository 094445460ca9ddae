"""Device-side A/B comparison (wrappers) and the host definitions the tests hold them to.
Reference counterpart: crates/kern-test/src/compare.rs:16-92 (Cmp), crates/kern-runtime/src/compare.cu."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .launcher import Kernels, i32, ptr
import struct

_DT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2, torch.uint8: 3, torch.int8: 3}


@dataclass
class Cmp:
    n: int = 0
    n_diff: int = 0
    signed_zero: int = 0
    nan_only_one_side: int = 0
    measured: int = 0
    max_ulp: int = 0
    max_abs: float = 0.0

    @property
    def equal(self) -> bool:
        return self.n_diff == 0


def _u64(v: int) -> bytes:
    return struct.pack("<Q", int(v))


def cmp_reduce(a: torch.Tensor, b: torch.Tensor) -> Cmp:
    assert a.dtype == b.dtype and a.numel() == b.numel() and a.is_contiguous() and b.is_contiguous()
    k = Kernels.get(a.device)
    out = torch.zeros(6, dtype=torch.int64, device=a.device)
    n = a.numel()
    k.launch("compare", "kern_cmp_reduce", (max(1, min(1184, (n + 255) // 256)),), (256,),
             [ptr(a), ptr(b), _u64(n), i32(_DT[a.dtype]), ptr(out)])
    o = out.cpu().tolist()
    return Cmp(n=n, n_diff=o[0], signed_zero=o[1], nan_only_one_side=o[2], measured=o[3], max_ulp=o[4],
               max_abs=struct.unpack("<d", struct.pack("<q", o[5]))[0])


def cmp_reference(a: torch.Tensor, b: torch.Tensor) -> Cmp:
    fa, fb = a.double().flatten(), b.double().flatten()
    na, nb = fa.isnan(), fb.isnan()
    nan_one = int((na ^ nb).sum())
    both0 = (fa == 0) & (fb == 0)
    zero = int((both0 & (torch.signbit(fa) != torch.signbit(fb))).sum())
    ok = ~na & ~nb & ~both0 & (fa != fb)
    return Cmp(n=fa.numel(), n_diff=int(ok.sum()) + nan_one, signed_zero=zero, nan_only_one_side=nan_one,
               measured=int(ok.sum()), max_abs=float((fa - fb).abs()[ok].max()) if ok.any() else 0.0)


def changed_blocks(pre: torch.Tensor, post: torch.Tensor) -> torch.Tensor:
    """-> bool tensor, one entry per 64-byte block."""
    k = Kernels.get(pre.device)
    pb, qb = pre.contiguous().view(torch.uint8).flatten(), post.contiguous().view(torch.uint8).flatten()
    nbytes = pb.numel()
    blocks = (nbytes + 63) // 64
    bits = torch.zeros((blocks + 31) // 32, dtype=torch.int32, device=pre.device)
    k.launch("compare", "kern_changed_blocks", (max(1, min(1184, (blocks + 255) // 256)),), (256,),
             [ptr(pb), ptr(qb), _u64(nbytes), ptr(bits)])
    idx = torch.arange(blocks, device=pre.device)
    return ((bits[idx // 32] >> (idx % 32)) & 1).bool()


def logit_rows(a: torch.Tensor, b: torch.Tensor):
    """-> (argmax_a, argmax_b, top-1 margin of a, KL(a || b)) per row."""
    assert a.shape == b.shape and a.dim() == 2 and a.dtype == b.dtype and a.stride(0) == b.stride(0)
    k = Kernels.get(a.device)
    rows, cols = a.shape
    out = torch.zeros(rows, 4, dtype=torch.int64, device=a.device)
    k.launch("compare", "kern_logit_rows", (rows,), (256,),
             [ptr(a), ptr(b), struct.pack("<I", cols), i32(_DT[a.dtype]), _u64(a.stride(0)), ptr(out)])
    f = out[:, 2:].to(torch.int32).view(torch.float32)
    return out[:, 0], out[:, 1], f[:, 0], f[:, 1]
