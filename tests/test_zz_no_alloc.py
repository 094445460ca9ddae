"""The allocation-free C entry point for split-KV decode attention, called through its exported symbol.

Some callers cannot allocate device memory when they need attention (a plugin inside another engine's
no-malloc section, a process whose memory belongs to a pool it does not own, a plain C host), so the
library carries the split-KV workspace itself. This test calls `kern_attn_decode_split_noalloc` with
ctypes twice in a row — the second call reuses the workspace the first one left dirty — and holds
both results to the ordinary entry point's (`paged_attention` with a caller-allocated workspace) within
the tolerance the other attention tests use. It also checks that an ask beyond the built-in workspace is
refused with a clear message instead of being launched.
"""
import ctypes
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = Path(__file__).resolve().parent.parent / "kern_b200" / "libattn_decode_noalloc.so"


def _load():
    import kern_b200  # noqa: F401  (builds the library if it is missing)

    lib = ctypes.CDLL(str(LIB))
    lib.kern_attn_decode_split_noalloc.restype = ctypes.c_int
    lib.kern_attn_decode_split_noalloc.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int] * 11 + [ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p]
    lib.kern_noalloc_last_error.restype = ctypes.c_char_p
    return lib


def _case(cuda, seed, lens, hq=32, hk=8, d=128, page=16):
    torch.manual_seed(seed)
    seqs = len(lens)
    max_pages = max((l + page - 1) // page for l in lens) + 1
    total = sum((l + page - 1) // page for l in lens) + 2
    pool = (torch.randn(total, 2, hk, page, d, device=cuda)).to(torch.bfloat16)
    perm = torch.randperm(total)
    table = torch.zeros(seqs, max_pages, dtype=torch.int32, device=cuda)
    nxt = 0
    for s, l in enumerate(lens):
        for p in range((l + page - 1) // page):
            table[s, p] = int(perm[nxt])
            nxt += 1
    q = torch.randn(seqs, hq * d, device=cuda).to(torch.bfloat16)
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=cuda)
    return q, pool, table, seq_lens


def _call(lib, q, pool, table, seq_lens, hq, splits):
    pages, _, hk, page, d = pool.shape
    out = torch.empty(q.shape[0], hq * d, dtype=torch.bfloat16, device=q.device)
    err = torch.zeros(1, dtype=torch.int32, device=q.device)
    rc = lib.kern_attn_decode_split_noalloc(
        q.data_ptr(), pool.data_ptr(), table.data_ptr(), seq_lens.data_ptr(), out.data_ptr(), table.shape[0], 1, hq, hk, d,
        page, table.shape[1], pages, q.stride(0), out.stride(0), splits, float(d ** -0.5), err.data_ptr(),
        torch.cuda.current_stream().cuda_stream)
    return rc, out, err


def test_no_alloc_entry_matches_the_allocating_one_twice(cuda):
    from kern_b200.ops import attention as A

    lib = _load()
    for seed, lens, splits in ((0, [700, 64, 1500, 3], 4), (1, [129, 2048], 8)):
        q, pool, table, seq_lens = _case(cuda, seed, lens)
        ref = A.paged_attention(q, pool, table, seq_lens, 32, splits=splits)
        rc, out, err = _call(lib, q, pool, table, seq_lens, 32, splits)
        assert rc == 0, lib.kern_noalloc_last_error()
        torch.cuda.synchronize()
        assert int(err.item()) == 0
        torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-2)


def _fp32_statement(q, pool, table, seq_lens, hq):
    """Plain PyTorch fp32 decode attention over the paged pool; an empty sequence gives a zero row."""
    _, _, hk, page, d = pool.shape
    out = torch.zeros(q.shape[0], hq * d, dtype=torch.float32, device=q.device)
    for s, l in enumerate(seq_lens.tolist()):
        if l == 0:
            continue
        ids = table[s, : (l + page - 1) // page].long()
        k = pool[ids, 0].permute(1, 0, 2, 3).reshape(hk, -1, d)[:, :l].float()
        v = pool[ids, 1].permute(1, 0, 2, 3).reshape(hk, -1, d)[:, :l].float()
        qs = q[s].float().view(hk, hq // hk, d)
        p = torch.softmax(torch.einsum("kgd,kld->kgl", qs, k) * d ** -0.5, -1)
        out[s] = torch.einsum("kgl,kld->kgd", p, v).reshape(-1)
    return out


def test_no_alloc_entry_with_an_empty_sequence_against_fp32(cuda):
    """A sequence of length 0 launches no work for its rows: they must come out zero, on a workspace the call before
    left dirty, and the live rows must match a plain fp32 statement of the op."""
    lib = _load()
    q, pool, table, seq_lens = _case(cuda, 3, [300, 1, 90])
    _call(lib, q, pool, table, seq_lens, 32, 4)                 # dirties the workspace for every row
    seq_lens[1] = 0
    rc, out, err = _call(lib, q, pool, table, seq_lens, 32, 4)
    assert rc == 0, lib.kern_noalloc_last_error()
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    assert float(out[1].float().abs().max()) == 0.0
    torch.testing.assert_close(out.float(), _fp32_statement(q, pool, table, seq_lens, 32), rtol=2e-2, atol=2e-2)


def test_no_alloc_entry_refuses_what_does_not_fit(cuda):
    lib = _load()
    q, pool, table, seq_lens = _case(cuda, 2, [64] * 40)
    # 40 rows * 32 heads * 32 splits * 128 = 5.2 Mi floats: more than the 2 Mi the library carries
    rc, _, _ = _call(lib, q, pool, table, seq_lens, 32, 32)
    assert rc == 2
    assert b"exceeds the built-in workspace" in lib.kern_noalloc_last_error()
    rc, _, _ = _call(lib, q, pool, table, seq_lens, 32, 1)
    assert rc == 1 and b"splits must be 2..32" in lib.kern_noalloc_last_error()
