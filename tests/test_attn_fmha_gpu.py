"""The tcgen05 causal prefill attention (S and O in TMEM, P through shared memory, V as an MN-major operand) against a
plain PyTorch fp32 statement: ragged rows, cached prefixes, pages smaller and larger than a tile, GQA groups."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def bf(t):
    return t.to(torch.bfloat16)


def _build_cache(cuda, lens, hk, d, page_size):
    seqs = len(lens)
    max_pages = max((l + page_size - 1) // page_size for l in lens) + 1
    total = sum((l + page_size - 1) // page_size for l in lens) + 3
    pool = bf(torch.randn(total, 2, hk, page_size, d, device=cuda) * 0.5)
    perm = torch.randperm(total)
    table = torch.zeros(seqs, max_pages, dtype=torch.int32, device=cuda)
    nxt, ks, vs = 0, [], []
    for s, l in enumerate(lens):
        n = (l + page_size - 1) // page_size
        ids = perm[nxt:nxt + n]
        nxt += n
        table[s, :n] = ids.to(torch.int32).to(cuda)
        k = pool[ids.to(cuda), 0].permute(0, 2, 1, 3).reshape(-1, hk, d)[:l]
        v = pool[ids.to(cuda), 1].permute(0, 2, 1, 3).reshape(-1, hk, d)[:l]
        ks.append(k)
        vs.append(v)
    return pool, table, ks, vs


@pytest.mark.parametrize("hq,hk,page_size", [(8, 2, 64), (4, 4, 16), (16, 2, 128), (4, 1, 64)])
@pytest.mark.parametrize("new,prefix", [([128], [0]), ([5, 64, 130, 257], [0, 17, 64, 300]), ([700, 33], [1000, 0])])
def test_fmha_prefill_matches_fp32(cuda, hq, hk, page_size, new, prefix):
    from kern_b200.ops import attention as A
    from kern_b200.ops.launcher import Kernels

    d = 128
    torch.manual_seed(6 + hq + page_size)
    lens = [n + p for n, p in zip(new, prefix)]
    pool, table, ks, vs = _build_cache(cuda, lens, hk, d, page_size)
    cu = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32, device=cuda)
    total = int(cu[-1])
    wide = bf(torch.randn(total, (hq + 2 * hk) * d, device=cuda))
    q = wide[:, : hq * d]
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=cuda)
    out = A.fmha_prefill(q, pool, table, seq_lens, hq, cu)
    torch.cuda.synchronize()
    Kernels.get(cuda).check_error()
    for s in range(len(lens)):
        lo, hi = int(cu[s]), int(cu[s + 1])
        qs = q[lo:hi].reshape(hi - lo, hq, d)
        pos = torch.arange(prefix[s], lens[s], device=cuda)
        ref = A.attention_reference(qs, ks[s], vs[s], pos)
        torch.testing.assert_close(out[lo:hi].float(), ref, rtol=2e-2, atol=2e-2)
