"""Every hand-written op against a plain PyTorch fp32 statement of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def bf(x):
    return x.to(torch.bfloat16)


def check_err(dev):
    from kern_b200.ops.launcher import Kernels

    torch.cuda.synchronize()
    Kernels.get(dev).check_error()


@pytest.mark.parametrize("rows,n", [(1, 64), (7, 4096), (33, 5120), (4, 8192), (3, 16384)])
@pytest.mark.parametrize("plus_one", [False, True])
def test_rms_norm(cuda, rows, n, plus_one):
    from kern_b200.ops import basic

    torch.manual_seed(0)
    x, w = bf(torch.randn(rows, n, device=cuda) * 3), bf(torch.randn(n, device=cuda))
    y = basic.rms_norm(x, w, 1e-6, plus_one=plus_one)
    ref = basic.rms_norm_reference(x, w, 1e-6, plus_one)
    check_err(cuda)
    torch.testing.assert_close(y.float(), ref.float(), rtol=1.6e-2, atol=1e-2)


def test_fused_add_rms_norm(cuda):
    from kern_b200.ops import basic

    torch.manual_seed(1)
    x, r, w = bf(torch.randn(9, 4096, device=cuda)), bf(torch.randn(9, 4096, device=cuda)), bf(torch.randn(4096, device=cuda))
    r_ref = bf(x.float() + r.float())
    ref = basic.rms_norm_reference(r_ref, w)
    y = basic.fused_add_rms_norm(x, r, w)
    check_err(cuda)
    torch.testing.assert_close(r.float(), r_ref.float(), rtol=0, atol=0)
    torch.testing.assert_close(y.float(), ref.float(), rtol=1.6e-2, atol=1e-2)


def test_embedding_silu_sigmoid(cuda):
    from kern_b200.ops import basic

    torch.manual_seed(2)
    table = bf(torch.randn(1000, 512, device=cuda))
    ids = torch.randint(0, 1000, (37,), device=cuda)
    assert torch.equal(basic.embedding(ids, table), table[ids])
    assert torch.equal(basic.embedding(ids.int(), table), table[ids])
    x = bf(torch.randn(19, 2 * 1536, device=cuda))
    torch.testing.assert_close(basic.silu_mul(x).float(), basic.silu_mul_reference(x).float(), rtol=1.6e-2, atol=1e-2)
    a, g = bf(torch.randn(5, 768, device=cuda)), bf(torch.randn(5, 768, device=cuda))
    ref = bf(a.float() * torch.sigmoid(g.float()))
    torch.testing.assert_close(basic.sigmoid_mul(a, g).float(), ref.float(), rtol=1.6e-2, atol=1e-2)
    check_err(cuda)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_argmax(cuda, dtype):
    from kern_b200.ops import basic

    torch.manual_seed(3)
    logits = torch.randn(13, 151936, device=cuda).to(dtype)
    logits[3, 100] = logits[3, 70000] = 50.0  # a tie resolves to the lowest index
    got = basic.argmax(logits)
    check_err(cuda)
    ref = torch.stack([(row == row.max()).nonzero()[0, 0] for row in logits.float()])
    assert torch.equal(got, ref)
    assert int(got[3]) == 100


def test_sample_filters(cuda):
    from kern_b200.ops import basic

    torch.manual_seed(4)
    rows, vocab = 64, 5000
    logits = torch.randn(rows, vocab, device=cuda) * 3
    temp = torch.full((rows,), 0.8, device=cuda)
    temp[0] = 0.0  # greedy row
    top_k = torch.full((rows,), 50, dtype=torch.int32, device=cuda)
    top_p = torch.full((rows,), 0.9, device=cuda)
    min_p = torch.full((rows,), 0.02, device=cuda)
    seeds = torch.arange(rows, dtype=torch.int64, device=cuda) + 7
    offs = torch.zeros(rows, dtype=torch.int32, device=cuda)
    a = basic.sample(logits, temp, top_k, top_p, min_p, seeds, offs)
    b = basic.sample(logits, temp, top_k, top_p, min_p, seeds, offs)
    check_err(cuda)
    assert torch.equal(a, b), "same (seed, offset) must repeat the draw"
    assert int(a[0]) == int(logits[0].argmax())
    for r in range(1, rows):
        keep = basic.kept_set_reference(logits[r], 0.8, 50, 0.9, 0.02)
        # a token at the edge of a threshold may differ by rounding: allow neighbours of the kept set
        p = torch.softmax(logits[r] / 0.8, -1)
        assert bool(keep[a[r]]) or float(p[a[r]]) >= 0.95 * float(p[keep].min())
    c = basic.sample(logits, temp, top_k, top_p, min_p, seeds, offs + 1)
    assert not torch.equal(a[1:], c[1:])


def _build_cache(cuda, seqs, lens, hk, d, page_size, extra_pages=3):
    """Random K/V per sequence scattered over shuffled pages; returns pool, table, k/v lists."""
    max_pages = max((l + page_size - 1) // page_size for l in lens) + 1
    total = sum((l + page_size - 1) // page_size for l in lens) + extra_pages
    pool = bf(torch.randn(total, 2, hk, page_size, d, device=cuda))  # stale finite data everywhere
    perm = torch.randperm(total)
    table = torch.zeros(seqs, max_pages, dtype=torch.int32, device=cuda)
    ks, vs, nxt = [], [], 0
    for s, l in enumerate(lens):
        k = bf(torch.randn(l, hk, d, device=cuda))
        v = bf(torch.randn(l, hk, d, device=cuda))
        ks.append(k)
        vs.append(v)
        for p in range((l + page_size - 1) // page_size):
            pg = int(perm[nxt]); nxt += 1
            table[s, p] = pg
            lo, hi = p * page_size, min(l, (p + 1) * page_size)
            pool[pg, 0, :, : hi - lo] = k[lo:hi].transpose(0, 1)
            pool[pg, 1, :, : hi - lo] = v[lo:hi].transpose(0, 1)
    return pool, table, ks, vs


@pytest.mark.parametrize("hq,hk,d,page_size", [(32, 8, 128, 16), (8, 2, 64, 64), (24, 4, 256, 32), (4, 4, 128, 128)])
@pytest.mark.parametrize("rows,splits", [(1, 1), (1, 4), (3, None)])
def test_decode_attention(cuda, hq, hk, d, page_size, rows, splits):
    from kern_b200.ops import attention as A

    torch.manual_seed(5)
    lens = [1 + rows, 63, 64, 65, 300, 1000][: 6]
    lens = [max(l, rows) for l in lens]
    seqs = len(lens)
    pool, table, ks, vs = _build_cache(cuda, seqs, lens, hk, d, page_size)
    q = bf(torch.randn(seqs * rows, hq * d, device=cuda))
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=cuda)
    out = A.paged_attention(q, pool, table, seq_lens, hq, rows_per_seq=rows, splits=splits)
    check_err(cuda)
    for s, l in enumerate(lens):
        qs = q[s * rows:(s + 1) * rows].view(rows, hq, d)
        pos = torch.arange(l - rows, l, device=cuda)
        ref = A.attention_reference(qs, ks[s], vs[s], pos)
        torch.testing.assert_close(out[s * rows:(s + 1) * rows].float(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("hq,hk,d,page_size", [(32, 8, 128, 16), (8, 8, 64, 64), (12, 2, 256, 64)])
def test_prefill_attention_ragged_with_prefix(cuda, hq, hk, d, page_size):
    from kern_b200.ops import attention as A

    torch.manual_seed(6)
    new = [5, 64, 130, 257]      # this step's rows per sequence
    prefix = [0, 17, 64, 300]    # tokens already in the cache
    lens = [n + p for n, p in zip(new, prefix)]
    seqs = len(lens)
    pool, table, ks, vs = _build_cache(cuda, seqs, lens, hk, d, page_size)
    cu = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32, device=cuda)
    total = int(cu[-1])
    wide = bf(torch.randn(total, (hq + 2 * hk) * d, device=cuda))
    q = wide[:, : hq * d]  # q as a column slice of a fused qkv buffer
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=cuda)
    out = A.paged_attention(q, pool, table, seq_lens, hq, prefill=True, cu_q=cu, max_rows=max(new))
    check_err(cuda)
    for s in range(seqs):
        lo, hi = int(cu[s]), int(cu[s + 1])
        qs = q[lo:hi].reshape(hi - lo, hq, d)
        pos = torch.arange(prefix[s], lens[s], device=cuda)
        ref = A.attention_reference(qs, ks[s], vs[s], pos)
        torch.testing.assert_close(out[lo:hi].float(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("hq,hk,d,page_size", [(32, 8, 128, 64), (8, 2, 64, 16), (4, 4, 128, 128)])
@pytest.mark.parametrize("one_launch", [True, False])
def test_ragged_attention_both_lists(cuda, hq, hk, d, page_size, one_launch):
    """Prompt chunks and decode rows in one call: the one-launch form (both kernels' CTAs side by side) and the
    two-launch form against the fp32 statement, with more decode sequences than prompt blocks and the reverse."""
    from kern_b200.ops import attention as A

    torch.manual_seed(16)
    g = hq // hk
    small = max(1, 16 // g)
    for new, prefix in (([300, 1, 1, small, 70, 1, 1, 1, 1, 1, 1, 1], [0, 500, 63, 200, 64, 1, 127, 128, 129, 900, 31, 5]),
                        ([1, 257, 130, 5, 64], [40, 300, 0, 17, 64])):
        lens = [n + p for n, p in zip(new, prefix)]
        seqs = len(lens)
        pool, table, ks, vs = _build_cache(cuda, seqs, lens, hk, d, page_size)
        cu = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32, device=cuda)
        total = int(cu[-1])
        wide = bf(torch.randn(total, (hq + 2 * hk) * d, device=cuda))
        q = wide[:, : hq * d]
        seq_lens = torch.tensor(lens, dtype=torch.int32, device=cuda)
        out = A.ragged_attention(q, pool, table, seq_lens, hq, cu, one_launch=one_launch)
        check_err(cuda)
        for s in range(seqs):
            lo, hi = int(cu[s]), int(cu[s + 1])
            qs = q[lo:hi].reshape(hi - lo, hq, d)
            pos = torch.arange(prefix[s], lens[s], device=cuda)
            ref = A.attention_reference(qs, ks[s], vs[s], pos)
            torch.testing.assert_close(out[lo:hi].float(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("hq,hk,d,rot,qk_norm", [(32, 8, 128, 128, False), (24, 4, 256, 64, True), (4, 2, 64, 64, True)])
def test_rope_kv_append(cuda, hq, hk, d, rot, qk_norm):
    from kern_b200.ops import attention as A
    from kern_b200.ops import basic

    torch.manual_seed(7)
    t, page_size, pages, theta = 50, 16, 12, 1e6
    qkv = bf(torch.randn(t, (hq + 2 * hk) * d, device=cuda))
    orig = qkv.clone()
    pool = torch.zeros(pages, 2, hk, page_size, d, dtype=torch.bfloat16, device=cuda)
    positions = torch.randint(0, 40000, (t,), device=cuda)
    slots = torch.randperm(pages * page_size, device=cuda)[:t]
    slots[5] = -1  # padding row: no append
    cos, sin = A.rope_tables(40000, rot, theta, cuda)
    qn = bf(torch.randn(d, device=cuda)) if qk_norm else None
    kn = bf(torch.randn(d, device=cuda)) if qk_norm else None
    A.rope_kv_append(qkv, pool, positions, slots, cos, sin, hq, hk, d, rot, qn, kn, 1e-6)
    check_err(cuda)
    q0 = orig[:, : hq * d].view(t, hq, d)
    k0 = orig[:, hq * d:(hq + hk) * d].view(t, hk, d)
    v0 = orig[:, (hq + hk) * d:].view(t, hk, d)
    if qk_norm:
        q0 = basic.rms_norm_reference(q0.reshape(-1, d), qn).view(t, hq, d)
        k0 = basic.rms_norm_reference(k0.reshape(-1, d), kn).view(t, hk, d)
    q_ref = A.rope_reference(q0, positions, rot, theta)
    k_ref = A.rope_reference(k0, positions, rot, theta)
    torch.testing.assert_close(qkv[:, : hq * d].view(t, hq, d).float(), q_ref, rtol=2e-2, atol=2e-2)
    for i in range(t):
        s = int(slots[i])
        if s < 0:
            continue
        pg, off = s // page_size, s % page_size
        torch.testing.assert_close(pool[pg, 0, :, off].float(), k_ref[i], rtol=2e-2, atol=2e-2)
        assert torch.equal(pool[pg, 1, :, off], v0[i])


@pytest.mark.parametrize("width", [2, 4])
def test_decode_attention_context_parallel_partials(cuda, width):
    """Positions dealt round-robin over `width` ranks (rank m holds p with p % width == m): every rank's partial over
    its own pages, written into its run of slots of one workspace, merged once, equals attention over the whole context."""
    from kern_b200.ops import attention as A

    torch.manual_seed(11)
    hq, hk, d, page = 16, 4, 128, 16
    lens = [1, 3, 64, 65, 300, 777]
    seqs = len(lens)
    q = bf(torch.randn(seqs, hq * d, device=cuda))
    ks = [bf(torch.randn(l, hk, d, device=cuda)) for l in lens]
    vs = [bf(torch.randn(l, hk, d, device=cuda)) for l in lens]
    splits = 2
    ws = A.new_partials(seqs, hq, d, width * splits, cuda)
    out = torch.empty(seqs, hq * d, dtype=torch.bfloat16, device=cuda)
    for m in range(width):
        local = [len(range(m, l, width)) for l in lens]
        pages_needed = sum(-(-n // page) for n in local) + 1
        pool = torch.zeros(pages_needed, 2, hk, page, d, dtype=torch.bfloat16, device=cuda)
        table = torch.zeros(seqs, max(1, max(-(-n // page) for n in local)), dtype=torch.int32, device=cuda)
        nxt = 1
        for s, l in enumerate(lens):
            kk, vv = ks[s][m::width], vs[s][m::width]
            for p in range(-(-local[s] // page)):
                table[s, p] = nxt
                lo, hi = p * page, min(local[s], (p + 1) * page)
                pool[nxt, 0, :, : hi - lo] = kk[lo:hi].transpose(0, 1)
                pool[nxt, 1, :, : hi - lo] = vv[lo:hi].transpose(0, 1)
                nxt += 1
        A.paged_attention(q, pool, table, torch.tensor(local, dtype=torch.int32, device=cuda), hq, out=out, splits=splits,
                          workspace=ws, partial=(m * splits, width * splits))
    A.merge_partials(ws[0], ws[1], out, seqs, hq, d, width * splits)
    check_err(cuda)
    for s, l in enumerate(lens):
        ref = A.attention_reference(q[s:s + 1].view(1, hq, d), ks[s], vs[s], torch.tensor([l - 1], device=cuda))
        torch.testing.assert_close(out[s:s + 1].float(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("heads,splits", [(16, 1), (16, 4), (40, None), (128, 2)])
def test_mla_absorbed_decode(cuda, heads, splits):
    """Latent attention decode (keys = 576-wide latent rows, values = their first 512 columns, one shared cache):
    ragged context lengths over paged latents against the fp32 statement; head counts that are not a multiple of the
    16-head CTA tile; one split, fixed splits and the automatic choice."""
    from kern_b200.ops import mla

    torch.manual_seed(heads)
    page = 32
    lens = [1, 63, 64, 65, 300, 1000]
    seqs = len(lens)
    lat = [bf(torch.randn(l, mla.DQK, device=cuda) * 0.5) for l in lens]
    pages_needed = sum(-(-l // page) for l in lens) + 1
    cache = torch.zeros(pages_needed, page, mla.DQK, dtype=torch.bfloat16, device=cuda)
    table = torch.zeros(seqs, max(-(-l // page) for l in lens), dtype=torch.int32, device=cuda)
    nxt = 1
    for s, l in enumerate(lens):
        for p in range(-(-l // page)):
            table[s, p] = nxt
            lo, hi = p * page, min(l, (p + 1) * page)
            cache[nxt, : hi - lo] = lat[s][lo:hi]
            nxt += 1
    q = bf(torch.randn(seqs, heads * mla.DQK, device=cuda) * 0.5)
    out = mla.mla_decode(q, cache, table, torch.tensor(lens, dtype=torch.int32, device=cuda), heads, splits=splits)
    check_err(cuda)
    for s in range(seqs):
        ref = mla.mla_decode_ref(q[s].view(heads, mla.DQK), lat[s], heads)
        torch.testing.assert_close(out[s].float().view(heads, mla.DV), ref, rtol=2e-2, atol=2e-2)
