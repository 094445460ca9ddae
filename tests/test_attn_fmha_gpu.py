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


@pytest.mark.parametrize("tile", [64, 128])
@pytest.mark.parametrize("hq,hk,page_size", [(8, 2, 64), (4, 4, 16), (16, 2, 128), (4, 1, 64)])
@pytest.mark.parametrize("new,prefix", [([128], [0]), ([5, 64, 130, 257], [0, 17, 64, 300]), ([700, 33], [1000, 0])])
def test_fmha_prefill_matches_fp32(cuda, hq, hk, page_size, new, prefix, tile):
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
    out = A.fmha_prefill(q, pool, table, seq_lens, hq, cu, tile=tile)
    torch.cuda.synchronize()
    Kernels.get(cuda).check_error()
    for s in range(len(lens)):
        lo, hi = int(cu[s]), int(cu[s + 1])
        qs = q[lo:hi].reshape(hi - lo, hq, d)
        pos = torch.arange(prefix[s], lens[s], device=cuda)
        ref = A.attention_reference(qs, ks[s], vs[s], pos)
        torch.testing.assert_close(out[lo:hi].float(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("tile", [64, 128])
@pytest.mark.parametrize("hq,hk", [(8, 2), (32, 8)])
def test_fmha_prefill_rescales_rows_whose_maximum_moves_late(cuda, hq, hk, tile):
    """Keys that grow with their position: the running maximum of a row outgrows its lazy reference by more than 2^8 at
    some later KV tile, at a different tile for different rows of a warp, so the pass that rescales O in TMEM runs with
    only some of the warp's rows moving (the pass itself must run for the whole warp: `tcgen05.ld` / `st` are
    warp-wide instructions)."""
    from kern_b200.ops import attention as A
    from kern_b200.ops.launcher import Kernels

    d, page_size = 128, 64
    torch.manual_seed(41)
    new, prefix = [384, 200], [512, 0]
    lens = [n + p for n, p in zip(new, prefix)]
    pool, table, ks, vs = _build_cache(cuda, lens, hk, d, page_size)
    # scale every key by a ramp over its position: 1x at the start, 12x at the end of its sequence
    for s, l in enumerate(lens):
        ramp = torch.linspace(1.0, 12.0, l, device=cuda).view(l, 1, 1)
        knew = bf(ks[s].float() * ramp)
        ks[s] = knew
        for p in range((l + page_size - 1) // page_size):
            lo, hi = p * page_size, min(l, (p + 1) * page_size)
            pool[int(table[s, p]), 0, :, : hi - lo] = knew[lo:hi].transpose(0, 1)
    cu = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32, device=cuda)
    q = bf(torch.randn(int(cu[-1]), hq * d, device=cuda))
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=cuda)
    # the premise: for the first 32 query rows of sequence 0 (one warp's rows; all of the 512-token prefix is visible to
    # them), the KV tile at which the running maximum first exceeds the first tile's by 8 (log2 domain) differs by row
    s0 = (q[:32].view(32, hq, d)[:, 0].float() @ ks[0][:512, 0].float().T) * (d ** -0.5) * 1.4427
    run = torch.cummax(s0.view(32, 4, 128).max(-1).values, dim=1).values
    first_move = ((run - run[:, :1]) > 8).float().argmax(1)                 # 0: never within these four tiles
    assert len(set(first_move.tolist())) >= 2, first_move.tolist()
    out = A.fmha_prefill(q, pool, table, seq_lens, hq, cu, tile=tile)
    torch.cuda.synchronize()
    Kernels.get(cuda).check_error()
    for s in range(len(lens)):
        lo, hi = int(cu[s]), int(cu[s + 1])
        qs = q[lo:hi].reshape(hi - lo, hq, d)
        pos = torch.arange(prefix[s], lens[s], device=cuda)
        ref = A.attention_reference(qs, ks[s], vs[s], pos)
        torch.testing.assert_close(out[lo:hi].float(), ref, rtol=3e-2, atol=3e-2)


def test_dense_decoder_with_head_dim_128_uses_the_tcgen05_prefill_kernel(cuda, monkeypatch):
    """A small dense decoder with head_dim 128 through the runtime and the engine: ragged calls that mix prompt chunks
    (the tcgen05 kernel's list) with decode rows (the token-parallel kernel's list), against the fp32 oracle."""
    import dataclasses

    from kern_b200.engine import Engine
    from kern_b200.models import dense
    from kern_b200.runtime import Runtime

    monkeypatch.setenv("KERN_B200_FMHA", "1")
    cfg = dataclasses.replace(dense.TINY, name="tiny-d128", head_dim=128, heads=8, kv_heads=2, hidden=256, max_tokens=512,
                              max_context=512, page_size=64)
    doc = dense.build_manifest(cfg)
    assert doc["ops"]["attn_prefill"]["impl"]["launches"][0]["entry"] == "kern_attn_ragged_fmha_d128"
    w = dense.random_weights(cfg, seed=0, std=0.05)
    rt = Runtime(doc, tokens=cfg.page_size * 40)
    rt.load_tensors(lambda name: w[name].cuda())
    rt.once()
    eng = Engine(rt)
    oracle = dense.DenseOracle(cfg, w, device="cuda")
    torch.manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (200, 3, 70)]
    seqs = [eng.open(len(p) + 200) for p in prompts]
    caches = [oracle.new_cache() for _ in prompts]
    first = eng.step(list(zip(seqs, prompts)))
    rt.check_error()
    logits = rt.tensor("logits")[:3].float()
    for i, (p, c) in enumerate(zip(prompts, caches)):
        assert float((logits[i] - oracle.forward(p, c)[-1]).abs().max()) < 0.12
    # a mixed call: two sequences decode one row each while the third is fed a 150-token chunk
    toks = [f[0] for f in first]
    chunk = torch.randint(0, cfg.vocab, (150,)).tolist()
    feeds = [[toks[0]], [toks[1]], chunk]
    refs = [oracle.forward(f, c)[-1] for f, c in zip(feeds, caches)]
    eng.step(list(zip(seqs, feeds)))
    rt.check_error()
    logits = rt.tensor("logits")[:3].float()
    for i in range(3):
        assert float((logits[i] - refs[i]).abs().max()) < 0.12


@pytest.mark.parametrize("hq,hk,page_size", [(32, 8, 64), (8, 2, 16), (4, 4, 128)])
def test_ragged_attention_with_tcgen05_prompt_rows(cuda, hq, hk, page_size):
    """Prompt chunks (the tcgen05 kernel's CTAs) and decode rows (the token-parallel kernel's CTAs) in one launch,
    against the fp32 statement; more decode sequences than prompt blocks and the reverse."""
    from kern_b200.ops import attention as A
    from kern_b200.ops.launcher import Kernels

    d = 128
    torch.manual_seed(17)
    small = max(1, 16 // (hq // hk))
    for new, prefix in (([300, 1, 1, small, 70, 1, 1, 1, 1, 1, 1, 1], [0, 500, 63, 200, 64, 1, 127, 128, 129, 900, 31, 5]),
                        ([1, 257, 130, 5, 64], [40, 300, 0, 17, 64])):
        lens = [n + p for n, p in zip(new, prefix)]
        pool, table, ks, vs = _build_cache(cuda, lens, hk, d, page_size)
        cu = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32, device=cuda)
        wide = bf(torch.randn(int(cu[-1]), (hq + 2 * hk) * d, device=cuda))
        q = wide[:, : hq * d]
        seq_lens = torch.tensor(lens, dtype=torch.int32, device=cuda)
        out = A.ragged_attention(q, pool, table, seq_lens, hq, cu, fmha=True)
        torch.cuda.synchronize()
        Kernels.get(cuda).check_error()
        for s in range(len(lens)):
            lo, hi = int(cu[s]), int(cu[s + 1])
            qs = q[lo:hi].reshape(hi - lo, hq, d)
            pos = torch.arange(prefix[s], lens[s], device=cuda)
            ref = A.attention_reference(qs, ks[s], vs[s], pos)
            torch.testing.assert_close(out[lo:hi].float(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("two_per_sm", [True, False])
@pytest.mark.parametrize("heads,new,prefix", [(4, [128], [0]), (16, [5, 64, 130, 257], [0, 17, 64, 300]), (2, [700, 33], [1000, 0]), (8, [1, 200], [0, 0])])
def test_fmha_context_qk192_v128_matches_fp32(cuda, heads, new, prefix, two_per_sm):
    """Context attention with a 192-wide q.k and 128-wide values over contiguous ragged K / V (the un-absorbed prefill of a
    latent-attention layer): ragged lengths, prefixes, tiles that run into the next sequence's rows and past the tensor's end."""
    from kern_b200.ops import attention as A
    from kern_b200.ops.launcher import Kernels

    torch.manual_seed(23 + heads)
    lens = [n + p for n, p in zip(new, prefix)]
    cu_q = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32, device=cuda)
    cu_k = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=cuda)
    q = bf(torch.randn(int(cu_q[-1]), heads * 192, device=cuda))
    k = bf(torch.randn(int(cu_k[-1]), heads * 192, device=cuda) * 0.6)
    v = bf(torch.randn(int(cu_k[-1]), heads * 128, device=cuda) * 0.5)
    # keys that grow along one sequence: rows whose maximum moves at a later tile (the O rescale pass)
    k[: lens[0]] = bf(k[: lens[0]].float() * torch.linspace(1.0, 6.0, lens[0], device=cuda)[:, None])
    out = A.fmha_context(q, k, v, cu_q, cu_k, heads, two_per_sm=two_per_sm)
    torch.cuda.synchronize()
    Kernels.get(cuda).check_error()
    ref = A.context_reference(q, k, v, cu_q, cu_k, heads)
    torch.testing.assert_close(out.float(), ref, rtol=3e-2, atol=3e-2)
