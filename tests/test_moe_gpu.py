"""MoE routing, planning, routed tcgen05 GEMMs and combine against the PyTorch fp32 statement."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def bf(x):
    return x.to(torch.bfloat16)


@pytest.mark.parametrize("mode,bias", [("sigmoid", False), ("sigmoid", True), ("softmax", False)])
@pytest.mark.parametrize("t,e,k", [(1, 8, 2), (37, 64, 6), (300, 384, 8)])
def test_route(cuda, t, e, k, mode, bias):
    from kern_b200.ops import moe

    torch.manual_seed(t + e)
    logits = torch.randn(t, e, device=cuda) * 2
    b = torch.randn(e, device=cuda) * 0.5 if bias else None
    ids, w = moe.route(logits, k, b, mode, True, 2.5)
    rid, rw = moe.route_reference(logits, k, b, mode, True, 2.5)
    torch.cuda.synchronize()
    assert torch.equal(ids.sort(-1).values, rid.sort(-1).values)
    order, rorder = ids.argsort(-1), rid.argsort(-1)
    torch.testing.assert_close(torch.gather(w, 1, order), torch.gather(rw, 1, rorder), rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("t,e,k,e_lo,e_n", [(5, 8, 2, 0, 8), (200, 32, 4, 8, 16), (1000, 16, 2, 0, 16)])
def test_plan_is_a_partition(cuda, t, e, k, e_lo, e_n):
    from kern_b200.ops import moe
    from kern_b200.ops.launcher import Kernels

    torch.manual_seed(1)
    ids = torch.stack([torch.randperm(e, device=cuda)[:k] for _ in range(t)]).int()
    pl = moe.plan(ids, e_n, e_lo)
    torch.cuda.synchronize()
    Kernels.get(cuda).check_error()
    flat, perm = ids.flatten().cpu(), pl["perm"].cpu()
    offsets = pl["offsets"].cpu()
    local = (flat >= e_lo) & (flat < e_lo + e_n)
    assert bool((perm[~local] == -1).all())
    assert sorted(perm[local].tolist()) == list(range(int(local.sum())))
    assert int(pl["rows"]) == int(local.sum())
    for x in range(e_n):
        mine = perm[flat == x + e_lo]
        assert sorted(mine.tolist()) == list(range(int(offsets[x]), int(offsets[x + 1])))     # an expert's rows are its own run
    n = int(pl["tile_count"])
    covered = []
    for ex, r0, nr, _ in pl["tiles"][:n].cpu().tolist():
        assert 0 < nr <= 128 and int(offsets[ex]) <= r0 and r0 + nr <= int(offsets[ex + 1])
        covered += list(range(r0, r0 + nr))
    assert covered == list(range(int(local.sum())))


@pytest.mark.parametrize("t,h,inter,e,k", [(3, 256, 128, 8, 2), (150, 512, 256, 16, 4), (700, 1024, 512, 32, 8)])
def test_moe_layer(cuda, t, h, inter, e, k):
    from kern_b200.ops import moe
    from kern_b200.ops.launcher import Kernels

    torch.manual_seed(t)
    x = bf(torch.randn(t, h, device=cuda))
    wr = bf(torch.randn(e, h, device=cuda) * 0.1)
    w1 = bf(torch.randn(e, 2 * inter, h, device=cuda) * h ** -0.5)
    w2 = bf(torch.randn(e, h, inter, device=cuda) * inter ** -0.5)
    shared = bf(torch.randn(t, h, device=cuda))
    got = moe.moe_layer(x, wr, w1, w2, k, scale=1.5, shared=shared)
    torch.cuda.synchronize()
    Kernels.get(cuda).check_error()
    ref = moe.moe_reference(x, wr, w1, w2, k, scale=1.5, shared=shared)
    torch.testing.assert_close(got.float(), ref, rtol=3e-2, atol=3e-2)


def test_moe_expert_parallel_shares_sum_to_the_whole(cuda):
    from kern_b200.ops import moe

    torch.manual_seed(9)
    t, h, inter, e, k = 90, 256, 128, 16, 4
    x = bf(torch.randn(t, h, device=cuda))
    wr = bf(torch.randn(e, h, device=cuda) * 0.1)
    w1 = bf(torch.randn(e, 2 * inter, h, device=cuda) * h ** -0.5)
    w2 = bf(torch.randn(e, h, inter, device=cuda) * inter ** -0.5)
    whole = moe.moe_reference(x, wr, w1, w2, k)
    parts = sum(moe.moe_layer(x, wr, w1[lo:lo + 4].contiguous(), w2[lo:lo + 4].contiguous(), k, e_lo=lo).float()
                for lo in range(0, e, 4))
    torch.testing.assert_close(parts, whole, rtol=4e-2, atol=4e-2)


def test_moe_decoder_end_to_end(cuda):
    """The MoE decoder's manifest on the native runtime: prefill + graph-replayed decode against the fp32 oracle."""
    from kern_b200.engine import Engine
    from kern_b200.models import moe
    from kern_b200.runtime import Runtime

    cfg = moe.TINY_MOE
    w = moe.random_weights(cfg, seed=1, std=0.05)
    rt = Runtime(moe.build_manifest(cfg), tokens=cfg.page_size * 64)
    rt.load_tensors(lambda name: w[name].cuda())
    rt.once()
    eng, oracle = Engine(rt), moe.MoeOracle(cfg, w, device="cuda")
    torch.manual_seed(0)
    prompts = [torch.randint(1, cfg.vocab, (n,)).tolist() for n in (150, 9)]
    seqs = [eng.open(200) for _ in prompts]
    caches = [oracle.new_cache() for _ in prompts]
    first = eng.step(list(zip(seqs, prompts)))
    logits = rt.tensor("logits")[:2].float()
    diffs = [(logits[i] - oracle.forward(p, c)[-1]).abs() for i, (p, c) in enumerate(zip(prompts, caches))]
    toks = [f[0] for f in first]
    for _ in range(4):
        refs = [oracle.forward([t], c)[-1] for t, c in zip(toks, caches)]
        nxt = eng.step([(s, [t]) for s, t in zip(seqs, toks)])
        logits = rt.tensor("logits")[:2].float()
        diffs += [(logits[i] - refs[i]).abs() for i in range(2)]
        toks = [n[0] for n in nxt]
    rt.check_error()
    assert max(float(d.max()) for d in diffs) < 0.3 and max(float(d.mean()) for d in diffs) < 0.05
    assert rt.graphs >= 1


def test_moe_decoder_with_block_scaled_experts(cuda):
    """The `mx_experts` decoder on the GPU (MXFP4 expert weights through the TMA unpacking type, MXFP8 activations, scales
    through TMEM) against the same manifest on the host-memory executor, which states every kernel in PyTorch."""
    import dataclasses

    from kern_b200.cpu import CpuRuntime
    from kern_b200.engine import Engine
    from kern_b200.models import moe
    from kern_b200.runtime import Runtime

    cfg = dataclasses.replace(moe.TINY_MOE, name="tiny-moe-mx", mx_experts=True, moe_intermediate=128, experts=8, top_k=2)
    doc = moe.build_manifest(cfg)
    w = moe.mx_checkpoint(cfg, moe.random_weights(cfg, seed=3, std=0.05))
    rt = Runtime(doc, tokens=cfg.page_size * 32)
    rt.load_tensors(lambda name: w[name].cuda())
    rt.once()
    ref_rt = CpuRuntime(doc, weights=w, tokens=cfg.page_size * 32)
    ref_rt.once()
    eng, ref = Engine(rt), Engine(ref_rt)
    torch.manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (37, 5)]
    seqs, rseqs = [eng.open(60) for _ in prompts], [ref.open(60) for _ in prompts]
    a = eng.step(list(zip(seqs, prompts)))
    b = ref.step(list(zip(rseqs, prompts)))
    rt.check_error()
    got, want = rt.tensor("logits")[:2].float().cpu(), ref_rt.tensor("logits")[:2].float()
    assert float((got - want).abs().max()) < 0.08 * float(want.abs().max()) + 0.02
    for _ in range(3):
        toks = [t[0] for t in b]
        a = eng.step([(s, [t]) for s, t in zip(seqs, toks)])
        b = ref.step([(s, [t]) for s, t in zip(rseqs, toks)])
        rt.check_error()
        got, want = rt.tensor("logits")[:2].float().cpu(), ref_rt.tensor("logits")[:2].float()
        assert float((got - want).abs().max()) < 0.08 * float(want.abs().max()) + 0.02
