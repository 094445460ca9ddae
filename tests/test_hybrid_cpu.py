"""The hybrid (GDN + gated attention) manifest through the CPU executor against the PyTorch oracle:
ragged prefill, decode steps, per-sequence state lines, checkpoint/restore of a state slot."""
import torch

from kern_b200.cpu import CpuRuntime
from kern_b200.engine import Engine
from kern_b200.models import hybrid
from kern_b200.runtime import verify


def make(cfg=hybrid.TOY_HYBRID, slots=6):
    w = hybrid.random_weights(cfg, seed=3, std=0.08)
    rt = CpuRuntime(hybrid.build_manifest(cfg), weights=w, tokens=cfg.page_size * 24, slots=slots)
    rt.once()
    return cfg, w, rt, Engine(rt), hybrid.HybridOracle(cfg, w)


def test_manifest_verifies_and_projects_both_tables():
    cfg = hybrid.TOY_HYBRID
    m, diags = verify(hybrid.build_manifest(cfg))
    assert m is not None, diags
    import json
    p = json.loads(m.protocol(sampled=False))
    assert [t["name"] for t in p["page_tables"]] == ["block_table"]
    assert [(t["name"], t["lines"]) for t in p["line_tables"]] == [("lines", 1)]
    m27, diags = verify(hybrid.build_manifest(hybrid.HYBRID_27B))
    assert m27 is not None, diags[:5]


def test_prefill_and_decode_match_oracle():
    cfg, w, rt, eng, oracle = make()
    torch.manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (21, 3, 9)]
    seqs = [eng.open(40) for _ in prompts]
    assert sorted(s.lease.slot for s in seqs) == [1, 2, 3]
    caches = [oracle.new_cache() for _ in prompts]
    first = eng.step(list(zip(seqs, prompts)))
    logits = rt.tensor("logits")[:3].float()
    worst = 0.0
    for i, (p, c) in enumerate(zip(prompts, caches)):
        ref = oracle.forward(p, c)[-1]
        worst = max(worst, float((logits[i] - ref).abs().max()))
    toks = [f[0] for f in first]
    for _ in range(5):
        refs = [oracle.forward([t], c)[-1] for t, c in zip(toks, caches)]
        nxt = eng.step([(s, [t]) for s, t in zip(seqs, toks)])
        logits = rt.tensor("logits")[:3].float()
        for i in range(3):
            worst = max(worst, float((logits[i] - refs[i]).abs().max()))
        toks = [n[0] for n in nxt]
    assert worst < 0.12, worst


def test_chunked_rule_statement_through_the_manifest():
    """GDN heads of 128: the prefill program runs the chunked (WY) pair of launches; prompts longer than one 64-token
    chunk, then decode steps through the fused step, against the oracle's token-by-token rule."""
    cfg, w, rt, eng, oracle = make(hybrid.TINY_HYBRID_K128)
    entries = {l["entry"] for op in hybrid.build_manifest(cfg)["ops"].values() for l in op.get("impl", {}).get("launches", [])}
    assert {"kern_gdn_chunk_prep_k128_v128", "kern_gdn_chunk_rule_k128_v128", "kern_gdn_step_k128_v128"} <= entries
    torch.manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (150, 5)]
    seqs = [eng.open(160), eng.open(16)]
    caches = [oracle.new_cache() for _ in prompts]
    first = eng.step(list(zip(seqs, prompts)))
    logits = rt.tensor("logits")[:2].float()
    worst = max(float((logits[i] - oracle.forward(p, c)[-1]).abs().max()) for i, (p, c) in enumerate(zip(prompts, caches)))
    toks = [f[0] for f in first]
    for _ in range(2):
        refs = [oracle.forward([t], c)[-1] for t, c in zip(toks, caches)]
        nxt = eng.step([(s, [t]) for s, t in zip(seqs, toks)])
        logits = rt.tensor("logits")[:2].float()
        worst = max(worst, max(float((logits[i] - refs[i]).abs().max()) for i in range(2)))
        toks = [n[0] for n in nxt]
    assert worst < 0.2, worst


def test_chunked_prefill_equals_one_shot():
    cfg, w, rt, eng, oracle = make()
    torch.manual_seed(1)
    prompt = torch.randint(0, cfg.vocab, (30,)).tolist()
    a, b = eng.open(40), eng.open(40)
    one = eng.step([(a, prompt)])
    la = rt.tensor("logits")[0].float().clone()
    eng.step([(b, prompt[:11])])
    eng.step([(b, prompt[11:12])])
    two = eng.step([(b, prompt[12:])])
    lb = rt.tensor("logits")[0].float()
    assert float((la - lb).abs().max()) < 0.05
    assert one == two


def test_checkpoint_restores_state_slot():
    cfg, w, rt, eng, oracle = make()
    torch.manual_seed(2)
    prompt = torch.randint(0, cfg.vocab, (16,)).tolist()
    s = eng.open(40)
    t0 = eng.step([(s, prompt)])[0]
    ck, copies = eng.pool.checkpoint(s.lease, 16)
    rt.run_copies(copies)
    # the original runs on; the restored copy must replay the same continuation from the snapshot
    cont = [t0[0]]
    for _ in range(4):
        cont.append(eng.step([(s, [cont[-1]])])[0][0])
    lease, copies = eng.pool.restore(ck, 16, 40)
    rt.run_copies(copies)
    from kern_b200.engine import Sequence, Sampling
    r = Sequence(lease=lease, sampling=Sampling())
    r.length = 16
    again = [t0[0]]
    for _ in range(4):
        again.append(eng.step([(r, [again[-1]])])[0][0])
    assert again == cont
