"""The MoE decoder's manifest through the CPU executor against the fp32 oracle."""
import torch

from kern_b200.cpu import CpuRuntime
from kern_b200.engine import Engine
from kern_b200.models import moe
from kern_b200.runtime import verify


def test_manifest_verifies_at_full_size():
    for cfg in (moe.TOY_MOE, moe.MOE_30B):
        m, d = verify(moe.build_manifest(cfg))
        assert m is not None, d[:5]


def test_prefill_and_decode_match_oracle():
    cfg = moe.TOY_MOE
    w = moe.random_weights(cfg, seed=2, std=0.08)
    rt = CpuRuntime(moe.build_manifest(cfg), weights=w, tokens=16 * 24)
    rt.once()
    eng, oracle = Engine(rt), moe.MoeOracle(cfg, w)
    torch.manual_seed(0)
    prompts = [torch.randint(1, cfg.vocab, (n,)).tolist() for n in (17, 5)]
    seqs = [eng.open(40) for _ in prompts]
    caches = [oracle.new_cache() for _ in prompts]
    first = eng.step(list(zip(seqs, prompts)))
    logits = rt.tensor("logits")[:2].float()
    worst = max(float((logits[i] - oracle.forward(p, c)[-1]).abs().max()) for i, (p, c) in enumerate(zip(prompts, caches)))
    toks = [f[0] for f in first]
    for _ in range(4):
        refs = [oracle.forward([t], c)[-1] for t, c in zip(toks, caches)]
        nxt = eng.step([(s, [t]) for s, t in zip(seqs, toks)])
        logits = rt.tensor("logits")[:2].float()
        worst = max([worst] + [float((logits[i] - refs[i]).abs().max()) for i in range(2)])
        toks = [n[0] for n in nxt]
    assert worst < 0.15, worst
