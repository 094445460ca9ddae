"""The CPU toy decoder: verify the toy manifest, execute it on the host-memory executor with paged KV,
and check logits and greedy tokens against the PyTorch fp32 oracle.

vocab 256, hidden 64, 2 layers, 4 Q / 2 KV heads, head_dim 16, SwiGLU 128, RMSNorm eps 1e-6, RoPE theta
10000, bf16 weights ~ N(0, 0.02) from seed 0; batch of 4 prompts of 16 uniform-random token ids, 8 greedy
output tokens, page size 16."""
import numpy as np
import torch

from kern_b200.cpu import CpuRuntime
from kern_b200.engine import Engine
from kern_b200.models import dense
from kern_b200.runtime import verify


def _setup():
    cfg = dense.TOY
    weights = dense.random_weights(cfg, seed=0, std=0.02)
    doc = dense.build_manifest(cfg)
    m, errs = verify(doc)
    assert m is not None, errs[:5]
    rt = CpuRuntime(doc, weights=weights, tokens=cfg.page_size * 16)
    rt.once()
    return cfg, weights, rt


def test_toy_manifest_logits_and_tokens_match_fp32_oracle():
    cfg, weights, rt = _setup()
    eng = Engine(rt)
    oracle = dense.DenseOracle(cfg, weights)               # fp32 math over the bf16 checkpoint
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, cfg.vocab, 16).tolist() for _ in range(4)]
    seqs = [eng.open(16 + 8) for _ in prompts]
    caches = [oracle.new_cache() for _ in prompts]
    first = eng.step(list(zip(seqs, prompts)))
    logits = rt.tensor("logits")[:4].float()
    refs = torch.stack([oracle.forward(p, c)[-1] for p, c in zip(prompts, caches)])
    assert torch.allclose(logits, refs, atol=3e-3, rtol=3e-2), float((logits - refs).abs().max())
    outs = [[f[0]] for f in first]
    ref_outs = [[int(r.argmax())] for r in refs]
    for _ in range(7):
        nxt = eng.step([(s, [o[-1]]) for s, o in zip(seqs, outs)])
        logits = rt.tensor("logits")[:4].float()
        refs = torch.stack([oracle.forward([o[-1]], c)[-1] for o, c in zip(ref_outs, caches)])
        for o, n, ro, r, lg in zip(outs, nxt, ref_outs, refs, logits):
            o.append(n[0])
            ro.append(int(r.argmax()))
            if o[:-1] == ro[:-1]:        # same history: same logits up to bf16 rounding
                assert torch.allclose(lg, r, atol=3e-3, rtol=3e-2)
    # greedy tokens agree unless the oracle's top-2 margin is inside bf16 rounding (a near tie)
    agree = sum(a == b for o, ro in zip(outs, ref_outs) for a, b in zip(o, ro))
    assert agree >= 28, (outs, ref_outs)
    for s in seqs:
        eng.close(s)
    assert eng.pool.free_pages == eng.pool.total_pages


def test_toy_chunked_prefill_and_page_boundaries():
    cfg, weights, rt = _setup()
    eng = Engine(rt)
    rng = np.random.default_rng(1)
    prompt = rng.integers(0, cfg.vocab, 33).tolist()      # crosses two page boundaries
    whole = eng.generate(prompt, 6)
    chunked = eng.generate(prompt, 6, chunk=7)
    assert whole == chunked
