"""Speculative rounds on a GPU: one captured graph per round; emitted tokens equal the target's plain greedy decoding."""
import dataclasses

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("copy_draft", [False, True])
def test_rounds_equal_plain_greedy_on_gpu(cuda, copy_draft):
    from kern_b200.engine import Engine
    from kern_b200.models import dense, spec
    from kern_b200.runtime import Runtime
    from kern_b200.serve.scheduler import Request, Scheduler

    T = dataclasses.replace(dense.TINY, max_tokens=256, max_seqs=8)
    draft = dataclasses.replace(T, name="tiny-draft", layers=1) if copy_draft else None
    w = spec.random_weights(T, draft, seed=3, std=0.05, draft_from_target=copy_draft)
    if copy_draft:
        for n in list(w):
            if n.startswith("model.layers.1.") and (n.endswith("o_proj.weight") or n.endswith("down_proj.weight")):
                w[n] = torch.zeros_like(w[n])
    outs = []
    for doc, names in ((dense.build_manifest(T), [k for k in w if not k.startswith("draft.")]), (spec.build_manifest(T, draft, k=3), list(w))):
        rt = Runtime(doc, tokens=T.page_size * 64)
        rt.load_tensors(lambda name: w[name].cuda())
        rt.once()
        sch = Scheduler(Engine(rt), chunk=128, max_seqs=4)
        torch.manual_seed(0)
        prompts = [torch.randint(1, T.vocab, (n,)).tolist() for n in (40, 7, 90)]
        reqs = [Request(id=str(i), prompt=p, max_tokens=10) for i, p in enumerate(prompts)]
        for r in reqs:
            sch.submit(r)
        sch.run_until_idle(400)
        rt.check_error()
        assert sch.idle()
        outs.append(([r.out for r in reqs], sch.stats, rt.graphs))
    assert outs[0][0] == outs[1][0]
    assert outs[1][1].proposed > 0 and outs[1][2] >= 1
    if copy_draft:
        assert outs[1][1].accepted == outs[1][1].proposed
