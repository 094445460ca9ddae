"""Speculative rounds on the CPU executor: a round's emitted tokens must equal plain greedy decoding of the target,
whatever the draft proposes (a random draft: mostly 1 token per round; a draft that copies the target: all R)."""
import dataclasses
import json

import pytest
import torch

from kern_b200.cpu import CpuRuntime
from kern_b200.engine import Engine
from kern_b200.models import dense, spec
from kern_b200.runtime import verify
from kern_b200.serve.scheduler import Request, Scheduler

T = dataclasses.replace(dense.TOY, max_tokens=64, max_seqs=4)


def test_manifest_and_protocol():
    m, d = verify(spec.build_manifest(T, k=3))
    assert m is not None, d[:5]
    p = json.loads(m.protocol(sampled=False))
    fw = {f["name"]: f for f in p["forwards"]}
    assert fw["round"]["rows"] == 4 and fw["round"]["emits"] == "round_tokens" and fw["round"]["count"] == "round_count"
    assert fw["decode"]["rows"] == 1 and fw["decode"]["count"] is None


@pytest.mark.parametrize("copy_draft", [False, True])
def test_rounds_equal_plain_greedy(copy_draft):
    draft = dataclasses.replace(T, name="toy-draft", layers=1) if copy_draft else None
    w = spec.random_weights(T, draft, seed=7, std=0.08, draft_from_target=copy_draft)
    if copy_draft:       # a one-layer copy of a two-layer target would rarely agree: make the target's 2nd layer a no-op
        for n in list(w):
            if n.startswith("model.layers.1.") and (n.endswith("o_proj.weight") or n.endswith("down_proj.weight")):
                w[n] = torch.zeros_like(w[n])
    plain = CpuRuntime(dense.build_manifest(T), weights={k: v for k, v in w.items() if not k.startswith("draft.")}, tokens=16 * 30)
    plain.once()
    rt = CpuRuntime(spec.build_manifest(T, draft, k=3), weights=w, tokens=16 * 30)
    rt.once()
    torch.manual_seed(0)
    prompts = [torch.randint(1, T.vocab, (n,)).tolist() for n in (11, 25, 6)]
    outs = []
    for runtime in (plain, rt):
        sch = Scheduler(Engine(runtime), chunk=32, max_seqs=3)
        reqs = [Request(id=str(i), prompt=p, max_tokens=9) for i, p in enumerate(prompts)]
        for r in reqs:
            sch.submit(r)
        sch.run_until_idle(400)
        assert sch.idle()
        outs.append(([r.out for r in reqs], sch.stats))
    assert outs[0][0] == outs[1][0]
    st = outs[1][1]
    assert st.proposed > 0
    if copy_draft:
        assert st.accepted == st.proposed            # every proposal is the target's own token
    assert outs[1][1].steps < outs[0][1].steps or not copy_draft
