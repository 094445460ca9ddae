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


def _copy_draft_runtime():
    draft = dataclasses.replace(T, name="toy-draft", layers=1)
    w = spec.random_weights(T, draft, seed=7, std=0.08, draft_from_target=True)
    for n in list(w):
        if n.startswith("model.layers.1.") and (n.endswith("o_proj.weight") or n.endswith("down_proj.weight")):
            w[n] = torch.zeros_like(w[n])
    plain = CpuRuntime(dense.build_manifest(T), weights={k: v for k, v in w.items() if not k.startswith("draft.")}, tokens=16 * 30)
    plain.once()
    rt = CpuRuntime(spec.build_manifest(T, draft, k=3), weights=w, tokens=16 * 30)
    rt.once()
    return plain, rt


@pytest.mark.parametrize("max_tokens", [13, 15])      # 13 = 1 + three whole rounds of 4; 15 ends inside the fourth round
def test_history_after_rounds_keys_the_prefix_cache(max_tokens):
    """After speculative rounds the kept prefix must be keyed by the tokens its positions really hold: a follow-up whose
    prompt is the first prompt + its output hits the cache over all whole pages of that history, and decodes the same
    tokens as a run without rounds. A request that ends inside a round keeps only the accepted positions."""
    plain, rt = _copy_draft_runtime()
    torch.manual_seed(1)
    prompt = torch.randint(1, T.vocab, (21,)).tolist()
    outs = []
    for runtime in (plain, rt):
        sch = Scheduler(Engine(runtime), chunk=32, max_seqs=3)
        first = Request(id="a", prompt=prompt, max_tokens=max_tokens)
        sch.submit(first)
        sch.run_until_idle(200)
        history = prompt + first.out
        hit = sch.prefix.lookup(history, len(history) - 1)
        assert hit is not None
        # pure KV: whole pages of the positions in the states (everything but the last emitted token)
        assert hit[0] == ((len(history) - 1) // T.page_size) * T.page_size
        second = Request(id="b", prompt=history + [3, 5], max_tokens=4)
        sch.submit(second)
        sch.run_until_idle(200)
        assert second.cached == hit[0]
        outs.append((first.out, second.out))
    assert outs[0] == outs[1]


def test_a_prefill_chunk_as_long_as_a_round_is_not_a_round():
    """A 36-token prompt with a 32-row chunk budget leaves a 4-token tail, the row count of this model's round: it must
    run through the ragged prefill program and give the plain decoder's tokens."""
    plain, rt = _copy_draft_runtime()
    torch.manual_seed(1)
    for _ in range(3):
        torch.randint(1, T.vocab, (1,))
    prompt = torch.randint(1, T.vocab, (36,)).tolist()
    outs = []
    for runtime in (plain, rt):
        sch = Scheduler(Engine(runtime), chunk=32, max_seqs=3, prefix_cache=False)
        r = Request(id="a", prompt=prompt, max_tokens=5)
        sch.submit(r)
        sch.run_until_idle(100)
        outs.append(r.out)
    assert outs[0] == outs[1]
