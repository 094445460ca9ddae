"""The exact integer model served through the scheduler on the CPU executor: every emitted token must equal the
host twin's, across chunked prefill, batching, prefix-cache hits, eviction and (stateful) slot snapshots."""
import random

import pytest

from kern_b200.cpu import CpuRuntime
from kern_b200.engine import Engine
from kern_b200.models import toy_int
from kern_b200.runtime import verify
from kern_b200.serve.scheduler import Request, Scheduler


@pytest.mark.parametrize("lined", [False, True])
def test_manifests_verify(lined):
    m, diags = verify(toy_int.build_manifest(lined))
    assert m is not None, diags


def serve(lined, prompts, max_tokens, pages=40, chunk=24, max_seqs=4):
    rt = CpuRuntime(toy_int.build_manifest(lined), tokens=16 * pages, slots=12 if lined else 0)
    sch = Scheduler(Engine(rt), chunk=chunk, max_seqs=max_seqs)
    waves = prompts if prompts and isinstance(prompts[0][0], list) else [prompts]
    reqs = []
    for wave in waves:          # a later wave finds what the earlier ones left in the prefix cache
        if callable(wave):
            wave = wave(reqs)
        new = [Request(id=str(len(reqs) + i), prompt=p, max_tokens=max_tokens, stop_ids=(toy_int.EOS,)) for i, p in enumerate(wave)]
        reqs += new
        for r in new:
            sch.submit(r)
        for _ in range(2000):
            if sch.idle():
                break
            sch.step()
        assert sch.idle()
    return reqs, sch


@pytest.mark.parametrize("lined", [False, True])
def test_served_tokens_equal_the_twin(lined):
    rng = random.Random(7)
    base = [rng.randrange(256) for _ in range(70)]
    prompts = [[rng.randrange(256) for _ in range(rng.randint(1, 60))] for _ in range(6)]
    # the next turn of a conversation (prompt + answer + more) and shared prefixes -> cache hits
    turn = lambda reqs: [reqs[0].prompt + [t for t in reqs[0].out if t != toy_int.EOS] + [7, 8]]
    again = lambda reqs: turn(reqs) + [base[:50] + [1, 2, 3], base[:33], base]
    reqs, sch = serve(lined, [prompts + [base[:50]], again], 12)
    for r in reqs:
        want = toy_int.generate(r.prompt, 12, lined)
        got = [t for t in r.out if t != toy_int.EOS]
        assert got == want, (r.id, len(r.prompt))
    assert sch.stats.prefix_hits >= 1


@pytest.mark.parametrize("lined", [False, True])
def test_eviction_under_pressure_keeps_answers_exact(lined):
    rng = random.Random(11)
    prompts = [[rng.randrange(256) for _ in range(rng.randint(20, 90))] for _ in range(14)]
    reqs, sch = serve(lined, prompts, 8, pages=16, chunk=32, max_seqs=3)
    for r in reqs:
        assert [t for t in r.out if t != toy_int.EOS] == toy_int.generate(r.prompt, 8, lined)
    assert sch.stats.evictions >= 1


def test_per_sequence_prefill_that_emits_nothing():
    """A package whose ragged program takes one sequence per call and emits nothing (the reference's paged shape): the
    scheduler runs a ragged call per admitted prompt, holds back the prompt's last token for the first step, and every
    emitted token still equals the twin's — with chunking, several requests at once and a prefix-cache hit."""
    doc = toy_int.build_manifest(False, per_sequence_prefill=True)
    m, diags = verify(doc)
    assert m is not None, diags
    rt = CpuRuntime(doc, tokens=16 * 40)
    sch = Scheduler(Engine(rt), chunk=24, max_seqs=4)
    assert sch.split and not sch.prefill_emits
    rng = random.Random(5)
    prompts = [[rng.randrange(256) for _ in range(n)] for n in (1, 7, 30, 53, 16, 17)]
    reqs = [Request(id=str(i), prompt=p, max_tokens=6, stop_ids=(toy_int.EOS,)) for i, p in enumerate(prompts)]
    for r in reqs:
        sch.submit(r)
    sch.run_until_idle(500)
    assert sch.idle()
    for r in reqs:
        want = toy_int.generate(r.prompt, 6)
        assert r.out[:len(want)] == want and len(r.out) in (len(want), len(want) + 1), (r.id, r.out, want)
    again = Request(id="again", prompt=prompts[3] + reqs[3].out[:2], max_tokens=3, stop_ids=(toy_int.EOS,))
    sch.submit(again)
    sch.run_until_idle(100)
    assert again.cached >= 48 and again.out[:3][:len(toy_int.generate(again.prompt, 3))] == toy_int.generate(again.prompt, 3)
