"""Pooled tier: key chains, the memory and SSD stores, and two engines sharing one store — the second serves a prompt
from pages the first computed, and the exact integer model proves the pages are the right ones."""
import random

import pytest

from kern_b200.cpu import CpuRuntime
from kern_b200.engine import Engine
from kern_b200.models import toy_int
from kern_b200.serve import pooled
from kern_b200.serve.scheduler import Request, Scheduler


def test_key_chain_names_prefixes():
    a = pooled.page_keys(list(range(40)), 16)
    b = pooled.page_keys(list(range(32)) + [99] * 8, 16)
    c = pooled.page_keys([7] + list(range(1, 40)), 16)
    assert len(a) == 2 and a == b and a[0] != c[0] and a[1] != c[1]
    assert pooled.page_keys(list(range(40)), 16, b"other-model")[0] != a[0]
    same_second_page = pooled.page_keys([0] * 16 + list(range(16, 32)), 16)
    assert same_second_page[1] != a[1]                      # a page's key covers everything before it


def test_ssd_ring_overwrites_oldest_and_never_returns_wrong_bytes(tmp_path):
    t = pooled.SsdTier(str(tmp_path), chunk_bytes=64, chunks=4)
    keys = [bytes([i]) * 32 for i in range(6)]
    for i, k in enumerate(keys):
        t.put(k, bytes([i]) * 64)
    assert [t.get(k) is not None for k in keys] == [False, False, True, True, True, True]
    assert t.get(keys[5]) == bytes([5]) * 64 and t.probe(keys[2:]) == 4 and t.probe(keys) == 0
    # a chunk damaged on disk is a miss
    import os
    os.pwrite(t.fd, b"\xff" * 8, t.index[keys[4]] * t.chunk + t.HEADER)
    assert t.get(keys[4]) is None and t.corrupt == 1
    with pytest.raises(ValueError):
        t.put(b"x" * 32, b"short")
    t.close()


@pytest.mark.parametrize("kind", ["memory", "ssd"])
def test_second_engine_serves_from_the_tier(tmp_path, kind):
    doc = toy_int.build_manifest(False)
    rts = [CpuRuntime(doc, tokens=16 * 30) for _ in range(2)]
    page_bytes = pooled.PagedStates(rts[0]).page_bytes
    tier = pooled.MemoryTier(64) if kind == "memory" else pooled.SsdTier(str(tmp_path), page_bytes, 64)
    scheds = [Scheduler(Engine(rt), chunk=32, max_seqs=2, pooled=pooled.PooledCache(rt, tier)) for rt in rts]
    rng = random.Random(4)
    base = [rng.randrange(256) for _ in range(75)]

    def run(s, prompt, rid):
        r = Request(id=rid, prompt=prompt, max_tokens=6, stop_ids=(toy_int.EOS,))
        s.submit(r)
        s.run_until_idle(300)
        assert [t for t in r.out if t != toy_int.EOS] == toy_int.generate(prompt, 6)
        return r

    run(scheds[0], base, "a")
    assert scheds[0].pooled.put_pages >= 4
    r = run(scheds[1], base[:70] + [1, 2, 3], "b")           # engine 1 never saw this prefix: it comes from the tier
    assert scheds[1].stats.pooled_hit_tokens == 64 and r.cached == 64 and scheds[1].stats.prefix_hits == 0
    assert scheds[1].stats.prefill_tokens == len(r.prompt) - 64
    run(scheds[1], base[:20], "c")                            # now the local prefix cache has it: the tier is not asked for more
    assert scheds[1].stats.pooled_hit_tokens == 64 and scheds[1].stats.prefix_hit_tokens == 16
