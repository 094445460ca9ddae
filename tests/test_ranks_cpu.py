"""Multi-rank serving on CPU: rank executors (threads over real TCP sockets, one CPU runtime each), the head's
per-rank pool accounting, lockstep fan-out, and the same scheduler on top; wire framing; Layout; watch."""
import socket
import threading
import time

import pytest
import torch

from kern_b200.cpu import CpuRuntime
from kern_b200.engine import Engine
from kern_b200.models import dense, hybrid
from kern_b200.serve import executor, ranks, wire
from kern_b200.serve.scheduler import Request, Scheduler
from kern_b200.serve.watch import Watch


def test_wire_roundtrip_and_clean_close():
    l = wire.listen()
    got = []

    def srv():
        s = wire.accept(l)
        while (m := wire.recv(s)) is not None:
            got.append(m)
            wire.send(s, {"echo": m})
        s.close()

    t = threading.Thread(target=srv)
    t.start()
    c = wire.connect(l.getsockname())
    msg = {"a": [1, 2, 3], "blob": b"\x00\x01\xff", "nested": {"x": 1.5}}
    wire.send(c, msg)
    assert wire.recv(c) == {"echo": msg}
    wire.send(c, {})
    assert wire.recv(c) == {"echo": {}}
    c.close()
    t.join(5)
    assert got == [msg, {}]


@pytest.mark.parametrize("total,t", [(0, 2), (1, 4), (7, 2), (8, 4), (13, 8)])
def test_layout_own_rows_first(total, t):
    lay = ranks.Layout(total, t)
    assert sum(lay.lens) == total and max(lay.lens) - min(lay.lens) <= 1
    for m in range(t):
        order, blocks = lay.order(m), lay.blocks(m)
        assert sorted(order) == list(range(total))
        assert order[:lay.lens[m]] == list(range(lay.starts[m], lay.starts[m] + lay.lens[m]))
        assert blocks[0] == 0 and blocks[-1] == total and blocks[1] == lay.lens[m]


def _group(cfg, build, weights, world, slots=0):
    doc = build(cfg)          # every member holds the whole model: the head-side logic is what is under test
    made = {}

    def maker(q):
        def make():
            rt = CpuRuntime(doc, weights=weights, tokens=cfg.page_size * 24, slots=slots, topology={"tp": (q, world)})
            rt.offer = lambda: {}
            rt.connect = lambda g, offers: made.setdefault(q, len(offers))
            return rt
        return make

    ex, threads = executor.spawn_threads(world, maker, {"tp": world}, timeout=20)
    probe = CpuRuntime(doc, tokens=16)
    eng = ranks.GroupEngine(ex, probe.protocol, ex.hellos[0]["unit"], tp=world)
    return ex, eng, made


def test_group_scheduler_matches_single_engine():
    cfg = dense.TOY
    w = dense.random_weights(cfg, seed=1, std=0.08)
    ex, geng, made = _group(cfg, dense.build_manifest, w, world=2)
    assert made == {0: 2, 1: 2}
    rt = CpuRuntime(dense.build_manifest(cfg), weights=w, tokens=cfg.page_size * 24)
    rt.once()
    torch.manual_seed(0)
    prompts = [torch.randint(1, cfg.vocab, (n,)).tolist() for n in (9, 20, 5, 9)]
    prompts[3] = prompts[0][:]                      # a repeat: served from the prefix cache on both
    outs = []
    for engine in (Engine(rt), geng):
        sch = Scheduler(engine, chunk=16, max_seqs=2)
        reqs = [Request(id=str(i), prompt=p, max_tokens=6) for i, p in enumerate(prompts)]
        for r in reqs:
            sch.submit(r)
        for _ in range(200):
            if sch.idle():
                break
            sch.step()
        assert sch.idle()
        outs.append(([r.out for r in reqs], sch.stats.prefix_hits))
    assert outs[0] == outs[1]
    assert all(len(o) == 6 for o in outs[0][0])
    # nothing leaked on any rank: all pages are free or held by kept prefixes that can be evicted
    ex.close()


def test_group_engine_stateful_slots_and_copies():
    cfg = hybrid.TOY_HYBRID
    w = hybrid.random_weights(cfg, seed=3, std=0.08)
    ex, geng, _ = _group(cfg, hybrid.build_manifest, w, world=2, slots=6)
    rt = CpuRuntime(hybrid.build_manifest(cfg), weights=w, tokens=cfg.page_size * 24, slots=6)
    rt.once()
    single = Engine(rt)
    torch.manual_seed(5)
    prompt = torch.randint(1, cfg.vocab, (19,)).tolist()
    res = []
    for engine in (single, geng):
        s = engine.open(40)
        t = engine.step([(s, prompt)])[0]
        ck, copies = engine.pool.checkpoint(s.lease, 19)
        engine.rt.run_copies(copies)
        out = [t[0]]
        for _ in range(3):
            out.append(engine.step([(s, [out[-1]])])[0][0])
        lease, copies = engine.pool.restore(ck, 19, 40)
        engine.rt.run_copies(copies)
        from kern_b200.engine import Sequence
        r = Sequence(lease=lease, length=19)
        again = [t[0]]
        for _ in range(3):
            again.append(engine.step([(r, [again[-1]])])[0][0])
        assert again == out
        res.append(out)
    assert res[0] == res[1]
    ex.close()


def test_all_or_nothing_lease_over_members():
    p = CpuRuntime(dense.build_manifest(dense.TOY), tokens=16).protocol
    rk = ranks.Ranks(p, 16, pages=[4, 2], slots=[0, 0], tp=2)     # member 1 is smaller
    from kern_b200 import _native
    with pytest.raises(_native.Denied):
        rk.lease(0, 16 * 3)
    assert rk.pools[0].free_pages == 2 and rk.pools[1].free_pages == 2      # the group's smallest geometry
    l = rk.lease(0, 16 * 2)
    assert l.members[0].pages == l.members[1].pages
    assert rk.pools[0].free_pages == 0 and rk.pools[1].free_pages == 0
    l.release()
    assert rk.pools[0].free_pages == 2 and rk.pools[1].free_pages == 2


def test_watch_reports_a_closed_peer():
    l = wire.listen()
    lost = []
    w = Watch(on_lost=lost.append, interval=0.02)
    c = wire.connect(l.getsockname())
    s = wire.accept(l)
    w.add(s, "rank 3")
    time.sleep(0.1)
    assert lost == []
    c.close()
    for _ in range(100):
        if lost:
            break
        time.sleep(0.02)
    w.stop()
    assert lost == ["rank 3"]


def test_a_rank_that_cannot_start_fails_the_head_fast():
    def maker(q):
        def make():
            if q == 1:
                raise ValueError("no such checkpoint")
            rt = CpuRuntime(dense.build_manifest(dense.TOY), tokens=64)
            rt.offer = lambda: {}
            return rt
        return make

    with pytest.raises(RuntimeError, match="rank 1 could not start"):
        executor.spawn_threads(2, maker, {"tp": 2}, timeout=20)


def test_dp_tier_places_by_prefix_then_backlog_and_answers_exactly():
    import random

    from kern_b200.models import toy_int
    from kern_b200.serve.dp import DpTier

    doc = toy_int.build_manifest(False)

    def maker(q):
        def make():
            rt = CpuRuntime(doc, tokens=16 * 40)
            rt.offer = lambda: {}
            rt.connect = lambda g, offers: None
            return rt
        return make

    ex, _ = executor.spawn_threads(4, maker, {"tp": 1}, timeout=20)
    probe = CpuRuntime(doc, tokens=16)
    tier = DpTier(ex, probe.protocol, ex.hellos[0]["unit"], tp=1, chunk=32, max_seqs=3, patience=2)
    rng = random.Random(0)
    base = [rng.randrange(256) for _ in range(64)]
    first = Request(id="a", prompt=base[:48], max_tokens=5, stop_ids=(toy_int.EOS,))
    home = tier.submit(first)
    while not tier.idle():
        tier.step()
    # a prompt sharing the prefix goes where the prefix lives; strangers spread over the least loaded replicas
    again = Request(id="b", prompt=base[:48] + [3, 4, 5], max_tokens=5, stop_ids=(toy_int.EOS,))
    assert tier.submit(again) == home
    others = [Request(id=f"o{i}", prompt=[rng.randrange(256) for _ in range(20)], max_tokens=5, stop_ids=(toy_int.EOS,)) for i in range(6)]
    spots = [tier.submit(r) for r in others]
    assert len(set(spots)) == 4 and max(spots.count(g) for g in range(4)) <= 2
    # patience: when the home replica is far busier than the rest, the hit is given up
    for i in range(4):
        tier.scheds[home].submit(Request(id=f"x{i}", prompt=[1, 2, 3], max_tokens=2))
    late = Request(id="c", prompt=base[:48] + [9], max_tokens=5, stop_ids=(toy_int.EOS,))
    assert tier.submit(late) != home
    for _ in range(500):
        if tier.idle():
            break
        tier.step()
    assert tier.idle()
    for r in [first, again, late] + others:
        assert [t for t in r.out if t != toy_int.EOS] == toy_int.generate(r.prompt, 5), r.id
    assert tier.scheds[home].stats.prefix_hits >= 1
    ex.close()
