"""The pipeline timeline: `pp item` lines of the stages -> per-stage wait / held / period, and a Gantt row per stage."""
import dataclasses

from kern_b200.serve import pp_timeline as T


def lines(stage, items):
    return "\n".join(f"12:00:00.000 DEBUG pp item stage={stage} item={k} rows=16 issued_us={i} done_us={d}" for k, (i, d) in enumerate(items))


def test_wait_held_and_period_per_stage():
    # stage 0 works 100 us per item back to back; stage 1 takes 150 us, so it is the bottleneck and never waits after the first
    s0 = lines(0, [(0, 100), (5, 200), (10, 300), (15, 400)])
    s1 = lines(1, [(2, 250), (6, 400), (11, 550), (16, 700)])
    issued, done, rows = T.parse([s0, s1, "noise\n"])
    assert rows[3] == 16 and done[1][2] == 550
    tl = T.timeline(issued, done)
    assert [r["start"] for r in tl[0]] == [0, 100, 200, 300] and [r["held"] for r in tl[0]] == [100, 100, 100, 100]
    # stage 1 starts item k when its upstream is done with k and it is done with k - 1
    assert [r["start"] for r in tl[1]] == [100, 250, 400, 550] and [r["wait"] for r in tl[1]] == [0, 0, 0, 0]
    sm = {r["stage"]: r for r in T.summary(tl)}
    assert sm[0]["period_us_p50"] == 100 and sm[1]["period_us_p50"] == 150 and sm[1]["held_us_p50"] == 150 and sm[1]["busy"] == 1.0
    # a clock 1000 us ahead on stage 1 is taken out by --skew
    ahead = lines(1, [(1002, 1250), (1006, 1400), (1011, 1550), (1016, 1700)])
    issued2, done2, _ = T.parse([s0, ahead])
    assert T.summary(T.timeline(issued2, done2, {1: -1000})) == T.summary(tl)
    g = T.gantt(tl, width=70)
    assert len(g) == 3 and g[0].startswith("stage  0 |#") and g[1].count("#") > g[0].count("#") and g[1].startswith("stage  1 |.")
    assert T.timeline(issued, done, first=1, last=2)[0][0]["item"] == 1 and len(T.timeline(issued, done, first=1, last=2)[1]) == 2


def test_stages_of_a_real_pipeline_stamp_their_items():
    """Two stages in one process (the host-memory executor): every item run by a stage leaves a stamp, and the tool reads
    the same numbers back from the log lines."""
    import logging

    import torch

    from kern_b200.cpu import CpuRuntime
    from kern_b200.models import dense
    from kern_b200.serve import pp_ranks

    cfg = dataclasses.replace(dense.TOY, layers=2, name="toy2")
    doc = dense.build_manifest(cfg)
    rt = CpuRuntime(doc, weights=dense.random_weights(cfg, seed=0, std=0.05), tokens=cfg.page_size * 8)
    rt.once()
    records = []
    handler = logging.Handler()
    handler.emit = lambda rec: records.append(rec.getMessage())
    lg = logging.getLogger("kern.serve")
    lg.addHandler(handler)
    old = lg.level
    lg.setLevel(logging.DEBUG)
    try:
        stage = pp_ranks.Stage(rt, [doc], 0)
        from kern_b200.engine import Engine

        eng = Engine(rt)
        # items as the head would announce them: drive the stage through its own run()
        proto = rt.protocol
        from kern_b200 import fills

        lease = eng.pool.lease(40)
        for k, toks in enumerate(([3, 4, 5, 6, 7], [9])):
            e = fills.Entry(length=0 if k == 0 else 5, new=toks, pages=lease.pages, slot=lease.slot,
                            slots=lease.slots_of(0 if k == 0 else 5, (0 if k == 0 else 5) + len(toks)), sampling=fills.Sampling())
            call = fills.build(proto, rt.page_unit, [e])
            item = pp_ranks.Item(k=k, program=call.program, vars=dict(call.vars),
                                 columns={n: [dt, col.tolist()] for n, (dt, col) in call.columns.items()}, emits=call.forward["emits"],
                                 groups=call.groups, real=1, width=1)
            stage.run(item)
    finally:
        lg.removeHandler(handler)
        lg.setLevel(old)
    assert [t[0] for t in stage.timeline] == [0, 1] and all(t[3] >= t[2] for t in stage.timeline)
    issued, done, rows = T.parse(records)
    assert done[0][1] == stage.timeline[1][3] and rows[0] == 5 and rows[1] == 1
